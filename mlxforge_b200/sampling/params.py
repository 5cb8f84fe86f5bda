"""Sampling options, with the reference's names, meanings and defaults
(src/sample/sampler.h:15-36), and the counter-based uniform draw.

The reference splits an MLX random key once per step (src/runtime/worker.cpp:416,465-466);
here draw ``i`` of a request is a pure function of ``(seed, i)``, so a stream
does not depend on batching and continues unchanged after a preemption.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0          # <= 0 (or not finite) => greedy argmax
    top_k: int = 0                    # <= 0 => disabled
    top_p: float = 1.0                # >= 1 => disabled
    min_p: float = 0.0                # <= 0 => disabled (keep prob >= min_p * max prob)
    repetition_penalty: float = 1.0   # 1 => disabled (divides positive / multiplies negative seen logits)
    frequency_penalty: float = 0.0    # 0 => disabled (subtracts penalty * count)
    presence_penalty: float = 0.0     # 0 => disabled (subtracts penalty if seen)
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0 and math.isfinite(self.temperature))

    @property
    def has_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                or self.presence_penalty != 0.0)

    @property
    def has_filters(self) -> bool:
        return self.top_k > 0 or self.top_p < 1.0 or self.min_p > 0.0


GREEDY = SamplingParams(temperature=0.0)


def uniform_draw(seed: int, index: int) -> float:
    """Uniform number in [0, 1) with 24 bits for output ``index`` of a request
    with ``seed``: a splitmix64 finaliser over the two."""
    z = (int(seed) * 0x9E3779B97F4A7C15 + (int(index) + 1) * 0xD1B54A32D192ED03) & _MASK
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)
