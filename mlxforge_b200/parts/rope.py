"""Rotary position encoding with the reference's frequency schedules.

``freqs[i] = theta ** (2i / rotary_dim)`` in float32, then the llama3 or linear
rescaling (src/model/decoder_model.cpp:44-49, :65-70, :116-146); an angle is
``position / freqs[i]`` and pairs are half-split, ``(i, i + rotary_dim/2)``
(``traditional=false``, :220-228).  Keys are cached after rotation, values are
never rotated (:255-258).  The kernel that rotates also writes keys and values
into their pages, so the encoding owns that step of the mixer.

``"none"`` is the encoding without positions: the same kernel with nothing
rotated.
"""
from __future__ import annotations

import numpy as np
import torch

from ..config.model_config import RopeScaling, validate_rope_scaling
from ..csrc import ops
from .base import PositionEncoding, register_position

_TWO_PI = np.float32(6.283185307179586)   # src/model/decoder_model.cpp:21


def rope_frequencies(rotary_dim: int, theta: float, scaling) -> np.ndarray:
    """float32 [rotary_dim/2], computed in float32 as the reference does."""
    if rotary_dim <= 0 or rotary_dim % 2:
        raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
    idx = np.arange(0, rotary_dim, 2, dtype=np.float32)
    freqs = np.power(np.float32(theta), idx / np.float32(rotary_dim)).astype(np.float32)
    if scaling is None:
        return freqs
    rs = scaling if isinstance(scaling, RopeScaling) else RopeScaling.from_json(scaling)
    validate_rope_scaling(rs)
    if rs.rope_type == "default":
        return freqs
    factor = np.float32(rs.factor)
    if rs.rope_type == "linear":
        return (freqs * factor).astype(np.float32)
    low_ff, high_ff = np.float32(rs.low_freq_factor), np.float32(rs.high_freq_factor)
    old_ctx = np.float32(rs.original_max_position_embeddings)
    low_wl, high_wl = old_ctx / low_ff, old_ctx / high_ff
    wavelens = (_TWO_PI * freqs).astype(np.float32)
    scaled = np.where(wavelens > low_wl, freqs * factor, freqs).astype(np.float32)
    medium = (wavelens > high_wl) & (wavelens < low_wl)      # strict on both sides
    smooth = ((old_ctx / wavelens - low_ff) / (high_ff - low_ff)).astype(np.float32)
    denom = ((np.float32(1.0) - smooth) / factor + smooth).astype(np.float32)
    return np.where(medium, (scaled / denom).astype(np.float32), scaled).astype(np.float32)


@register_position("rope")
class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim exceeds head_dim")
        self.freqs_host = rope_frequencies(self.rotary_dim, float(params["theta"]), params.get("scaling"))
        self.freqs = torch.from_numpy(self.freqs_host).to(runtime.device)

    def rotate_and_store(self, qkv, batch, q_out, lane, n_heads, n_kv_heads, writes_cache):
        ops.rope_kv_write(qkv, batch.positions, batch.seq_of_token, batch.block_table(lane.group),
                          lane.page_size, self.freqs, q_out, lane.k, lane.v, n_heads, n_kv_heads,
                          self.head_dim, self.rotary_dim, writes_cache, self.rt.precise)


@register_position("none")
class NoPositions(PositionEncoding):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.head_dim = int(params["head_dim"])

    def rotate_and_store(self, qkv, batch, q_out, lane, n_heads, n_kv_heads, writes_cache):
        ops.rope_kv_write(qkv, batch.positions, batch.seq_of_token, batch.block_table(lane.group),
                          lane.page_size, None, q_out, lane.k, lane.v, n_heads, n_kv_heads,
                          self.head_dim, 0, writes_cache, self.rt.precise)
