"""Random-weights mode: write a model folder (``config.json`` +
``model.safetensors``) from a configuration and a seed.

The reference has no such mode (it always loads a checkpoint,
src/core/weights.cpp:208-265); its tests need the real Llama-3.2-1B files.  Here
every matrix is seeded normal with ``std`` (0.02 unless told otherwise) and
every norm weight is ``1 + N(0, norm_std)`` (exactly 1 when ``norm_std`` is 0).
Each tensor has its own generator stream keyed by (seed, position in the file),
so a tensor's values do not depend on the others' sizes.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import numpy as np

from ..config.model_config import ModelConfig
from ..config.registry import get_architecture
from .safetensors_io import write_safetensors_streaming


def float32_to_bfloat16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16, returned as uint16 words."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return rounded.astype(np.uint16)


def write_random_model(model_dir: str, config: ModelConfig, seed: int, *, dtype: str = "bfloat16",
                       std: float = 0.02, norm_std: float = 0.0) -> str:
    """Write ``model_dir/config.json`` and ``model_dir/model.safetensors``.

    ``dtype`` is the storage type of every tensor: ``"bfloat16"`` or ``"float32"``.
    Tensors are generated and written one at a time (torch's CPU generator, one
    stream per tensor seeded by ``(seed, position in the file)``).  Returns
    ``model_dir``.
    """
    import torch
    if dtype not in ("bfloat16", "float32"):
        raise ValueError(f"random weights: dtype must be 'bfloat16' or 'float32', got '{dtype}'")
    arch = get_architecture(config.architecture)
    if arch.random_tensors is None:
        raise ValueError(f"architecture '{config.architecture}' does not describe its tensors for random weights")
    os.makedirs(model_dir, exist_ok=True)
    tensors = list(arch.random_tensors(config))
    tag = "BF16" if dtype == "bfloat16" else "F32"

    def produce(i):
        name, shape, kind = tensors[i]
        g = torch.Generator().manual_seed((int(seed) * 1000003 + i) & (2**63 - 1))
        if kind == "norm":
            a = torch.ones(shape, dtype=torch.float32)
            if norm_std:
                a += torch.empty(shape, dtype=torch.float32).normal_(0.0, float(norm_std), generator=g)
        else:
            a = torch.empty(shape, dtype=torch.float32).normal_(0.0, float(std), generator=g)
        if dtype == "bfloat16":
            return a.to(torch.bfloat16).view(torch.int16).numpy()
        return a.numpy()

    write_safetensors_streaming(os.path.join(model_dir, "model.safetensors"),
                                [(n, tag, tuple(s)) for n, s, _ in tensors], produce)
    j = config.to_json()
    j["torch_dtype"] = dtype
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(j, f, indent=2)
    return model_dir
