"""From a model folder to a runnable model: config.json chooses the architecture
through the registry, the architecture's builder turns the typed configuration
into a ``ModelSpec``, the spec is built from parts and the checkpoint's tensors
are bound by name (the reference's path: src/runtime/engine.cpp:116-187,
apps/mlxforge_cli.cpp:96-116)."""
from __future__ import annotations

from typing import Tuple

import torch

from ..config.model_config import apply_rope_scaling_override, read_config_json
from ..config.registry import config_from_json, get_architecture
from ..models.decoder import DecoderModel
from .runtime import Runtime

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got '{name}'") from None


def require_gpu() -> None:
    """The engine has no CPU path: say so instead of running something else."""
    if not torch.cuda.is_available():
        raise RuntimeError("mlxforge_b200 needs a CUDA device (built for sm_100a); none is visible. "
                           "There is no CPU fallback.")


def load_model(model_dir: str, dtype="bfloat16", device: str = "cuda",
               rope_scaling: str = None) -> Tuple[DecoderModel, object]:
    """``rope_scaling``: a JSON object that replaces the checkpoint's
    ``rope_scaling`` wholesale (src/core/config.cpp:282-300)."""
    require_gpu()
    from ..csrc.binding import library
    library()      # build or load the kernels now: fail before any weight is read
    j = read_config_json(model_dir)
    if rope_scaling:
        j = apply_rope_scaling_override(j, rope_scaling)
    config = config_from_json(j)
    arch = get_architecture(config.architecture)
    rt = Runtime(parse_dtype(dtype), device)
    model = DecoderModel(arch.build_spec(config), rt)
    model.load(model_dir)
    return model, config
