"""Binding of checkpoint tensors to the model's parts by tensor name.

The reference looks tensors up lazily, so a missing tensor is found only when
the forward first touches it (src/core/weights.cpp:82-88); here every name the
model declares is checked at load time and ONE error lists all missing tensors,
all unexpected ones and all wrong shapes.  Names are cleaned the way
src/core/weights.cpp:34-65 does for text models: rotary ``inv_freq`` buffers are
dropped and a ``language_model.`` wrapper prefix is stripped.

dtypes: 16-bit floats are kept as bfloat16 (float16 is converted), a tensor
stored in 32-bit stays 32-bit, integer tensors become int32.  What a part then
needs in the compute dtype (a matrix for a bfloat16 product) it converts for
itself when it is bound.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..parts.base import TensorSpec
from .safetensors_io import SafetensorsFile, model_files


class WeightError(ValueError):
    """One error for everything that is wrong with a checkpoint's tensors."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[Tuple[str, tuple, tuple]],
                 where: str = ""):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"weights: checkpoint {where} does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        super().__init__("\n".join(lines))


def clean_name(name: str) -> Optional[str]:
    """None for a tensor that is dropped (src/core/weights.cpp:34-65)."""
    if name.endswith("rotary_emb.inv_freq") or name.endswith(".inv_freq"):
        return None
    for prefix in ("model.language_model.", "language_model."):
        if name.startswith(prefix):
            rest = name[len(prefix):]
            return rest if rest.startswith(("model.", "lm_head.")) else "model." + rest
    return name


def check_names(specs: Dict[str, TensorSpec], found: Dict[str, tuple], where: str = "") -> None:
    """Compare declared tensors with the shapes found in the files."""
    missing = sorted(n for n, s in specs.items() if n not in found and not s.optional)
    unexpected = sorted(n for n in found if n not in specs)
    wrong = sorted((n, tuple(found[n]), tuple(s.shape)) for n, s in specs.items()
                   if n in found and tuple(found[n]) != tuple(s.shape))
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where)


def _to_torch(a: np.ndarray, tag: str, exact: bool = False) -> torch.Tensor:
    if tag == "BF16":
        return torch.from_numpy(a.copy()).view(torch.bfloat16)
    if tag == "F16":
        # float16 is no subset of bfloat16: the 32-bit path upcasts it exactly instead
        return torch.from_numpy(a.copy()).to(torch.float32 if exact else torch.bfloat16)
    if tag == "F32":
        return torch.from_numpy(a.copy())
    if tag == "F64":
        return torch.from_numpy(a.astype(np.float32))
    if tag in ("I64", "I32", "I16", "I8", "U8", "BOOL"):
        return torch.from_numpy(a.astype(np.int32))
    raise ValueError(tag)


def load_tensors(model_dir: str, specs: Dict[str, TensorSpec], device, exact: bool = False) -> Dict[str, torch.Tensor]:
    """Read every declared tensor of ``model_dir`` onto ``device``.  ``exact``: the
    caller computes in 32-bit, so nothing may lose bits on the way in."""
    files = [SafetensorsFile(p) for p in model_files(model_dir)]
    try:
        entries = {}
        for f in files:
            for e in f.entries:
                name = clean_name(e.name)
                if name is not None:
                    entries[name] = (f, e)
        check_names(specs, {n: e.shape for n, (_, e) in entries.items()}, f"'{model_dir}'")
        out: Dict[str, torch.Tensor] = {}
        for name in specs:
            if name not in entries:
                continue
            f, e = entries[name]
            out[name] = _to_torch(f.array(e), e.dtype, exact).to(device)
        return out
    finally:
        for f in files:
            f.close()
