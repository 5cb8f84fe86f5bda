"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w`` over the last axis, the weight
multiplying directly (src/model/decoder_model.cpp:206-208).  The sum of squares,
the scaling and the residual sum it is fused with are 32-bit."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import Norm, TensorSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.prefix + "weight": TensorSpec((self.size,), role="vector")}

    def bind(self, tensors) -> None:
        self.weight = tensors[self.prefix + "weight"].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.size * 4

    def forward(self, x, out=None):
        return self.add_forward(x, None, out)

    def add_forward(self, residual, delta, out=None, rows=None):
        n = residual.shape[0] if rows is None else rows.shape[0]
        if out is None:
            out = self.rt.buffer("norm.out", (n, self.size))
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows)
        return out
