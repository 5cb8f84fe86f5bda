"""Dense SiLU-gated feed-forward: ``down( silu(gate(x)) * up(x) )``
(src/model/decoder_model.cpp:277-282).  Gate and up are one matrix here, their
rows interleaved in groups of 8 (8 gate rows, then the matching 8 up rows) so a
kernel that owns 16 consecutive output rows holds both halves of a product;
when the intermediate size is no multiple of 8 the two are simply stacked."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.group = 8 if self.inter % 8 == 0 else self.inter
        self.w_gu = None
        self.w_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {
            self.prefix + "gate_proj.weight": TensorSpec((self.inter, self.hidden)),
            self.prefix + "up_proj.weight": TensorSpec((self.inter, self.hidden)),
            self.prefix + "down_proj.weight": TensorSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors) -> None:
        dt = self.rt.dtype
        g = tensors[self.prefix + "gate_proj.weight"].to(dt)
        u = tensors[self.prefix + "up_proj.weight"].to(dt)
        n = self.inter // self.group
        gu = torch.stack([g.view(n, self.group, self.hidden), u.view(n, self.group, self.hidden)], dim=1)
        self.w_gu = gu.reshape(2 * self.inter, self.hidden).contiguous()
        self.w_down = tensors[self.prefix + "down_proj.weight"].to(dt).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gu.numel() + self.w_down.numel()) * self.w_gu.element_size()

    def forward(self, x, batch):
        rt = self.rt
        T = x.shape[0]
        act = rt.linear_swiglu(x, self.w_gu, self.group, rt.buffer("ffn.act", (T, self.inter)))
        return rt.linear(act, self.w_down, rt.buffer("ffn.delta", (T, self.hidden)))
