"""Grouped-query attention over the paged cache.

``q = x Wq^T, k = x Wk^T, v = x Wv^T`` (weights ``(out, in)``, no bias; head ``h``
is output rows ``[h*hd, (h+1)*hd)``), position encoding on q and k, keys and
values appended to the cache, ``softmax(q k^T * scale) v`` with the causal mask
aligned to the end of the keys, query head ``h`` reading KV head
``h // (n_heads / n_kv_heads)``, then the output projection
(src/model/decoder_model.cpp:234-275, :315-328; src/model/sdpa.cpp:27,44-46,71-95).
The three projections are one matrix here (stacked at load time), which changes
no number.  ``window`` > 0 limits every query to the last ``window`` keys.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import POSITIONS, Mixer, PagedKV, TensorSpec, build_part, register_mixer


@register_mixer("attention")
class AttentionMixer(Mixer):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.hd = int(p["head_dim"])
        self.scale = float(p["softmax_scale"])
        self.window = int(p.get("window", 0) or 0)
        if self.n_heads % self.n_kv:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if self.hd % 16 or not (16 <= self.hd <= 256):
            raise ValueError(f"attention: head_dim {self.hd} is not a multiple of 16 in [16, 256]")
        self.position = build_part(POSITIONS, p["position"], runtime)
        self.w_qkv = None
        self.w_o = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        q, kv = self.n_heads * self.hd, self.n_kv * self.hd
        specs = {
            self.prefix + "q_proj.weight": TensorSpec((q, self.hidden)),
            self.prefix + "k_proj.weight": TensorSpec((kv, self.hidden)),
            self.prefix + "v_proj.weight": TensorSpec((kv, self.hidden)),
            self.prefix + "o_proj.weight": TensorSpec((self.hidden, q)),
        }
        specs.update(self.position.tensor_specs())      # a position encoding may have tensors of its own
        return specs

    def bind(self, tensors) -> None:
        self.position.bind(tensors)
        dt = self.rt.dtype
        self.w_qkv = torch.cat([tensors[self.prefix + n + "_proj.weight"].to(dt) for n in ("q", "k", "v")],
                               dim=0).contiguous()
        self.w_o = tensors[self.prefix + "o_proj.weight"].to(dt).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()

    def cache_need(self):
        return PagedKV(self.n_kv, self.hd, self.window)

    def forward(self, x, batch, cache, writes_cache: bool = True):
        rt = self.rt
        T = x.shape[0]
        qkv = rt.linear(x, self.w_qkv, rt.buffer("attn.qkv", (T, (self.n_heads + 2 * self.n_kv) * self.hd)))
        q = rt.buffer("attn.q", (T, self.n_heads * self.hd))
        self.position.rotate_and_store(qkv, batch, q, cache, self.n_heads, self.n_kv, writes_cache)
        o = rt.buffer("attn.o", (T, self.n_heads * self.hd))
        batch.attention(q, cache, o, self.n_heads, self.scale, self.window)
        return rt.linear(o, self.w_o, rt.buffer("attn.delta", (T, self.hidden)))
