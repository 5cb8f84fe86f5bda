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


def paged_attention(rt, batch, q, lane, out, n_heads: int, scale: float, window: int) -> None:
    """Attention of the step's queries over ``lane``; the kernel is chosen by dtype and by how
    many tokens each sequence brings.  bfloat16: the sequences that bring one token (the batch
    lays them out first: ``batch.n_decode``) go to the split-key decode kernel, the others to the
    prefill kernel.  float32: the generic kernel for all."""
    need = lane.need
    table = batch.block_table(lane.group)
    nd = batch.n_decode if q.dtype == torch.bfloat16 else 0
    if nd > 0:
        # contexts of very unequal length (the host knows them, the launcher does not): said to the
        # kernel's launcher, which then avoids dealing many items of unequal size out in turn
        lens = batch.ctx_len[:nd]
        unequal = nd >= 8 and max(lens) * nd > 1.3 * sum(lens)
        n_o, n_ml = ops.attention_decode_scratch(nd, n_heads, need.head_dim, batch.max_ctx)
        ops.attention_decode(q[:nd], lane.k, lane.v, out[:nd],
                             rt.buffer("attn.part_o", (n_o,), torch.float32),
                             rt.buffer("attn.part_ml", (n_ml,), torch.float32),
                             batch.positions[:nd], batch.seq_of_token[:nd], table, lane.page_size, n_heads,
                             need.n_kv_heads, need.head_dim, scale, window, batch.max_ctx, unequal)
    if nd < batch.n_tokens and q.dtype == torch.bfloat16:
        ops.attention_prefill(q, lane.k, lane.v, out, batch.seq_q_start[nd:], batch.seq_q_len[nd:],
                              batch.seq_ctx_len[nd:], nd, max(batch.q_len[nd:]), table, lane.page_size,
                              n_heads, need.n_kv_heads, need.head_dim, scale, window)
    elif nd < batch.n_tokens:
        ops.attention_generic(q[nd:], lane.k, lane.v, out[nd:], batch.positions[nd:],
                              batch.seq_of_token[nd:], table, lane.page_size, n_heads, need.n_kv_heads,
                              need.head_dim, scale, window)


@register_mixer("attention")
class AttentionMixer(Mixer):
    """``forward`` is four steps, each a method of its own, so that a variant (a norm on queries
    and keys, a gate on the output, another kernel) overrides one step and keeps the rest."""

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

    def project(self, x):
        """[T, H] -> queries, keys and values side by side, [T, (n_heads + 2 n_kv) * head_dim]."""
        T = x.shape[0]
        return self.rt.linear(x, self.w_qkv, self.rt.buffer("attn.qkv", (T, (self.n_heads + 2 * self.n_kv) * self.hd)))

    def encode_and_store(self, qkv, batch, cache, writes_cache: bool):
        """Position-encode queries and keys, append keys and values to the cache; returns the queries."""
        q = self.rt.buffer("attn.q", (qkv.shape[0], self.n_heads * self.hd))
        self.position.rotate_and_store(qkv, batch, q, cache, self.n_heads, self.n_kv, writes_cache)
        return q

    def attend(self, q, batch, cache):
        o = self.rt.buffer("attn.o", (q.shape[0], self.n_heads * self.hd))
        paged_attention(self.rt, batch, q, cache, o, self.n_heads, self.scale, self.window)
        return o

    def output(self, o):
        return self.rt.linear(o, self.w_o, self.rt.buffer("attn.delta", (o.shape[0], self.hidden)))

    def forward(self, x, batch, cache, writes_cache: bool = True):
        qkv = self.project(x)
        q = self.encode_and_store(qkv, batch, cache, writes_cache)
        return self.output(self.attend(q, batch, cache))
