"""The cache manager: device pools for every group of layers with the same
needs, a block table per request and group, and slots of fixed-size state.

Groups.  The model's mixers declare what they need (``PagedKV`` or
``FixedState``, see ``parts/base.py``).  Runs of layers with equal needs form a
group; each run is a *lane* of its group.  All lanes of a paged group share the
request's block table (page ``p`` of every lane belongs to the same request), a
group with another geometry or another window has pools, pages and block tables
of its own.  The reference shows the two kinds in its hybrid models: only the
full-attention layers grow keys and values (src/cache/kv_budget.cpp:14-20), the
linear layers hold fixed state per row (:25-39; src/cache/batch_kv_cache.h:132-153).

Pool layout of a paged lane: ``[page][kv_head][slot][head_dim]`` for keys and the
same for values, so one head's page is contiguous.

Pages are given back when a request is closed and, in a windowed group, as soon
as every position of a page is older than the window of the next query.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import FixedState, PagedKV
from .pages import OutOfPages, OutOfSlots, PagePool, SequenceCache, SlotPool


@dataclass(frozen=True)
class GroupLayout:
    need: object          # PagedKV | FixedState
    n_lanes: int


@dataclass(frozen=True)
class CacheLayout:
    """Groups of the model and, for every item of the schedule, which group and
    lane it uses (None for a run without cache)."""

    paged: Tuple[GroupLayout, ...]
    state: Tuple[GroupLayout, ...]
    item_lane: Tuple[Optional[Tuple[str, int, int]], ...]    # ("paged"|"state", group, lane)

    def bytes_per_token(self, elt_bytes: int) -> int:
        """Key+value bytes one token adds over all paged lanes
        (the reference's arithmetic: src/cache/kv_budget.cpp:50-60)."""
        return sum(2 * g.n_lanes * g.need.n_kv_heads * g.need.head_dim * elt_bytes for g in self.paged)

    def bytes_per_request(self) -> int:
        total = 0
        for g in self.state:
            n = getattr(torch, getattr(g.need, "dtype", "float32")).itemsize
            for s in g.need.shape:
                n *= s
            total += n * g.n_lanes
        return total


class KVLane:
    """One run's keys and values: two pools and the group's geometry."""

    __slots__ = ("k", "v", "group", "need", "page_size")

    def __init__(self, k, v, group: int, need: PagedKV, page_size: int):
        self.k, self.v, self.group, self.need, self.page_size = k, v, group, need, page_size

    def store(self, qkv, batch, q_out, n_heads: int, n_kv_heads: int, writes_cache: bool = True,
              precise: bool = False) -> None:
        """The lane's own write: from ``qkv`` ([T, (n_heads + 2 n_kv_heads) * head_dim], queries,
        keys and values side by side, already position-encoded) the keys and values of token ``t``
        go to page ``block_table[seq_of_token[t], p // page_size]``, slot ``p % page_size``
        (``p = batch.positions[t]``) and the queries to ``q_out``.  Nothing is rotated here, so a
        position encoding never has to know how the cache is laid out."""
        from ..csrc import ops
        ops.rope_kv_write(qkv, batch.positions, batch.seq_of_token, batch.block_table(self.group), self.page_size,
                          None, q_out, self.k, self.v, n_heads, n_kv_heads, self.need.head_dim, 0, writes_cache, precise)


class StateLane:
    """One run's fixed-size state: ``tensor[slot]`` is the request's state."""

    __slots__ = ("tensor", "group", "need")

    def __init__(self, tensor, group: int, need: FixedState):
        self.tensor, self.group, self.need = tensor, group, need


class CacheManager:
    def __init__(self, layout: CacheLayout, *, page_size: int, max_tokens: int, max_seqs: int,
                 dtype: torch.dtype, device: str = "cuda"):
        if page_size <= 0 or page_size % 16:
            raise ValueError(f"page_size must be a positive multiple of 16, got {page_size}")
        self.layout = layout
        self.page_size = page_size
        self.dtype = dtype
        self.device = device
        self.n_pages = (max_tokens + page_size - 1) // page_size
        self.max_seqs = max_seqs
        self.pools = [PagePool(self.n_pages) for _ in layout.paged]
        self.slots = SlotPool(max_seqs)
        self._next_id = 0
        self._live: Dict[int, SequenceCache] = {}
        self._k: List[torch.Tensor] = []
        self._v: List[torch.Tensor] = []
        for g in layout.paged:
            shape = (g.n_lanes, self.n_pages, g.need.n_kv_heads, page_size, g.need.head_dim)
            self._k.append(torch.zeros(shape, dtype=dtype, device=device))
            self._v.append(torch.zeros(shape, dtype=dtype, device=device))
        self._state = [torch.zeros((g.n_lanes, max_seqs) + tuple(g.need.shape),
                                   dtype=getattr(torch, getattr(g.need, "dtype", "float32")), device=device)
                       for g in layout.state]

    # ------------------------------------------------------------------ views for the model
    def lane(self, item: int):
        where = self.layout.item_lane[item]
        if where is None:
            return None
        kind, g, lane = where
        if kind == "paged":
            return KVLane(self._k[g][lane], self._v[g][lane], g, self.layout.paged[g].need, self.page_size)
        return StateLane(self._state[g][lane], g, self.layout.state[g].need)

    # ------------------------------------------------------------------ requests
    def open_sequence(self) -> SequenceCache:
        slot = self.slots.take()
        for st in self._state:
            st[:, slot].zero_()
        seq = SequenceCache(seq_id=self._next_id, slot=slot, blocks=[[] for _ in self.layout.paged],
                            block_rows=[np.full(16, -1, dtype=np.int32) for _ in self.layout.paged])
        self._next_id += 1
        self._live[seq.seq_id] = seq
        return seq

    def _first_needed_block(self, g: int, length: int) -> int:
        """First logical block that the query at position ``length`` can still see."""
        w = self.layout.paged[g].need.window
        if w <= 0:
            return 0
        return max(0, length - w + 1) // self.page_size

    def pages_needed(self, seq: SequenceCache, n_new: int) -> List[int]:
        """New pages per group to hold ``n_new`` more tokens."""
        out = []
        for g in range(len(self.pools)):
            have = len(seq.blocks[g])
            want = (seq.length + n_new + self.page_size - 1) // self.page_size
            out.append(max(0, want - have))
        return out

    def reserve(self, requests: Sequence[Tuple[SequenceCache, int]]) -> None:
        """Pages for every (request, number of new tokens) of one step, or
        ``OutOfPages`` with nothing taken."""
        need = [0] * len(self.pools)
        per = []
        for seq, n_new in requests:
            if seq.closed:
                raise RuntimeError(f"sequence {seq.seq_id} is closed")
            p = self.pages_needed(seq, n_new)
            per.append(p)
            for g, n in enumerate(p):
                need[g] += n
        for g, n in enumerate(need):
            if n > self.pools[g].n_free:
                raise OutOfPages(g, n, self.pools[g].n_free, self.pools[g].n_pages)
        for (seq, _), p in zip(requests, per):
            for g, n in enumerate(p):
                if n:
                    seq._extend(g, self.pools[g].take(n, g))

    def commit(self, seq: SequenceCache, n_new: int) -> None:
        """The step wrote ``n_new`` tokens: move the length on and give back pages
        that every later query's window has passed."""
        seq.length += n_new
        for g in range(len(self.pools)):
            first = self._first_needed_block(g, seq.length)
            blocks = seq.blocks[g]
            gone = [blocks[b] for b in range(min(first, len(blocks))) if blocks[b] >= 0]
            if gone:
                for b in range(min(first, len(blocks))):
                    blocks[b] = -1
                seq.block_rows[g][:min(first, len(blocks))] = -1
                self.pools[g].give_back(gone)

    def close(self, seq: SequenceCache) -> None:
        if seq.closed:
            raise RuntimeError(f"sequence {seq.seq_id} closed twice")
        for g, blocks in enumerate(seq.blocks):
            self.pools[g].give_back([p for p in blocks if p >= 0])
            seq.blocks[g] = []
        self.slots.give_back(seq.slot)
        seq.closed = True
        del self._live[seq.seq_id]

    # ------------------------------------------------------------------ accounting
    def free_pages(self) -> List[int]:
        return [p.n_free for p in self.pools]

    def total_pages(self) -> List[int]:
        return [p.n_pages for p in self.pools]

    def pages_for_tokens(self, n_tokens: int) -> List[int]:
        """Pages per group that a new request of ``n_tokens`` takes."""
        return [(n_tokens + self.page_size - 1) // self.page_size for _ in self.pools]

    def free_tokens(self) -> int:
        """Tokens that the tightest group can still take (whole pages)."""
        if not self.pools:
            return 1 << 60
        return min(p.n_free for p in self.pools) * self.page_size

    def check(self) -> None:
        """Every page is free or held by exactly one live request."""
        for g, pool in enumerate(self.pools):
            pool.check()
            seen = set()
            for seq in self._live.values():
                for p in seq.blocks[g]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise AssertionError(f"group {g}: page {p} is held twice")
                    seen.add(p)
            if len(seen) != pool.n_held:
                raise AssertionError(f"group {g}: {pool.n_held} pages held but live requests hold {len(seen)}")
