"""The step function: one flat batch of (request, its next tokens) — portions of
prompts beside single decoded tokens, cut anywhere — run from the cache, with
logits returned only at the places that were asked for.

The reference never mixes the two kinds of work: a prefill chunk is a left-padded
rectangle ``(B, L)`` and a decode step is ``(bucket, 1)`` with dummy rows, run
back to back (src/runtime/worker.cpp:263-268,375-402,516-561;
doc/architecture.md:123-125), and it computes logits for every position and
slices afterwards (src/runtime/batching.cpp:46-49).  Here there are no padding
rows and no buckets: ``T`` tokens of ``R`` sequences, each token with its own
position and sequence index, and a block table per sequence and cache group.
"""
from __future__ import annotations

import gc
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import SequenceCache
from ..csrc import ops


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them
    whose logits are wanted."""

    seq: SequenceCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepBatch:
    """Device-side description of one step, as every part sees it.

    Tokens are laid out sequence after sequence; sequences that bring one token
    (decoding) come first, and ``n_decode`` says how many there are: a fact about the
    layout that a mixer may use (the attention mixer gives those rows to its decode
    kernel) or ignore.  ``positions[t]`` is the token's index in its sequence,
    ``seq_of_token[t]`` the row of its sequence in the block tables and in ``slots``."""

    def __init__(self):
        self.n_tokens = 0
        self.n_seqs = 0
        self.n_wanted = 0
        self.n_decode = 0                 # leading sequences (and tokens) that bring one token
        self.tokens = None                # [T] int32, device: where the step's token ids are read
        self.meta_tokens = None           # the copy of the host's token ids inside the metadata buffer
        self.positions = None
        self.seq_of_token = None
        self.want_rows = None
        self.slots = None                 # [R] int32, device: state slot of every sequence
        self.q_start: List[int] = []      # host copies, per sequence
        self.q_len: List[int] = []
        self.ctx_len: List[int] = []      # length after this step
        self.slot_ids: List[int] = []
        self.seq_q_start = None           # [R] device copies of the three lists
        self.seq_q_len = None
        self.seq_ctx_len = None
        self._block_tables: Dict[int, torch.Tensor] = {}
        self.max_ctx = 0

    def block_table(self, group: int) -> torch.Tensor:
        return self._block_tables[group]


class ModelRunner:
    """Owns the model, its cache manager and the step function."""

    def __init__(self, model, cache: CacheManager, runtime, cuda_graphs: bool = False):
        self.model = model
        self.cuda_graphs = cuda_graphs and model.graph_safe
        self.cache = cache
        self.rt = runtime
        self.vocab = model.spec.vocab_size
        self._pinned: Optional[torch.Tensor] = None
        self._meta: Optional[torch.Tensor] = None
        self._copied = torch.cuda.Event()
        self._copy_pending = False
        self.last_meta_bytes = 0
        self.steps = 0
        self._last: Optional[dict] = None     # the last decode-only step's metadata, for _advance
        self._plain_groups = all(g.need.window == 0 for g in cache.layout.paged)
        # CUDA graphs of decode-only steps, keyed by the shape of the step's metadata
        self._graphs: "OrderedDict[tuple, tuple]" = OrderedDict()
        self.max_graphs = 256
        self._warm: set = set()
        self.graph_replays = 0
        self._feed: Optional[torch.Tensor] = None     # the last device buffer a step's tokens were fed from

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None
             ) -> Optional[torch.Tensor]:
        """Run the entries as one batch.  Returns float32 logits ``[wanted, vocab]``
        on the device in the order of the entries and of their ``want`` lists
        (None if nothing is wanted).  The returned tensor is scratch that the
        next step overwrites.  On ``OutOfPages`` nothing has changed.

        ``device_tokens`` (int32, one per entry): the step's tokens are taken from there, on
        the device, in the order of the entries, and the entries' own token ids are ignored;
        every entry must then bring exactly one token.  This is how a step is launched
        before the host has seen what the step before it sampled."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        if device_tokens is not None and any(len(e.tokens) != 1 for e in entries):
            raise ValueError("device_tokens: every entry must bring exactly one token")
        seen = set()
        for e in entries:
            if e.seq.closed:
                raise RuntimeError(f"sequence {e.seq.seq_id} is closed")
            if e.seq.seq_id in seen:
                raise ValueError(f"sequence {e.seq.seq_id} appears twice in one step")
            seen.add(e.seq.seq_id)
            n = len(e.tokens)
            for w in e.want:
                if not (0 <= w < n):
                    raise IndexError(f"want index {w} is outside the {n} tokens of its entry")
            lo, hi = (0, 0) if device_tokens is not None else (min(e.tokens), max(e.tokens))
            if lo < 0 or hi >= self.vocab:
                raise IndexError(f"token id {lo if lo < 0 else hi} is outside the vocabulary [0, {self.vocab})")
        self.cache.reserve([(e.seq, len(e.tokens)) for e in entries])
        graphed = self.cuda_graphs and all(len(e.tokens) == 1 for e in entries)
        decode_only = all(len(e.tokens) == 1 for e in entries)
        batch = self._build(entries, pad_tables=decode_only)
        # one-token entries keep their order, so row r of device_tokens is entry r's token; the
        # batch object may be last step's (see _advance), so the choice is made afresh every step
        if device_tokens is not None:
            self._feed = device_tokens
            batch.tokens = device_tokens[:len(entries)]
        elif graphed and self._feed is not None and self._feed.numel() >= len(entries):
            # a caller that feeds some steps on the device gets ONE graph per shape, reading from the
            # feed buffer: the steps whose tokens come from the host copy them there first
            batch.tokens = self._feed[:len(entries)]
            batch.tokens.copy_(batch.meta_tokens, non_blocking=True)
        else:
            batch.tokens = batch.meta_tokens
        logits = self._forward_graphed(batch) if graphed else self.model.forward(batch, self.cache)
        for e in entries:
            self.cache.commit(e.seq, len(e.tokens))
        self.steps += 1
        return logits

    # ------------------------------------------------------------------ metadata
    def _forward_graphed(self, batch: StepBatch) -> Optional[torch.Tensor]:
        """Decode-only steps replay a CUDA graph: the kernels read tokens, positions and
        block tables from the metadata buffer, whose layout is fixed by the key, so a
        replay needs no host work beyond the one copy of that buffer.  The first step of
        a shape runs eagerly (it sizes the scratch), the second is captured."""
        from ..csrc import binding
        # the graph holds the address its tokens come from: the metadata buffer, or the sampler's
        # output when the step was launched before the host saw the tokens
        key = (batch.n_seqs, batch.n_wanted, tuple(t.shape[1] for t in batch._block_tables.values()),
               batch.tokens.data_ptr())
        entry = self._graphs.get(key)
        if entry is not None and entry[0] == (self.rt.generation, self._meta.data_ptr()):
            self._graphs.move_to_end(key)
            entry[1].replay()
            binding.count_launches(entry[3])
            self.graph_replays += 1
            return entry[2]
        if key not in self._warm:
            self._warm.add(key)
            return self.model.forward(batch, self.cache)
        self._graphs.pop(key, None)                  # a graph over buffers that have moved since
        while len(self._graphs) >= self.max_graphs:
            self._graphs.popitem(last=False)         # the shape that has not run for the longest time
        graph = torch.cuda.CUDAGraph()
        before = binding.launch_count()
        # Nothing may free device or pinned memory while the stream is capturing (the allocators
        # then touch events, which invalidates the capture): keep the collector out of it.
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                logits = self.model.forward(batch, self.cache)
        finally:
            if gc_was_on:
                gc.enable()
        nodes = binding.launch_count() - before
        binding.count_launches(-nodes)          # capturing launched nothing
        self._graphs[key] = ((self.rt.generation, self._meta.data_ptr()), graph, logits, nodes)
        graph.replay()
        binding.count_launches(nodes)
        self.graph_replays += 1
        return logits

    def _advance(self, entries: Sequence[StepEntry]) -> Optional[StepBatch]:
        """Steady decoding: the same sequences as in the last step, one token each, the same
        wanted rows, no window anywhere, tables still within their width.  The metadata then
        differs from the last step's only in the tokens, in positions and lengths (one more)
        and in the block-table entries of sequences that got a new page; it is patched in
        place in the pinned buffer instead of being built again.  None if this is not that case."""
        last = self._last
        if last is None or len(entries) != len(last["seq_ids"]):
            return None
        for e, sid, want in zip(entries, last["seq_ids"], last["wants"]):
            if e.seq.seq_id != sid or len(e.tokens) != 1 or tuple(e.want) != want:
                return None
        b: StepBatch = last["batch"]
        for g, width in enumerate(last["widths"]):
            for e in entries:
                if len(e.seq.blocks[g]) > width:
                    return None
        if self._copy_pending:
            self._copied.synchronize()
        v = last["host"]
        v["tokens"][:] = [e.tokens[0] for e in entries]
        v["positions"] += 1
        v["ctx_len"] += 1
        b.ctx_len = [c + 1 for c in b.ctx_len]
        for g, tab in enumerate(v["tables"]):
            counts = last["counts"][g]
            for row, e in enumerate(entries):
                n = len(e.seq.blocks[g])
                if n != counts[row]:
                    tab[row, counts[row]:n] = e.seq.row(g)[counts[row]:n]
                    counts[row] = n
        total = last["total"]
        self.last_meta_bytes = total * 4
        self._meta[:total].copy_(self._pinned[:total], non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        return b

    def _build(self, entries: Sequence[StepEntry], pad_tables: bool = False) -> StepBatch:
        if pad_tables and self._plain_groups:
            fast = self._advance(entries)
            if fast is not None:
                return fast
        self._last = None
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
        R = len(entries)
        T = sum(len(e.tokens) for e in entries)
        b = StepBatch()
        b.n_seqs, b.n_tokens = R, T
        tokens = np.empty(T, dtype=np.int32)
        positions = np.empty(T, dtype=np.int32)
        seq_of = np.empty(T, dtype=np.int32)
        start_of_entry = [0] * R
        t = 0
        for row, i in enumerate(order):
            e = entries[i]
            n = len(e.tokens)
            tokens[t:t + n] = e.tokens
            positions[t:t + n] = np.arange(e.seq.length, e.seq.length + n, dtype=np.int32)
            seq_of[t:t + n] = row
            start_of_entry[i] = t
            b.q_start.append(t)
            b.q_len.append(n)
            b.ctx_len.append(e.seq.length + n)
            b.slot_ids.append(e.seq.slot)
            if n == 1:
                b.n_decode += 1
            t += n
        b.max_ctx = max(b.ctx_len)
        want: List[int] = []
        for i, e in enumerate(entries):
            want.extend(start_of_entry[i] + w for w in e.want)
        b.n_wanted = len(want)

        tables = []
        for g in range(len(self.cache.pools)):
            width = max(1, max(len(entries[i].seq.blocks[g]) for i in order))
            if pad_tables:
                # decode-only steps: widths in powers of two from 16 up, so that one CUDA graph serves
                # every step whose tables fit, and so that an eager step and a replayed one size
                # (and split) their attention alike
                width = max(16, 1 << (width - 1).bit_length())
                b.max_ctx = max(b.max_ctx, width * self.cache.page_size)
            tab = np.full((R, width), -1, dtype=np.int32)
            for row, i in enumerate(order):
                blocks = entries[i].seq.row(g)
                tab[row, :blocks.shape[0]] = blocks
            tables.append(tab)

        parts = [tokens, positions, seq_of, np.asarray(want, dtype=np.int32),
                 np.asarray(b.slot_ids, dtype=np.int32), np.asarray(b.q_start, dtype=np.int32),
                 np.asarray(b.q_len, dtype=np.int32), np.asarray(b.ctx_len, dtype=np.int32)]
        parts += [tab.reshape(-1) for tab in tables]
        # every part starts on a 16-byte boundary
        offsets, total = [], 0
        for p in parts:
            offsets.append(total)
            total += (p.size + 3) // 4 * 4
        self._ensure_meta(total)
        if self._copy_pending:
            self._copied.synchronize()
        host = self._pinned.numpy()
        for p, off in zip(parts, offsets):
            host[off:off + p.size] = p
        self.last_meta_bytes = total * 4
        self._meta[:total].copy_(self._pinned[:total], non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        views = [self._meta[off:off + p.size] for p, off in zip(parts, offsets)]
        (b.tokens, b.positions, b.seq_of_token, b.want_rows, b.slots, b.seq_q_start, b.seq_q_len,
         b.seq_ctx_len) = views[:8]
        b.meta_tokens = b.tokens
        for g, tab in enumerate(tables):
            b._block_tables[g] = views[8 + g].view(tab.shape)
        if pad_tables and self._plain_groups:
            def hv(i):
                return host[offsets[i]:offsets[i] + parts[i].size]
            self._last = {
                "seq_ids": [e.seq.seq_id for e in entries], "wants": [tuple(e.want) for e in entries],
                "batch": b, "total": total, "widths": [tab.shape[1] for tab in tables],
                "counts": [[len(e.seq.blocks[g]) for e in entries] for g in range(len(tables))],
                "host": {"tokens": hv(0), "positions": hv(1), "ctx_len": hv(7),
                         "tables": [hv(8 + g).reshape(tab.shape) for g, tab in enumerate(tables)]},
            }
        return b

    def _ensure_meta(self, n: int) -> None:
        if self._pinned is None or self._pinned.numel() < n:
            if self._copy_pending:
                self._copied.synchronize()
                self._copy_pending = False
            cap = max(4096, 2 * n)
            self._last = None
            self._pinned = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._meta = torch.empty(cap, dtype=torch.int32, device=self.rt.device)
