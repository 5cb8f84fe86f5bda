"""Token selection for the rows of one step, on the device.

Order of operations as in the reference (src/sample/sampler.cpp:141-166):
penalties over the request's history (they apply to greedy too), then
``temperature <= 0`` → argmax, else ``logits / temperature``, top-k, top-p,
min-p, and a categorical draw.  The draw uses one uniform number per row from
``uniform_draw(seed, output index)``.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams, uniform_draw


class Sampler:
    def __init__(self, device, max_rows: int = 1024):
        self.device = torch.device(device)
        self._cap = 0
        self._host = None
        self._dev = None
        self._out = None
        self._ensure(max_rows)

    def _ensure(self, n: int) -> None:
        if n <= self._cap:
            return
        self._cap = max(n, 2 * self._cap)
        # per turn, like the tokens' host buffers: a launch writes its rows' temperatures and draws
        # here while the copy of the launch before it may not have run yet
        self._host = torch.empty((2, 2, self._cap), dtype=torch.float32, pin_memory=True)
        self._dev = torch.empty((2, self._cap), dtype=torch.float32, device=self.device)
        self._out = torch.empty(self._cap, dtype=torch.int32, device=self.device)
        # two host buffers taken in turn: one launch may be in flight while the one before is read
        self._out_host = [torch.empty(self._cap, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        # the word in which kernels with bounded waits say that one gave up travels with the tokens
        self._status = ops.kernel_status(self.device)
        self._status_host = [torch.zeros(1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [torch.cuda.Event() for _ in range(2)]
        self._turn = 0
        # the tokens go to the host on a stream of their own, so that the next step's first copy (its
        # metadata, host to device) does not queue behind this one
        self._out_stream = torch.cuda.Stream(device=self.device)
        self._sampled = torch.cuda.Event()
        self._last_copy = None            # event of the last copy out of self._out

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], indices: Sequence[int],
               histories: Sequence[Sequence[int]] = ()) -> List[int]:
        """One token for every row of ``logits`` [n, V] (float32, device).
        ``indices[r]`` is the output index of row r's request (it selects the
        draw); ``histories[r]`` the tokens its penalties look at."""
        return self.collect(self.launch(logits, params, indices, histories))

    @property
    def device_ids(self) -> torch.Tensor:
        """Where the last launch writes its tokens on the device (int32, a row each)."""
        return self._out

    def collect(self, handle) -> List[int]:
        """Wait for a launch and return its tokens."""
        if handle is None:
            return []
        turn, n = handle
        self._events[turn].synchronize()
        code = int(self._status_host[turn][0])
        if code:
            raise ops.kernel_gave_up(code, self.device)
        return self._out_host[turn][:n].tolist()

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], indices: Sequence[int],
               histories: Sequence[Sequence[int]] = ()):
        """Start the sampling of every row and the copy of the tokens to the host; nothing
        waits.  The handle goes to ``collect``; at most two launches may be uncollected."""
        n = logits.shape[0]
        if n == 0:
            return None
        self._ensure(n)
        if any(p.has_penalties for p in params):
            ops.apply_penalties(logits, params, histories)
        all_greedy = all(p.greedy for p in params)
        out = self._out[:n]
        main = torch.cuda.current_stream(self.device)
        if self._last_copy is not None:
            main.wait_event(self._last_copy)      # the copy before this one has read `out` (long ago)
        if all_greedy:
            ops.sample(logits, None, None, out)
        else:
            h = self._host[self._turn].numpy()
            for r, (p, i) in enumerate(zip(params, indices)):
                h[0, r] = 0.0 if p.greedy else p.temperature
                h[1, r] = uniform_draw(p.seed, i)
            self._dev[:, :n].copy_(self._host[self._turn][:, :n], non_blocking=True)
            if any(p.has_filters and not p.greedy for p in params):
                ops.filter_logits(logits, params)
            ops.sample(logits, self._dev[0, :n], self._dev[1, :n], out)
        turn = self._turn
        self._turn ^= 1
        self._sampled.record(main)
        with torch.cuda.stream(self._out_stream):
            self._out_stream.wait_event(self._sampled)
            self._out_host[turn][:n].copy_(out, non_blocking=True)
            self._status_host[turn].copy_(self._status, non_blocking=True)
            self._events[turn].record(self._out_stream)
        self._last_copy = self._events[turn]
        return (turn, n)
