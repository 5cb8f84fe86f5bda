"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.  Host logic only; it sees tokens, pages and
slots and is tested without a GPU against a fake cache and step.

What it keeps of the reference: FIFO admission from a bounded waiting queue whose
``submit`` refuses when full (src/scheduler/scheduler.cpp:7-21, ``max_waiting`` 256
src/runtime/engine.h:25-67), prompts consumed in chunks of ``prefill_chunk``
(src/runtime/worker.cpp:375-383), the first token sampled from the last chunk's
last position (:404-446), EOS → "stop" without emitting the token, ``max_tokens``
→ "length", the cancel flag polled at step boundaries → "cancel"
(:45-58,541-553).  What is its own: one flat step that mixes decode tokens and
prompt portions under ``token_budget`` (the reference runs them back to back and
admits nothing while a prefill is pending, :231-241), and a decision for when
pages run out, which cannot happen in the reference (its cache is unbounded):

* at admission: the request stays in ``waiting`` until its next portion fits;
* in flight: the most recently admitted running request is preempted — its pages
  and slot are given back and it returns to the FRONT of ``waiting`` with
  everything generated so far kept, to be recomputed as a prompt; its sampling
  stream continues where it was because draws are indexed by output position;
* a request that cannot fit even alone in an empty pool ends with "error".
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Tuple

from ..cache.pages import OutOfSlots
from .request import FINISH_CANCEL, FINISH_ERROR, FINISH_LENGTH, FINISH_STOP, Request


@dataclass
class SchedulerConfig:
    max_running: int = 64          # live requests (also the number of state slots)
    max_waiting: int = 256         # src/runtime/engine.h: max_waiting
    token_budget: int = 2048       # most tokens one step runs
    prefill_chunk: int = 512       # most prompt tokens of one request in one step


@dataclass
class PlannedEntry:
    request: Request
    start: int                     # index into request.all_ids of the first token fed
    count: int
    samples: bool                  # the step's last token of this entry yields the next token


@dataclass
class SchedulerMetrics:
    steps: int = 0
    decode_tokens: int = 0
    prompt_tokens: int = 0
    completed: int = 0
    preemptions: int = 0
    peak_running: int = 0


class Scheduler:
    def __init__(self, cache, config: Optional[SchedulerConfig] = None):
        self.cache = cache
        self.cfg = config or SchedulerConfig()
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self.metrics = SchedulerMetrics()
        self._admitted = 0

    # ------------------------------------------------------------------ queue
    def submit(self, req: Request) -> bool:
        """False (and the request is not queued) when ``max_waiting`` are waiting
        (src/scheduler/scheduler.cpp:10-13)."""
        if len(self.waiting) >= self.cfg.max_waiting:
            return False
        if not req.prompt_ids:
            self._finish(req, FINISH_ERROR, "empty prompt")
            return True
        if req.max_tokens <= 0:
            self._finish(req, FINISH_LENGTH)
            return True
        self.waiting.append(req)
        return True

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ------------------------------------------------------------------ planning
    def _pages_fit(self, extra: List[int], need: List[int]) -> bool:
        free = self.cache.free_pages()
        return all(extra[g] + need[g] <= free[g] for g in range(len(free)))

    def plan(self) -> List[PlannedEntry]:
        """Decide the next step.  Decoding requests come first (one token each),
        then portions of prompts of running requests, oldest first, then new
        admissions, all within the token budget and the free pages."""
        self._drop_cancelled()
        cfg = self.cfg
        n_groups = len(self.cache.free_pages())
        preempted = False

        while True:
            entries: List[PlannedEntry] = []
            budget = cfg.token_budget
            taken = [0] * n_groups
            ok = True
            # running requests in admission order: decode tokens first
            decoders = [r for r in self.running if r.output_ids and r.computed == r.n_tokens - 1]
            in_decode = {id(r) for r in decoders}
            prefills = [r for r in self.running if id(r) not in in_decode]
            for r in decoders:
                need = self.cache.pages_needed(r.seq, 1)
                if budget < 1 or not self._pages_fit(taken, need):
                    ok = False
                    break
                taken = [a + b for a, b in zip(taken, need)]
                budget -= 1
                entries.append(PlannedEntry(r, r.computed, 1, True))
            if ok:
                for r in prefills:
                    left = r.n_tokens - r.computed
                    n = min(left, cfg.prefill_chunk, budget)
                    if n <= 0:
                        continue
                    need = self.cache.pages_needed(r.seq, n)
                    if not self._pages_fit(taken, need):
                        # shrink the portion to what fits; nothing at all is fine (it waits)
                        n = self._largest_fit(r, n, taken)
                        if n <= 0:
                            continue
                        need = self.cache.pages_needed(r.seq, n)
                    taken = [a + b for a, b in zip(taken, need)]
                    budget -= n
                    entries.append(PlannedEntry(r, r.computed, n, r.computed + n == r.n_tokens))
            if ok and (entries or not self.running):
                break
            if ok and not entries:
                # running requests exist but none can move: every one waits for pages
                ok = False
            if not ok:
                what = self._preempt_one()
                if what is None:
                    break
                preempted = preempted or what == "requeued"
        # admissions (none in a step that had to preempt: the pages just freed are
        # for the requests that were short of them)
        while not preempted and self.waiting and len(self.running) < cfg.max_running and budget > 0:
            r = self.waiting[0]
            if r.cancelled:
                self.waiting.popleft()
                self._finish(r, FINISH_CANCEL)
                continue
            total_pages = self.cache.pages_for_tokens(r.n_tokens + 1)
            if any(t > cap for t, cap in zip(total_pages, self.cache.total_pages())):
                self.waiting.popleft()
                self._finish(r, FINISH_ERROR,
                             f"request needs {max(total_pages)} pages, the pool has {min(self.cache.total_pages())}")
                continue
            n = min(r.n_tokens, cfg.prefill_chunk, budget)
            need = self.cache.pages_for_tokens(n)
            if not self._pages_fit(taken, need):
                break                                   # stays in waiting until pages are free
            try:
                r.seq = self.cache.open_sequence()
            except OutOfSlots:
                break
            self.waiting.popleft()
            r.computed = 0
            r.admit_order = self._admitted
            self._admitted += 1
            self.running.append(r)
            taken = [a + b for a, b in zip(taken, need)]
            budget -= n
            entries.append(PlannedEntry(r, 0, n, n == r.n_tokens))
        self.metrics.peak_running = max(self.metrics.peak_running, len(self.running))
        return entries

    def _largest_fit(self, r: Request, n: int, taken: List[int]) -> int:
        free = self.cache.free_pages()
        room = min(free[g] - taken[g] for g in range(len(free))) if free else 1 << 30
        if room < 0:
            return 0
        # tokens that fit in the request's last partly-filled page plus `room` whole pages
        ps = self.cache.page_size
        slack = (-r.seq.length) % ps
        return max(0, min(n, slack + room * ps))

    def _preempt_one(self) -> Optional[str]:
        """Give back the pages of the most recently admitted running request and
        put it at the front of the waiting queue ("requeued").  A request that
        runs alone and still cannot go on cannot fit at all: it ends with an
        error ("failed").  None if nothing runs."""
        if not self.running:
            return None
        victim = max(self.running, key=lambda r: r.admit_order)
        if len(self.running) == 1:
            self.running.remove(victim)
            self.cache.close(victim.seq)
            victim.seq = None
            self._finish(victim, FINISH_ERROR,
                         f"request of {victim.n_tokens} tokens does not fit in the cache pool even alone")
            return "failed"
        self.running.remove(victim)
        self.cache.close(victim.seq)
        victim.seq = None
        victim.computed = 0
        victim.preemptions += 1
        self.metrics.preemptions += 1
        self.waiting.appendleft(victim)
        return "requeued"

    def _drop_cancelled(self) -> None:
        for r in [r for r in self.running if r.cancelled]:
            self.running.remove(r)
            self.cache.close(r.seq)
            r.seq = None
            self._finish(r, FINISH_CANCEL)

    def continue_decoding(self, entries: List[PlannedEntry]) -> Optional[List[PlannedEntry]]:
        """``entries`` is a step that has been launched but not committed.  If the step after it
        is bound to be the same requests with one more token each, whatever the launched step
        samples short of an end-of-sequence token (every running request is in it and decoding,
        nobody waits who could be admitted, nobody is cancelled or would reach its length with the
        token on its way, and the pages are there), return that step; else None.  A request that
        does end with the token on its way leaves a row in the returned step whose result
        ``commit`` drops.  With every slot taken a waiting request cannot be admitted before a
        running one ends, so it does not stand in the way; if a running one meets its EOS with
        the token on its way, the waiting one gets in one step later than without this."""
        if self.waiting and len(self.running) < self.cfg.max_running:
            return None
        if len(entries) != len(self.running):
            return None
        n_groups = len(self.cache.free_pages())
        taken = [0] * n_groups
        nxt: List[PlannedEntry] = []
        for e, r in zip(entries, self.running):
            if e.request is not r or e.count != 1 or not e.samples or r.cancelled or r.finished:
                return None
            if not r.output_ids or len(r.output_ids) + 2 > r.max_tokens:
                return None
            need = self.cache.pages_needed(r.seq, 1)
            if not self._pages_fit(taken, need):
                return None
            taken = [a + b for a, b in zip(taken, need)]
            nxt.append(PlannedEntry(r, e.start + 1, 1, True))
        if len(nxt) > self.cfg.token_budget:
            return None
        return nxt

    # ------------------------------------------------------------------ after the step
    def commit(self, entries: List[PlannedEntry], sampled: List[int]) -> None:
        """``sampled`` holds one token for every entry with ``samples`` set, in order."""
        it = iter(sampled)
        self.metrics.steps += 1
        for e in entries:
            r = e.request
            if r.finished:                 # ended while this step was on its way: its row is dropped
                if e.samples:
                    next(it)
                continue
            r.computed += e.count
            if e.count == 1 and r.output_ids and e.start >= len(r.prompt_ids):
                self.metrics.decode_tokens += 1
            else:
                self.metrics.prompt_tokens += e.count
            if not e.samples:
                continue
            tok = int(next(it))
            if r.cancelled:
                self._retire(r, FINISH_CANCEL)
            elif tok in r.eos_ids:
                self._retire(r, FINISH_STOP)                 # EOS is not emitted
            else:
                r.emit(tok)
                if len(r.output_ids) >= r.max_tokens:
                    self._retire(r, FINISH_LENGTH)

    def _retire(self, r: Request, reason: str) -> None:
        self.running.remove(r)
        self.cache.close(r.seq)
        r.seq = None
        self._finish(r, reason)

    def _finish(self, r: Request, reason: str, error: Optional[str] = None) -> None:
        r.finish(reason, error)
        self.finished.append(r)
        self.metrics.completed += 1

    def fail_all(self, error: str) -> None:
        """The step itself failed: end every request with "error"."""
        for r in list(self.running):
            self.running.remove(r)
            if r.seq is not None and not r.seq.closed:
                self.cache.close(r.seq)
            r.seq = None
            self._finish(r, FINISH_ERROR, error)
        while self.waiting:
            self._finish(self.waiting.popleft(), FINISH_ERROR, error)
