"""A request: the unit of work between a caller and the engine
(src/scheduler/request.h:87-134: prompt ids, sampling options, ``max_tokens`` 64,
EOS ids, a cancel flag, a token queue that is closed when the request ends, and
``finish_reason``)."""
from __future__ import annotations

import queue
import threading
import time
from typing import List, Optional, Sequence

from ..sampling.params import SamplingParams

FINISH_STOP, FINISH_LENGTH, FINISH_CANCEL, FINISH_ERROR = "stop", "length", "cancel", "error"
_CLOSED = object()


class Request:
    _ids = 0
    _ids_lock = threading.Lock()

    def __init__(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None, max_tokens: int = 64,
                 eos_ids: Sequence[int] = ()):
        with Request._ids_lock:
            Request._ids += 1
            self.request_id = Request._ids
        self.prompt_ids: List[int] = [int(t) for t in prompt_ids]
        self.params = params or SamplingParams()
        self.max_tokens = int(max_tokens)
        self.eos_ids = tuple(int(e) for e in eos_ids)
        self.output_ids: List[int] = []
        self.finish_reason: Optional[str] = None
        self.error: Optional[str] = None
        self._cancelled = threading.Event()
        self._tokens: "queue.Queue" = queue.Queue()
        self.enqueue_time = time.perf_counter()
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        # engine-side state
        self.seq = None                    # SequenceCache while running
        self.computed = 0                  # tokens of `all_ids` whose keys/values are in the cache
        self.admit_order = -1
        self.preemptions = 0

    # ---- caller side
    def cancel(self) -> None:
        """Ask the engine to stop this request at the next step boundary
        (src/scheduler/request.h:122)."""
        self._cancelled.set()

    @property
    def cancelled(self) -> bool:
        return self._cancelled.is_set()

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def next(self, timeout: Optional[float] = None) -> Optional[int]:
        """Next generated token id; None once the request has ended and the queue
        is drained (the reference's ``mlxforge_request_next`` 0 / 1,
        src/capi/mlxforge.h:290-299).  Raises ``RuntimeError`` if the request
        ended with an error."""
        item = self._tokens.get(timeout=timeout)
        if item is _CLOSED:
            self._tokens.put(_CLOSED)
            if self.finish_reason == FINISH_ERROR:
                raise RuntimeError(self.error or "request failed")
            return None
        return item

    def __iter__(self):
        while True:
            t = self.next()
            if t is None:
                return
            yield t

    # ---- engine side
    @property
    def all_ids(self) -> List[int]:
        """Everything whose keys and values the cache must hold before the next
        token can be sampled: the prompt and what was generated so far."""
        return self.prompt_ids + self.output_ids

    @property
    def n_tokens(self) -> int:
        """len(all_ids) without building the list."""
        return len(self.prompt_ids) + len(self.output_ids)

    def tokens(self, start: int, count: int) -> List[int]:
        """all_ids[start:start + count] without building the whole list."""
        n_prompt = len(self.prompt_ids)
        end = start + count
        if end <= n_prompt:
            return self.prompt_ids[start:end]
        if start >= n_prompt:
            return self.output_ids[start - n_prompt:end - n_prompt]
        return self.prompt_ids[start:] + self.output_ids[:end - n_prompt]

    def emit(self, token: int) -> None:
        if self.first_token_time is None:
            self.first_token_time = time.perf_counter()
        self.output_ids.append(token)
        self._tokens.put(token)

    def finish(self, reason: str, error: Optional[str] = None) -> None:
        if self.finish_reason is None:
            self.finish_reason = reason
            self.error = error
            self.finish_time = time.perf_counter()
            self._tokens.put(_CLOSED)
