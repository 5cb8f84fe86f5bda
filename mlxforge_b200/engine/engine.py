"""The engine facade and its worker loop: the Python entry point.

Shape of the reference's surface (src/runtime/engine.h:25-117, src/capi/mlxforge.h:169-323):
an ``EngineConfig`` whose invalid combinations fail creation instead of falling
back, ``submit`` that returns a request handle, ``request.next()`` that yields
token ids until the request ends, ``cancel``, ``finish_reason``, ``metrics``,
``stop`` that completes in-flight requests.  It is token-id based (tokenizers
are out of scope) and in-process Python instead of a C ABI.

One loop iteration = one scheduler plan, one step of the model over a mixed
batch, one sampling call, one commit; the commit of a step happens in the
iteration after the one that launched it, and while every running request is
decoding the step after is launched first (see ``Engine.step``).
``Engine.step()`` runs an iteration on the caller's thread; ``Engine.start()``
runs the same loop on a worker thread, as the reference's single GPU thread
does (src/runtime/worker.cpp:196-280).
"""
from __future__ import annotations

import json
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..sampling.params import GREEDY, SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model, parse_dtype
from .request import FINISH_ERROR, Request
from .scheduler import PlannedEntry, Scheduler, SchedulerConfig
from .step import ModelRunner, StepEntry


class QueueFull(RuntimeError):
    pass


@dataclass
class EngineConfig:
    """Options of an engine.  Names follow the reference where it has them
    (``model_spec``, ``max_waiting``, ``kv_block_size``, ``kv_pool_bytes``,
    ``prefill_chunk``, ``skinny_mm``, ``rope_scaling``; src/runtime/engine.h:25-67)."""

    model_spec: str = ""
    dtype: str = "bfloat16"            # "bfloat16" | "float32"
    max_waiting: int = 256
    kv_block_size: int = 16            # tokens per cache page
    kv_pool_bytes: int = 1 << 30       # bytes of keys and values over all layers
    kv_pool_tokens: int = 0            # > 0: size the pool in tokens instead
    max_running: int = 64
    token_budget: int = 2048
    prefill_chunk: int = 512
    skinny_mm: bool = True             # few-row products by the skinny kernel
    cuda_graphs: bool = True           # replay decode-only steps from captured graphs
    pipeline: bool = True              # launch a decode step before the host has the tokens of the one before
    gemm: str = ""                     # many-row products: "auto" | "library" | "tcgen05" ("" = MLXFORGE_GEMM or auto)
    rope_scaling: str = ""             # JSON object replacing the checkpoint's rope_scaling

    def validate(self) -> None:
        if not self.model_spec:
            raise ValueError("EngineConfig: model_spec (a folder with config.json) is required")
        if self.kv_block_size <= 0 or self.kv_block_size % 16:
            raise ValueError(f"EngineConfig: kv_block_size must be a positive multiple of 16, got {self.kv_block_size}")
        if self.prefill_chunk <= 0 or self.token_budget <= 0:
            raise ValueError("EngineConfig: prefill_chunk and token_budget must be positive")
        if self.max_running <= 0 or self.max_waiting <= 0:
            raise ValueError("EngineConfig: max_running and max_waiting must be positive")
        if self.kv_pool_tokens <= 0 and self.kv_pool_bytes <= 0:
            raise ValueError("EngineConfig: give kv_pool_bytes or kv_pool_tokens")
        parse_dtype(self.dtype)


class Engine:
    def __init__(self, config: Optional[EngineConfig] = None, **kw):
        if config is None:
            config = EngineConfig(**kw)
        elif kw:
            raise TypeError("give either an EngineConfig or keyword options")
        config.validate()
        self.config = config
        dtype = parse_dtype(config.dtype)
        self.model, self.model_config = load_model(config.model_spec, dtype,
                                                   rope_scaling=config.rope_scaling or None)
        rt = self.model.rt
        rt.skinny_enabled = bool(config.skinny_mm)
        rt.reserve_rows = config.token_budget
        if config.gemm:
            if config.gemm not in ("auto", "library", "tcgen05"):
                raise ValueError(f"EngineConfig: gemm must be 'auto', 'library' or 'tcgen05', got '{config.gemm}'")
            rt.gemm_backend = config.gemm
        elt = 4 if dtype == torch.float32 else 2
        per_token = max(1, self.model.cache_layout.bytes_per_token(elt))
        tokens = config.kv_pool_tokens if config.kv_pool_tokens > 0 else config.kv_pool_bytes // per_token
        tokens = max(tokens, config.kv_block_size)
        self.cache = CacheManager(self.model.cache_layout, page_size=config.kv_block_size, max_tokens=tokens,
                                  max_seqs=config.max_running, dtype=dtype, device=str(rt.device))
        self._assemble(ModelRunner(self.model, self.cache, rt, cuda_graphs=config.cuda_graphs), Sampler(rt.device),
                       rt.device.index if rt.device.index is not None else torch.cuda.current_device())

    @classmethod
    def from_parts(cls, config: EngineConfig, model, cache, runner, sampler, device_index: int = 0) -> "Engine":
        """An engine around parts that already exist: ``model`` needs ``spec.vocab_size`` and
        ``spec.eos_token_ids``; ``runner.step(entries, device_tokens=None)`` returns what
        ``sampler.launch`` takes; ``sampler`` has ``launch``, ``collect`` and ``device_ids``.
        Nothing is loaded.  Tests drive the loop below with stand-ins this way."""
        self = cls.__new__(cls)
        self.config = config
        self.model, self.model_config, self.cache = model, None, cache
        self._assemble(runner, sampler, device_index)
        return self

    def _assemble(self, runner, sampler, device_index: int) -> None:
        config = self.config
        self.runner = runner
        self.scheduler = Scheduler(self.cache, SchedulerConfig(
            max_running=config.max_running, max_waiting=config.max_waiting,
            token_budget=config.token_budget, prefill_chunk=config.prefill_chunk))
        self.sampler = sampler
        self._lock = threading.Lock()
        self._wake = threading.Condition(self._lock)
        self._thread: Optional[threading.Thread] = None
        self._stop = False
        self._t_busy = 0.0
        # a launched step whose sampled tokens have not been collected: (entries, sampler handle)
        self._inflight = None
        self.pipeline = bool(config.pipeline)
        self.steps_ahead = 0              # steps launched before the tokens of the step before were known
        self._device_index = device_index

    # ------------------------------------------------------------------ submit
    @property
    def eos_token_ids(self):
        return tuple(self.model.spec.eos_token_ids)

    def submit_ids(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None,
                   max_tokens: int = 64, eos_ids: Optional[Sequence[int]] = None) -> Request:
        """Queue a request.  ``eos_ids`` None takes the model's; an empty list
        disables EOS (the reference's bench does that, apps/mlxforge_cli.cpp:319).
        Raises ``QueueFull`` when ``max_waiting`` requests are waiting."""
        vocab = self.model.spec.vocab_size
        for t in prompt_ids:
            if not (0 <= int(t) < vocab):
                raise ValueError(f"token id {t} is outside the vocabulary [0, {vocab})")
        req = Request(prompt_ids, params or SamplingParams(), max_tokens,
                      self.eos_token_ids if eos_ids is None else eos_ids)
        with self._wake:
            if not self.scheduler.submit(req):
                raise QueueFull(f"{self.config.max_waiting} requests are already waiting")
            self._wake.notify_all()
        return req

    # ------------------------------------------------------------------ the loop
    @property
    def idle(self) -> bool:
        """Nothing waiting, nothing running and no step on its way."""
        return self.scheduler.idle and self._inflight is None

    def step(self) -> int:
        """One iteration.  Returns the number of tokens it ran or committed (0 when there was
        nothing to do).

        A step is launched without waiting for it: its sampled tokens are collected by the
        NEXT call.  While every running request is decoding, that next call first launches the
        step after (its tokens are fed on the device from what the step on its way samples,
        ``Scheduler.continue_decoding`` says when that is sound) and only then collects, so the
        device goes from one step into the next while the host emits tokens and does its
        bookkeeping.  A request that ends with a token collected this way has a row in the step
        already launched; that row's result is dropped.  Requests with penalties need their
        history on the host before they sample: their steps are collected at once."""
        inflight = self._inflight
        if inflight is None:
            return self._launch_planned()
        entries, handle = inflight
        t0 = time.perf_counter()
        nxt, nxt_handle = None, None
        if self.pipeline:
            with self._lock:
                nxt = self.scheduler.continue_decoding(entries)
        try:
            if nxt is not None:
                try:
                    step_entries = [StepEntry(e.request.seq, [0], [0]) for e in nxt]
                    logits = self.runner.step(step_entries, device_tokens=self.sampler.device_ids)
                except OutOfPages:
                    nxt = None
                else:
                    rows = [e.request for e in nxt]
                    nxt_handle = self.sampler.launch(logits, [r.params for r in rows],
                                                     [len(r.output_ids) + 1 for r in rows])
                    self.steps_ahead += 1
            sampled = self.sampler.collect(handle)
        except Exception as exc:
            self._inflight = None
            with self._lock:
                self.scheduler.fail_all(f"{type(exc).__name__}: {exc}")
            raise
        with self._lock:
            self.scheduler.commit(entries, sampled)
        self._inflight = (nxt, nxt_handle) if nxt is not None else None
        self._t_busy += time.perf_counter() - t0
        return sum(e.count for e in entries)

    def _launch_planned(self) -> int:
        """Plan a step with the scheduler and launch it.  Its tokens are collected by the next
        call of ``step`` unless a request's penalties need them on the host first."""
        with self._lock:
            entries = self.scheduler.plan()
        if not entries:
            return 0
        t0 = time.perf_counter()
        try:
            step_entries = []
            for e in entries:
                ids = e.request.tokens(e.start, e.count)
                step_entries.append(StepEntry(e.request.seq, ids, [e.count - 1] if e.samples else []))
            logits = self.runner.step(step_entries)
            rows = [e.request for e in entries if e.samples]
            handle = None
            if logits is not None:
                handle = self.sampler.launch(logits, [r.params for r in rows], [len(r.output_ids) for r in rows],
                                             [r.all_ids if r.params.has_penalties else () for r in rows])
            if self.pipeline and not any(r.params.has_penalties for r in rows):
                self._inflight = (entries, handle)
                self._t_busy += time.perf_counter() - t0
                return sum(e.count for e in entries)
            sampled = self.sampler.collect(handle)
        except Exception as exc:    # the step failed: no request can go on
            with self._lock:
                self.scheduler.fail_all(f"{type(exc).__name__}: {exc}")
            raise
        with self._lock:
            self.scheduler.commit(entries, sampled)
        self._t_busy += time.perf_counter() - t0
        return sum(e.count for e in entries)

    def run_until_idle(self) -> None:
        while not self.idle:
            if self.step() == 0 and not self.idle:
                raise RuntimeError("scheduler made no progress with requests outstanding")

    # ------------------------------------------------------------------ worker thread
    def start(self) -> None:
        if self._thread is not None:
            return
        self._stop = False
        self._thread = threading.Thread(target=self._run, name="mlxforge-worker", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        try:
            torch.cuda.set_device(self._device_index)
            while True:
                with self._wake:
                    while self.idle and not self._stop:
                        self._wake.wait(timeout=0.1)
                    if self._stop and self.idle:
                        return
                try:
                    self.step()
                except Exception:
                    # step() has already ended every request with "error"; the
                    # worker itself stays up for later requests
                    if self._stop:
                        return
        except BaseException as exc:      # the worker cannot go on: nobody may wait forever
            with self._lock:
                self.scheduler.fail_all(f"worker died: {type(exc).__name__}: {exc}")
            raise

    def stop(self) -> None:
        """Complete what is in flight, then end the worker (src/runtime/worker.cpp:191-194,231-233)."""
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    # ------------------------------------------------------------------ conveniences
    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None,
                 max_tokens: int = 64, eos_ids: Optional[Sequence[int]] = None) -> List[List[int]]:
        """Token ids in, generated token ids out, for one prompt or a batch."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        batch = [prompts] if single else list(prompts)
        reqs = [self.submit_ids(p, params or GREEDY, max_tokens, eos_ids) for p in batch]
        if self._thread is None:
            self.run_until_idle()
        outs = []
        for r in reqs:
            while not r.finished:
                time.sleep(0.0005)
            if r.finish_reason == FINISH_ERROR:
                raise RuntimeError(r.error)
            outs.append(list(r.output_ids))
        return outs[0] if single else outs

    def metrics(self) -> Dict[str, float]:
        """Counters in the manner of src/runtime/metrics.h:9-27."""
        m = self.scheduler.metrics
        return {
            "steps": m.steps, "decode_tokens": m.decode_tokens, "prompt_tokens": m.prompt_tokens,
            "completed": m.completed, "preemptions": m.preemptions, "peak_running": m.peak_running,
            "running": len(self.scheduler.running), "waiting": len(self.scheduler.waiting),
            "pages_free": min(self.cache.free_pages()) if self.cache.pools else 0,
            "pages_total": min(self.cache.total_pages()) if self.cache.pools else 0,
            "busy_seconds": self._t_busy, "steps_ahead": self.steps_ahead,
        }
