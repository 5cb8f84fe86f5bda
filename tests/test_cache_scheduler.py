"""The cache manager's bookkeeping (no page lost, held twice or freed twice, under
random orders of requests; windowed groups give pages back) and the scheduler's
decisions (admission, portions under a token budget, decoding, finishing,
cancelling, what happens when pages run out).  CPU only: the scheduler is driven
with a fake step that returns chosen tokens."""
import random

import numpy as np

import pytest
import torch

from mlxforge_b200.cache import CacheLayout, CacheManager, GroupLayout, OutOfPages, OutOfSlots, PagePool
from mlxforge_b200.engine.request import Request
from mlxforge_b200.engine.scheduler import Scheduler, SchedulerConfig
from mlxforge_b200.parts.base import FixedState, PagedKV
from mlxforge_b200.sampling import GREEDY


def layout(window=0, with_state=False, two_groups=False):
    paged = [GroupLayout(PagedKV(2, 16, 0), 2)]
    lanes = [("paged", 0, 0), ("paged", 0, 1)]
    if two_groups or window:
        paged.append(GroupLayout(PagedKV(1, 32, window), 1))
        lanes.append(("paged", 1, 0))
    state = []
    if with_state:
        state.append(GroupLayout(FixedState((4,)), 1))
        lanes.append(("state", 0, 0))
    return CacheLayout(tuple(paged), tuple(state), tuple(lanes))


def manager(max_tokens=256, max_seqs=8, **kw):
    return CacheManager(layout(**kw), page_size=16, max_tokens=max_tokens, max_seqs=max_seqs,
                        dtype=torch.float32, device="cpu")


# ----------------------------------------------------------------------------- pool

def test_page_pool_discipline():
    p = PagePool(4)
    a = p.take(3)
    assert len(set(a)) == 3 and p.n_free == 1
    with pytest.raises(OutOfPages):
        p.take(2)
    assert p.n_free == 1, "a refused reservation must take nothing"
    p.give_back(a[:1])
    with pytest.raises(RuntimeError, match="not held"):
        p.give_back(a[:1])
    with pytest.raises(RuntimeError, match="not held"):
        p.give_back([99])
    p.check()
    assert p.high_water == 3


def test_reserve_is_all_or_nothing():
    m = manager(max_tokens=64)            # 4 pages
    a, b = m.open_sequence(), m.open_sequence()
    m.reserve([(a, 20)])                  # 2 pages
    m.commit(a, 20)
    with pytest.raises(OutOfPages):
        m.reserve([(a, 10), (b, 40)])     # 0 + 3 > 2 free
    assert m.free_pages() == [2] and b.blocks == [[]]
    m.reserve([(a, 10), (b, 30)])         # a still fits its second page; b takes 2
    m.commit(a, 10)
    m.commit(b, 30)
    assert m.free_pages() == [0]
    m.check()
    m.close(a)
    with pytest.raises(RuntimeError, match="closed twice"):
        m.close(a)
    with pytest.raises(RuntimeError, match="closed"):
        m.reserve([(a, 1)])
    m.close(b)
    assert m.free_pages() == [4]
    m.check()


def test_slots_and_state_zeroed():
    m = manager(max_seqs=2, with_state=True)
    a, b = m.open_sequence(), m.open_sequence()
    assert {a.slot, b.slot} == {0, 1}
    with pytest.raises(OutOfSlots):
        m.open_sequence()
    lane = m.lane(2)
    lane.tensor[a.slot] += 7.0
    m.close(a)
    c = m.open_sequence()
    assert c.slot == a.slot and float(lane.tensor[c.slot].abs().sum()) == 0.0, "a reused slot starts at zero"


def test_window_gives_pages_back():
    m = manager(max_tokens=4096, window=40)
    s = m.open_sequence()
    for _ in range(30):
        m.reserve([(s, 10)])
        m.commit(s, 10)
        m.check()
        # full-attention group keeps everything, the windowed one only what a next query can see
        assert s.pages_held(0) == (s.length + 15) // 16
        first_visible = max(0, s.length - 40 + 1)
        assert s.pages_held(1) == len(s.blocks[1]) - first_visible // 16
        assert all(p == -1 for p in s.blocks[1][:first_visible // 16])
    assert s.pages_held(1) <= 4
    m.close(s)
    assert m.free_pages() == m.total_pages()


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    m = manager(max_tokens=640, max_seqs=6, two_groups=True, window=0)
    live = []
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            live.append(m.open_sequence())
        elif op < 0.85 and live:
            batch = rng.sample(live, rng.randint(1, len(live)))
            req = [(s, rng.choice([1, 1, 1, 2, 7, 16, 33])) for s in batch]
            before = m.free_pages()
            try:
                m.reserve(req)
            except OutOfPages:
                assert m.free_pages() == before
            else:
                for s, n in req:
                    m.commit(s, n)
        elif live:
            m.close(live.pop(rng.randrange(len(live))))
        m.check()
    for s in live:
        m.close(s)
    m.check()
    assert m.free_pages() == m.total_pages()
    assert m.slots.n_free == 6


# ----------------------------------------------------------------------------- scheduler

class FakeEngine:
    """Drives a Scheduler the way Engine.step does, with a token function in place
    of the model: the next token of a request is f(request, number of tokens so far)."""

    def __init__(self, sched, cache, next_token):
        self.s, self.cache, self.next_token = sched, cache, next_token
        self.log = []

    def step(self):
        entries = self.s.plan()
        if not entries:
            return 0
        self.cache.reserve([(e.request.seq, e.count) for e in entries])   # must never raise: plan() checked
        for e in entries:
            assert e.start == e.request.seq.length, "portions of one request must run in order, once"
            self.cache.commit(e.request.seq, e.count)
        sampled = [self.next_token(e.request, e.start + e.count) for e in entries if e.samples]
        self.log.append([(e.request.request_id, e.start, e.count, e.samples) for e in entries])
        self.s.commit(entries, sampled)
        self.cache.check()
        return sum(e.count for e in entries)

    def run(self, limit=10000):
        n = 0
        while not self.s.idle:
            assert self.step() > 0 or self.s.idle, "no progress"
            n += 1
            assert n < limit
        return n


def tok(req, n_so_far):
    return (req.request_id * 7 + n_so_far) % 50 + 1


def make(max_tokens=4096, **cfg):
    m = manager(max_tokens=max_tokens, max_seqs=cfg.get("max_running", 8))
    s = Scheduler(m, SchedulerConfig(**cfg))
    return s, m, FakeEngine(s, m, tok)


def test_portions_budget_and_first_token():
    s, m, eng = make(token_budget=64, prefill_chunk=24, max_running=4)
    a = Request(list(range(1, 51)), GREEDY, max_tokens=3)
    assert s.submit(a)
    eng.run()
    flat = [x for step in eng.log for x in step]
    assert [(st, n, smp) for _, st, n, smp in flat[:3]] == [(0, 24, False), (24, 24, False), (48, 2, True)]
    assert [(n, smp) for _, _, n, smp in flat[3:]] == [(1, True), (1, True)]
    assert a.finish_reason == "length" and len(a.output_ids) == 3
    assert a.output_ids == [tok(a, 50), tok(a, 51), tok(a, 52)]
    assert m.free_pages() == m.total_pages()


def test_mixed_steps_decode_first_and_budget():
    s, m, eng = make(token_budget=40, prefill_chunk=32, max_running=4)
    a = Request([1] * 10, GREEDY, max_tokens=20)
    b = Request([2] * 100, GREEDY, max_tokens=2)
    s.submit(a)
    eng.step()                      # a's whole prompt
    s.submit(b)
    eng.step()
    ids = eng.log[-1]
    assert ids[0] == (a.request_id, 10, 1, True), "the decoding request comes first with one token"
    assert ids[1] == (b.request_id, 0, 32, False), "then a prompt portion, capped by prefill_chunk"
    for step in eng.log:
        assert sum(n for _, _, n, _ in step) <= 40
    eng.run()
    assert a.finish_reason == "length" and b.finish_reason == "length"
    assert len(a.output_ids) == 20 and len(b.output_ids) == 2
    # a kept decoding every step while b's prompt was being consumed
    steps_with_both = [st for st in eng.log if len(st) == 2]
    assert len(steps_with_both) >= 4


def test_eos_cancel_and_queue_bound():
    s, m, eng = make(max_waiting=2, max_running=1)
    a = Request([3, 4, 5], GREEDY, max_tokens=10)
    a.eos_ids = (tok(a, 5),)        # the third generated token is EOS
    b = Request([1, 2], GREEDY, max_tokens=50)
    c = Request([1, 2], GREEDY, max_tokens=5)
    assert s.submit(a) and s.submit(b)
    assert not s.submit(c), "submit refuses when max_waiting are waiting"
    eng.step()                      # a admitted (max_running 1), b still waits
    assert s.submit(c)
    c.cancel()                      # cancelled before admission
    for _ in range(4):
        eng.step()
    assert a.finish_reason == "stop" and a.output_ids == [tok(a, 3), tok(a, 4)], "EOS is not emitted"
    b.cancel()
    eng.run()
    assert b.finish_reason == "cancel" and c.finish_reason == "cancel" and c.output_ids == []
    assert m.free_pages() == m.total_pages() and m.slots.n_free == 1


def test_out_of_pages_waits_at_admission():
    s, m, eng = make(max_tokens=64, token_budget=256, prefill_chunk=256, max_running=4)   # 4 pages
    a = Request([1] * 40, GREEDY, max_tokens=4)     # 3 pages
    b = Request([2] * 30, GREEDY, max_tokens=4)     # 2 pages: does not fit beside a
    s.submit(a)
    s.submit(b)
    eng.step()
    assert [r.request_id for r in s.running] == [a.request_id] and list(s.waiting) == [b]
    eng.run()
    assert a.finish_reason == b.finish_reason == "length"
    assert s.metrics.preemptions == 0
    first_b = next(i for i, st in enumerate(eng.log) if any(x[0] == b.request_id for x in st))
    last_a = max(i for i, st in enumerate(eng.log) if any(x[0] == a.request_id for x in st))
    assert first_b > last_a, "b is admitted only after a gave its pages back"


def test_preemption_recomputes_and_keeps_the_stream():
    s, m, eng = make(max_tokens=64, token_budget=256, prefill_chunk=256, max_running=4)   # 4 pages
    a = Request([1] * 30, GREEDY, max_tokens=40)    # grows to 70 tokens: more than the pool -> error at the end
    b = Request([2] * 14, GREEDY, max_tokens=12)    # 14 + 12 = 26 tokens: 2 pages
    s.submit(a)
    s.submit(b)
    eng.run()
    assert s.metrics.preemptions >= 1
    assert b.finish_reason == "length" and b.output_ids == [tok(b, 14 + i) for i in range(12)], \
        "a preempted request resumes its own stream"
    assert b.preemptions >= 1, "the most recently admitted request is the one preempted"
    # a alone outgrows the pool: it ends with an error that says so, after emitting what fitted
    assert a.finish_reason == "error" and "does not fit" in a.error
    assert a.output_ids == [tok(a, 30 + i) for i in range(len(a.output_ids))] and len(a.output_ids) >= 30
    assert m.free_pages() == m.total_pages() and m.slots.n_free == 4


def test_request_larger_than_pool_fails_at_admission():
    s, m, eng = make(max_tokens=32)
    a = Request([1] * 100, GREEDY, max_tokens=4)
    s.submit(a)
    eng.step()
    assert a.finish_reason == "error" and "pages" in a.error
    with pytest.raises(RuntimeError):
        a.next()
    e = Request([], GREEDY)
    s.submit(e)
    assert e.finish_reason == "error"


@pytest.mark.parametrize("seed", range(4))
def test_random_load_every_request_gets_its_own_stream(seed):
    rng = random.Random(seed)
    s, m, eng = make(max_tokens=rng.choice([96, 160, 512]), token_budget=rng.choice([16, 48, 200]),
                     prefill_chunk=rng.choice([8, 32, 64]), max_running=rng.choice([2, 4, 8]))
    reqs = []
    for i in range(20):
        r = Request([rng.randrange(1, 50) for _ in range(rng.randrange(1, 60))], GREEDY,
                    max_tokens=rng.randrange(1, 20))
        reqs.append(r)
    pending = list(reqs)
    while pending or not s.idle:
        while pending and rng.random() < 0.5:
            assert s.submit(pending.pop(0))
        if eng.step() == 0 and not pending:
            assert s.idle
    for r in reqs:
        assert r.finish_reason in ("length", "error"), r.finish_reason
        n0 = len(r.prompt_ids)
        assert r.output_ids == [tok(r, n0 + i) for i in range(len(r.output_ids))]
        if r.finish_reason == "length":
            assert len(r.output_ids) == r.max_tokens
    assert m.free_pages() == m.total_pages() and m.slots.n_free == m.slots.n_slots


# ----------------------------------------------------------------------------- steps launched ahead

class PipelinedFakeEngine(FakeEngine):
    """Drives a Scheduler the way the pipelined Engine.step does: a step is launched (the cache
    reserved and advanced) and its tokens are only known at the next call, which, when
    ``continue_decoding`` allows it, launches the step after before it commits."""

    def __init__(self, sched, cache, next_token):
        super().__init__(sched, cache, next_token)
        self.inflight = None
        self.ahead = 0

    def _launch(self, entries):
        self.cache.reserve([(e.request.seq, e.count) for e in entries])
        for e in entries:
            assert e.start == e.request.seq.length, "portions of one request must run in order, once"
            self.cache.commit(e.request.seq, e.count)
        self.log.append([(e.request.request_id, e.start, e.count, e.samples) for e in entries])

    def step(self):
        if self.inflight is None:
            entries = self.s.plan()
            if not entries:
                return 0
            self._launch(entries)
            self.inflight = entries
            return sum(e.count for e in entries)
        entries = self.inflight
        nxt = self.s.continue_decoding(entries)
        if nxt is not None:
            self._launch(nxt)          # before the tokens of `entries` are known
            self.ahead += 1
        sampled = [self.next_token(e.request, e.start + e.count) for e in entries if e.samples]
        self.s.commit(entries, sampled)
        self.cache.check()
        self.inflight = nxt
        return sum(e.count for e in entries)

    def run(self, limit=10000):
        n = 0
        while not (self.s.idle and self.inflight is None):
            assert self.step() > 0 or (self.s.idle and self.inflight is None), "no progress"
            n += 1
            assert n < limit
        return n


def test_continue_decoding_says_when_the_next_step_is_known():
    s, m, _ = make(token_budget=64, prefill_chunk=32, max_running=4)
    eng = PipelinedFakeEngine(s, m, tok)
    a = Request([1] * 10, GREEDY, max_tokens=6)
    b = Request([2] * 5, GREEDY, max_tokens=50)
    s.submit(a), s.submit(b)
    eng.step()                                   # both prompts, launched
    assert s.continue_decoding(eng.inflight) is None, "a prompt portion is on its way: not a decode step"
    eng.step()                                   # commit: both have their first token
    eng.step()                                   # a decode step launched
    nxt = s.continue_decoding(eng.inflight)
    assert [(e.request.request_id, e.start, e.count, e.samples) for e in nxt] == \
        [(a.request_id, 11, 1, True), (b.request_id, 6, 1, True)]
    c = Request([3] * 4, GREEDY, max_tokens=3)
    s.submit(c)
    assert s.continue_decoding(eng.inflight) is None, "somebody waits: the next step has to be planned"
    s.cfg.max_running = 2
    assert s.continue_decoding(eng.inflight) is not None, "somebody waits, but no slot is free before one ends"
    s.cfg.max_running = 4
    eng.run()
    assert a.output_ids == [tok(a, 10 + i) for i in range(6)] and a.finish_reason == "length"
    assert len(b.output_ids) == 50 and len(c.output_ids) == 3
    assert eng.ahead > 20, "steady decoding was launched ahead"
    # the step in which a got its last token was not followed by one with a in it
    last_a = max(i for i, st in enumerate(eng.log) if any(x[0] == a.request_id for x in st))
    assert eng.log[last_a][[x[0] for x in eng.log[last_a]].index(a.request_id)][1] == 10 + 4
    assert m.free_pages() == m.total_pages()


def test_a_request_that_ends_while_a_step_is_ahead_leaves_a_dropped_row():
    s, m, _ = make(max_running=4)
    eng = PipelinedFakeEngine(s, m, tok)
    a = Request([3, 4, 5], GREEDY, max_tokens=40)
    b = Request([6, 7], GREEDY, max_tokens=40)
    a.eos_ids = (tok(a, 8),)                     # a's sixth token is EOS: nobody can know before it is sampled
    s.submit(a), s.submit(b)
    eng.run()
    assert a.finish_reason == "stop" and a.output_ids == [tok(a, 3 + i) for i in range(5)]
    assert b.finish_reason == "length" and b.output_ids == [tok(b, 2 + i) for i in range(40)]
    rows_of_a = [x for st in eng.log for x in st if x[0] == a.request_id]
    assert rows_of_a[-1][1] == 3 + 5, "one row of a ran past its end (launched before the EOS was seen)"
    assert m.free_pages() == m.total_pages() and m.slots.n_free == 4


@pytest.mark.parametrize("seed", range(6))
def test_pipelined_random_load_matches_the_plain_loop(seed):
    """Random arrivals, lengths, EOS tokens and cancels, few pages: launching ahead changes no
    request's tokens or finish reason, and no page is lost."""
    results = []
    for cls in (FakeEngine, PipelinedFakeEngine):
        rng = np.random.default_rng(seed)
        s, m, _ = make(max_tokens=int(rng.integers(200, 600)), token_budget=48, prefill_chunk=16, max_running=4)
        eng = cls(s, m, lambda r, n: (r.tag * 7 + n) % 13 + 1)
        reqs = []
        for i in range(14):
            r = Request([int(x) for x in rng.integers(1, 50, size=int(rng.integers(1, 60)))], GREEDY,
                        max_tokens=int(rng.integers(1, 40)))
            r.tag = i
            if rng.random() < 0.5:
                r.eos_ids = (int(rng.integers(1, 14)),)
            reqs.append(r)
        pending = list(reqs)
        n = 0
        while pending or not s.idle or getattr(eng, "inflight", None) is not None:
            while pending and rng.random() < 0.4:
                assert s.submit(pending.pop(0))
            if eng.step() == 0 and pending:
                assert s.submit(pending.pop(0))
            n += 1
            assert n < 5000
        m.check()
        assert m.free_pages() == m.total_pages()
        results.append([(r.output_ids, r.finish_reason) for r in reqs])
    assert results[0] == results[1]


def test_scratch_views_are_kept_until_a_buffer_moves():
    """The runtime hands out the same view for the same (name, shape) step after step, and a view
    made before a buffer grew is never handed out again (captured graphs are rebuilt on the same
    signal, ``generation``)."""
    import torch
    from mlxforge_b200.engine.runtime import Runtime
    rt = Runtime(torch.float32, device="cpu")
    a = rt.buffer("x", (4, 8))
    assert rt.buffer("x", (4, 8)) is a and rt.generation == 1
    other = rt.buffer("y", (3,), torch.int32)
    assert other.dtype == torch.int32 and rt.generation == 2
    assert rt.buffer("x", (4, 8)).data_ptr() == a.data_ptr(), "y's arrival moved nothing of x"
    big = rt.buffer("x", (16, 8))                      # x grows: its storage moves
    assert rt.generation == 3
    again = rt.buffer("x", (4, 8))
    assert again is not a and again.data_ptr() == big.data_ptr()
    rt.reserve_rows = 64
    wide = rt.buffer("z", (2, 5))
    assert rt.buffer("z", (64, 5)).data_ptr() == wide.data_ptr(), "made for reserve_rows rows at once"


# ----------------------------------------------------------------------------- a kernel that gave up

class _WordRunner:
    """Stands in for ModelRunner: moves the cache on as a step does and, at a chosen step, sets
    the word that a kernel sets when one of its bounded waits runs out."""

    def __init__(self, cache, word):
        self.cache, self.word = cache, word
        self.steps, self.fault_at = 0, None

    def step(self, entries, device_tokens=None):
        self.cache.reserve([(e.seq, len(e.tokens)) for e in entries])
        for e in entries:
            self.cache.commit(e.seq, len(e.tokens))
        self.steps += 1
        if self.steps == self.fault_at:
            self.word[0] = 2
        return sum(len(e.want) for e in entries) or None


class _WordSampler:
    """Stands in for Sampler: the word travels with the tokens and ``collect`` raises, as the
    real one does, when it is not zero."""

    device_ids = None

    def __init__(self, word):
        self.word = word

    def launch(self, n_rows, params, indices, histories=()):
        return (self.word[0], n_rows)

    def collect(self, handle):
        from mlxforge_b200.csrc.binding import KernelError
        if handle is None:
            return []
        code, n = handle
        if code:
            self.word[0] = 0
            raise KernelError(f"a kernel's bounded wait ran out (code {code})")
        return [7] * n


@pytest.mark.parametrize("pipeline", [False, True])
def test_a_kernel_that_gave_up_ends_every_request_with_error(pipeline):
    """The engine's own loop around stand-ins for the step and the sampler: when the status word
    comes back non-zero, no token of that step is emitted, every request ends with "error", all
    pages and slots come back, and the engine serves the next request."""
    from types import SimpleNamespace
    from mlxforge_b200.csrc.binding import KernelError
    from mlxforge_b200.engine.engine import Engine, EngineConfig
    word = [0]
    cache = manager(max_tokens=1024)
    runner = _WordRunner(cache, word)
    model = SimpleNamespace(spec=SimpleNamespace(vocab_size=100, eos_token_ids=()))
    cfg = EngineConfig(model_spec="-", max_running=8, token_budget=64, prefill_chunk=16, pipeline=pipeline)
    eng = Engine.from_parts(cfg, model, cache, runner, _WordSampler(word))
    reqs = [eng.submit_ids(list(range(1, 1 + n)), GREEDY, max_tokens=40) for n in (5, 30, 12)]
    runner.fault_at = 6
    with pytest.raises(KernelError):
        for _ in range(100):
            eng.step()
    assert runner.steps >= 6
    assert all(r.finished and r.finish_reason == "error" and "bounded wait" in r.error for r in reqs)
    assert eng.idle
    cache.check()
    assert cache.free_pages() == cache.total_pages() and cache.slots.n_free == 8
    emitted = [len(r.output_ids) for r in reqs]
    again = eng.submit_ids([1, 2, 3], GREEDY, max_tokens=4)
    eng.run_until_idle()
    assert again.finish_reason == "length" and again.output_ids == [7] * 4
    assert [len(r.output_ids) for r in reqs] == emitted
