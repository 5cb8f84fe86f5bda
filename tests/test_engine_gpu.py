"""Generation through the Python entry point and the command line, compared with
the plain implementation: greedy and temperature sampling, several requests at
once equal to each alone, pages running out in flight, and the sampling kernels
alone against the plain sampler."""
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_llama as P
from helpers import TINY, make_tiny, random_prompt

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("engine_models")
    return {w: make_tiny(tmp, w, "bfloat16") for w in TINY}


def _engine(model_dir, **kw):
    import mlxforge_b200 as mf
    opts = dict(model_spec=model_dir, dtype="float32", kv_pool_tokens=2048, max_running=8)
    opts.update(kw)
    return mf.Engine(**opts)


@pytest.mark.parametrize("which,lengths,steps", [("A", [5, 17, 31], 8), ("B", [1, 9, 40, 70], 12)])
def test_greedy_generation_matches_plain(tiny, which, lengths, steps):
    d, cfg, w = tiny[which]
    eng = _engine(d)
    prompts = [random_prompt(cfg, n, 10 + i) for i, n in enumerate(lengths)]
    expected = [P.generate(cfg, w, p, steps) for p in prompts]
    # each alone
    for p, e in zip(prompts, expected):
        assert eng.generate(p, max_tokens=steps) == e
    # all at once: the same tokens as alone (the reference's strongest property,
    # tests/scheduler/validation_test.cpp:44-89)
    assert eng.generate(prompts, max_tokens=steps) == expected
    # and in portions of 7 beside decoding requests
    eng2 = _engine(d, prefill_chunk=7, token_budget=16)
    assert eng2.generate(prompts, max_tokens=steps) == expected
    m = eng2.metrics()
    assert m["completed"] == len(prompts) and m["pages_free"] == m["pages_total"]


def test_bfloat16_greedy_agrees_where_the_margin_is_clear(tiny):
    d, cfg, w = tiny["B"]
    eng = _engine(d, dtype="bfloat16")
    for i, n in enumerate([9, 40]):
        p = random_prompt(cfg, n, 30 + i)
        got = eng.generate(p, max_tokens=10)
        seq = list(p)
        for t in got:
            row = P.forward_logits(cfg, w, seq)[-1]
            top2 = np.sort(row)[-2:]
            if top2[1] - top2[0] > 0.05:          # far beyond bfloat16 noise on these logits
                assert t == int(np.argmax(row))
            seq.append(t)


def test_temperature_sampling_matches_plain(tiny):
    import mlxforge_b200 as mf
    d, cfg, w = tiny["B"]
    eng = _engine(d)
    prompt = random_prompt(cfg, 40, 77)
    done = 0
    for seed in range(20):
        # the plain run, noting how close each draw came to an edge of the CDF
        seq, exp, margin = list(prompt), [], 1.0
        for i in range(12):
            row = P.forward_logits(cfg, w, seq)[-1]
            t, m = P.sample_token(row, 0.8, P.uniform_for(seed, i))
            margin = min(margin, m)
            exp.append(t)
            seq.append(t)
        if margin < 1e-5:
            continue      # a draw on an edge decides by rounding; such seeds prove nothing
        got = eng.generate(prompt, mf.SamplingParams(temperature=0.8, seed=seed), max_tokens=12)
        assert got == exp, f"seed {seed}"
        done += 1
        if done == 3:
            break
    assert done == 3
    assert len(set(exp)) > 3, "temperature sampling should not collapse to one token"


def test_eos_stops_and_is_not_emitted(tiny):
    d, cfg, w = tiny["A"]
    eng = _engine(d)
    p = random_prompt(cfg, 17, 5)
    full = P.generate(cfg, w, p, 8)
    req = eng.submit_ids(p, None, 8, eos_ids=[full[3]])
    req.params = __import__("mlxforge_b200").GREEDY
    eng.run_until_idle()
    first = full.index(full[3])
    assert req.output_ids == full[:first] and req.finish_reason == "stop"
    assert list(req) == full[:first]


def test_pages_run_out_in_flight(tiny):
    """A pool too small for all requests at once: some are preempted and recomputed,
    and every request still produces exactly its own tokens."""
    d, cfg, w = tiny["A"]
    prompts = [random_prompt(cfg, n, 50 + i) for i, n in enumerate([30, 25, 20, 28])]
    expected = [P.generate(cfg, w, p, 20) for p in prompts]
    eng = _engine(d, kv_pool_tokens=112, max_running=4)       # 7 pages of 16 for 4 x ~50 tokens
    assert eng.generate(prompts, max_tokens=20) == expected
    m = eng.metrics()
    assert m["preemptions"] >= 1 and m["pages_free"] == m["pages_total"]
    eng.cache.check()


def test_worker_thread_and_cancel(tiny):
    import mlxforge_b200 as mf
    d, cfg, w = tiny["A"]
    eng = _engine(d)
    eng.start()
    p = random_prompt(cfg, 12, 3)
    a = eng.submit_ids(p, mf.GREEDY, 8)
    b = eng.submit_ids(p, mf.GREEDY, 100000)
    assert list(a) == P.generate(cfg, w, p, 8)
    b.cancel()
    while b.next(timeout=10) is not None:
        pass
    assert b.finish_reason == "cancel"
    eng.stop()
    assert eng.scheduler.idle


def test_cli_generate_and_replay(tiny, tmp_path):
    d, cfg, w = tiny["A"]
    p = random_prompt(cfg, 9, 1)
    np.save(tmp_path / "ids.npy", np.asarray(p, dtype=np.int32))
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-m", "mlxforge_b200", "generate", d, str(tmp_path / "ids.npy"), "6",
                          "--dtype", "float32"], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr
    assert [int(t) for t in out.stdout.split()] == P.generate(cfg, w, p, 6)
    assert "time to first token" in out.stderr
    trace = '{"step": 0, "entries": [{"id": "a", "tokens": %s, "want": [8]}], "end": ["a"]}\n' % p
    out = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out",
                          str(tmp_path / "o"), "--max-tokens", "64"], input=trace, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0 and out.stdout.strip() == "done 0", out.stderr
    got = np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4")
    assert np.max(np.abs(got - P.forward_logits(cfg, w, p)[-1])) < 1e-4


# ----------------------------------------------------------------------------- sampling kernels alone

@pytest.mark.parametrize("V", [307, 4096, 128256])
def test_sample_kernel_against_plain(V):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(V)
    n = 6
    logits = (rng.standard_normal((n, V)) * 2.0).astype(np.float32)
    logits[0, 5] = logits[0, 200] = logits[0].max() + 1.0          # a tie: lowest index wins
    temps = np.array([0.0, 0.7, 1.0, 1.3, 0.0, 0.5], dtype=np.float32)
    us = np.array([0.3, 0.123, 0.999, 0.5, 0.0, 0.0], dtype=np.float32)
    dl = torch.from_numpy(logits).cuda()
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample(dl, None, None, out)
    assert out.tolist() == [int(np.argmax(r)) for r in logits] and out[0].item() == 5
    ops.sample(dl, torch.from_numpy(temps).cuda(), torch.from_numpy(us).cuda(), out)
    for r in range(n):
        tok, margin = P.sample_token(logits[r], float(temps[r]), float(us[r]))
        if margin > 1e-5:
            assert out[r].item() == tok, (r, tok, out[r].item())


def test_two_sampler_launches_in_flight_keep_their_own_draws():
    """The engine launches a step's sampling before it has collected the step before.  The second
    launch must not change what the first one reads from the host (its rows' temperatures and
    uniform draws), even if the first has not started when the second is issued: here the device
    is kept busy for a while before the first launch, and the two launches draw differently."""
    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.sampling.sampler import Sampler
    rng = np.random.default_rng(3)
    n, V = 5, 4099
    logits = [torch.from_numpy((rng.standard_normal((n, V)) * 1.5).astype(np.float32)).cuda() for _ in range(2)]
    params = [mf.SamplingParams(temperature=0.7 + 0.1 * r, seed=11 + r) for r in range(n)]
    one = Sampler("cuda")
    want = [one.sample(logits[i].clone(), params, [i * 7 + r for r in range(n)]) for i in range(2)]
    assert want[0] != want[1]
    two = Sampler("cuda")
    torch.cuda._sleep(200_000_000)                  # about a tenth of a second of device time
    h0 = two.launch(logits[0].clone(), params, [r for r in range(n)])
    h1 = two.launch(logits[1].clone(), params, [7 + r for r in range(n)])
    assert [two.collect(h0), two.collect(h1)] == want


def test_filters_and_penalties_against_plain():
    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(9)
    V = 5003
    cases = [mf.SamplingParams(temperature=0.9, top_k=40), mf.SamplingParams(temperature=1.2, top_p=0.85),
             mf.SamplingParams(temperature=0.6, min_p=0.05),
             mf.SamplingParams(temperature=0.8, top_k=200, top_p=0.9, min_p=0.01),
             mf.SamplingParams(temperature=0.0, top_k=5), mf.SamplingParams(temperature=1.0, top_k=V + 10)]
    logits = (rng.standard_normal((len(cases), V)) * 3.0).astype(np.float32)
    dl = torch.from_numpy(logits.copy()).cuda()
    ops.filter_logits(dl, cases)
    got = dl.cpu().numpy()
    for r, p in enumerate(cases):
        if p.greedy:
            assert np.array_equal(got[r], logits[r])
            continue
        want = P.filter_logits(logits[r], p.temperature, p.top_k, p.top_p, p.min_p)
        kept_want, kept_got = np.isfinite(want), np.isfinite(got[r])
        # the two may differ only on entries whose probability sits on a threshold
        diff = np.flatnonzero(kept_want != kept_got)
        assert diff.size <= 1, (r, diff)
        assert np.array_equal(got[r][kept_got], logits[r][kept_got])
    hist = [list(rng.integers(0, V, size=50)) + [7, 7, 7], [], list(range(10))]
    pp = [mf.SamplingParams(repetition_penalty=1.3, frequency_penalty=0.2, presence_penalty=0.4),
          mf.SamplingParams(), mf.SamplingParams(repetition_penalty=0.8)]
    logits = (rng.standard_normal((3, V)) * 3.0).astype(np.float32)
    dl = torch.from_numpy(logits.copy()).cuda()
    ops.apply_penalties(dl, pp, hist)
    got = dl.cpu().numpy()
    for r, p in enumerate(pp):
        want = P.apply_penalties(logits[r], hist[r], p.repetition_penalty, p.frequency_penalty, p.presence_penalty)
        assert np.max(np.abs(got[r] - want)) < 1e-5


def test_dependent_launch_and_graphs_change_no_bit(tiny):
    """Decoding with CUDA graphs and dependent launches gives the same logits, bit for
    bit, as launching every kernel eagerly one after the other."""
    import torch
    from mlxforge_b200.csrc import ops
    from mlxforge_b200.engine.replay import make_runner
    from mlxforge_b200.engine.step import StepEntry
    d, cfg, w = tiny["B"]
    prompts = [random_prompt(cfg, n, 90 + i) for i, n in enumerate([33, 70, 9])]

    def run(graphs, pdl):
        old = ops.set_dependent_launch(pdl)
        try:
            runner = make_runner(d, "bfloat16", 512)
            runner.cuda_graphs = graphs
            seqs = [runner.cache.open_sequence() for _ in prompts]
            runner.step([StepEntry(s, p[:-6], []) for s, p in zip(seqs, prompts)])
            outs = []
            for i in range(6, 0, -1):
                logits = runner.step([StepEntry(s, [p[-i]], [0]) for s, p in zip(seqs, prompts)])
                outs.append(logits.clone())
            torch.cuda.synchronize()
            return torch.stack(outs), runner.graph_replays
        finally:
            ops.set_dependent_launch(old)

    eager, n0 = run(False, False)
    fast, n1 = run(True, True)
    assert n0 == 0 and n1 >= 4, "the second run must have replayed graphs"
    assert torch.equal(eager, fast)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_no_token(tiny, dtype):
    """Decode steps launched before the host has the tokens of the step before (fed on the
    device) give every request the tokens it gets from the step-by-step loop: greedy and
    seeded temperature sampling, requests of different lengths, one that meets its EOS."""
    import mlxforge_b200 as mf
    d, cfg, w = tiny["B"]
    prompts = [random_prompt(cfg, n, 200 + i) for i, n in enumerate([12, 45, 3, 70])]
    lengths = [40, 25, 33, 40]

    def run(pipeline, params):
        eng = _engine(d, dtype=dtype, pipeline=pipeline)
        reqs = [eng.submit_ids(p, params, n, eos_ids=[]) for p, n in zip(prompts, lengths)]
        eng.run_until_idle()
        outs = [list(r.output_ids) for r in reqs]
        # again, now with the 10th token of the first request as its EOS
        eng2 = _engine(d, dtype=dtype, pipeline=pipeline)
        reqs2 = [eng2.submit_ids(p, params, n, eos_ids=([outs[0][9]] if i == 0 else []))
                 for i, (p, n) in enumerate(zip(prompts, lengths))]
        eng2.run_until_idle()
        m = eng2.metrics()
        assert m["pages_free"] == m["pages_total"]
        return outs, [(list(r.output_ids), r.finish_reason) for r in reqs2], eng.steps_ahead

    for params in (mf.GREEDY, mf.SamplingParams(temperature=0.9, top_k=20, seed=5)):
        plain, plain_eos, n0 = run(False, params)
        ahead, ahead_eos, n1 = run(True, params)
        assert n0 == 0 and n1 >= 20, "the second run must have launched steps ahead"
        assert ahead == plain and ahead_eos == plain_eos
        assert plain_eos[0][1] == "stop" and len(plain_eos[0][0]) <= 9


def test_rope_scaling_override_changes_what_is_generated(tmp_path):
    """The engine's ``rope_scaling`` option replaces the checkpoint's object: the tokens are those
    of the plain implementation for a config that has the override, in the engine and through the
    command line's ``--rope-scaling``."""
    from helpers import TINY_B, random_weights, write_model_dir
    cfg = TINY_B
    w = random_weights(cfg, seed=1, norm_std=0.1, std=0.1)       # large enough that the tokens vary
    d = write_model_dir(str(tmp_path / "m"), cfg, w, "bfloat16")
    w = {k: v.astype(np.float64) for k, v in w.items()}
    override = {"rope_type": "linear", "factor": 4.0}
    prompt = random_prompt(cfg, 70, 5)
    import json
    want = P.generate(dict(cfg, rope_scaling=override), w, prompt, 10)
    plain = P.generate(cfg, w, prompt, 10)
    assert want != plain, "the override must matter for this prompt, or the test shows nothing"
    assert _engine(d, rope_scaling=json.dumps(override)).generate(prompt, max_tokens=10) == want
    assert _engine(d).generate(prompt, max_tokens=10) == plain
    r = subprocess.run([sys.executable, "-m", "mlxforge_b200", "generate", d, ",".join(map(str, prompt)), "10",
                        "--dtype", "float32", "--rope-scaling", json.dumps(override)],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.strip().splitlines()[-1].replace(",", " ").split()] == want
