"""Replays the same requests whole, with the last 32 tokens decoded one by one,
in portions of changing size and mixed with other requests on a pool so small
that pages are used again, in 32-bit and in bfloat16, and compares every wanted
logit row with the plain implementation's whole-sequence result."""
import numpy as np
import pytest

import plain_llama as P
import trace_tools as TT
from helpers import TINY, make_tiny, random_prompt

pytestmark = pytest.mark.gpu

# Tolerances.  float32: the engine differs from float64 by rounding only; logits of
# these models are O(0.1 .. 1), so 1e-4 absolute (scaled up if a model's logits are
# larger).  bfloat16: the weights are exact in bfloat16, so the gap is the rounding of
# activations; its size depends on the model (a peaked softmax amplifies it), so it is
# measured, per model, as the gap the plain implementation opens against itself when
# it rounds its own activations to bfloat16 (plain_llama.ROUND), and the engine may
# be three times that far from the float64 result.
TOL_F32 = 1e-4
BF16_NOISE_FACTOR = 3.0

LENGTHS = {"A": [5, 17, 31, 70], "B": [1, 9, 40, 70, 131], "C": [3, 33, 64, 97], "D": [2, 19, 66]}


def _requests(cfg, which):
    return {f"r{i}": random_prompt(cfg, n, i) for i, n in enumerate(LENGTHS[which])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    out = {}
    for which in TINY:
        for gain in (1.0, 12.0):
            d, cfg, w = make_tiny(tmp, which, "bfloat16", qk_gain=gain)
            reqs = _requests(cfg, which)
            expected = {rid: P.forward_logits(cfg, w, toks) for rid, toks in reqs.items()}
            P.ROUND = P.round_bf16
            try:
                noise = max(float(np.max(np.abs(P.forward_logits(cfg, w, toks) - expected[rid])))
                            for rid, toks in reqs.items())
            finally:
                P.ROUND = None
            scale = max(float(np.max(np.abs(e))) for e in expected.values())
            tol = {"float32": TOL_F32 * max(1.0, scale), "bfloat16": BF16_NOISE_FACTOR * noise}
            out[(which, gain)] = (d, cfg, reqs, expected, tol)
    return out


def _replay(model_dir, dtype, trace, tmp_path, max_tokens=None):
    from mlxforge_b200.engine.replay import make_runner, replay
    import io
    runner = make_runner(model_dir, dtype, max_tokens or trace.live_tokens_rounded())
    out_dir = str(tmp_path / "out")
    log = io.StringIO()
    replay(runner, trace.lines(), out_dir, done=log)
    assert log.getvalue().splitlines() == [f"done {i}" for i in range(len(trace.steps))]
    runner.cache.check()
    assert all(p.n_held == 0 for p in runner.cache.pools), "pages still held after every request ended"
    return out_dir


MODES = {
    "whole": TT.whole,
    "decode_tail": TT.decode_tail,
    "portions": TT.portions,
    "mixed": TT.mixed,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("gain", [1.0, 12.0])
@pytest.mark.parametrize("which", list(TINY))
def test_replay_matches_plain(models, tmp_path, which, gain, mode, dtype):
    d, cfg, reqs, expected, tols = models[(which, gain)]
    trace = MODES[mode](reqs)
    out_dir = _replay(d, dtype, trace, tmp_path)
    got = TT.read_outputs(trace, out_dir, cfg["vocab_size"])
    assert got, "the trace asked for nothing"
    tol = tols[dtype]
    d_max, where = TT.worst(got, expected)
    assert d_max <= tol, (f"{which} gain {gain} {mode} {dtype}: max abs diff {d_max:.3e} at {where}, "
                          f"first beyond tolerance {tol:.3e} at {TT.first_bad(got, expected, tol)}")


def test_mixed_reuses_pages(models, tmp_path):
    """The mixed trace runs far more tokens through the pool than it holds."""
    d, cfg, reqs, expected, tols = models[("B", 12.0)]
    trace = TT.mixed(reqs, max_live=2, seed=3)
    budget = trace.live_tokens_rounded()
    total = sum(len(t) for t in reqs.values())
    assert total > budget, "the pool would hold everything at once; pages would not be used again"
    out_dir = _replay(d, "float32", trace, tmp_path, max_tokens=budget)
    got = TT.read_outputs(trace, out_dir, cfg["vocab_size"])
    d_max, where = TT.worst(got, expected)
    assert d_max <= tols["float32"], (d_max, where)


@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_replay_with_the_tcgen05_products(models, tmp_path, mode, monkeypatch):
    """The same traces with this engine's own tensor-memory product kernel in place of the
    library's for the many-row products."""
    monkeypatch.setenv("MLXFORGE_GEMM", "tcgen05")
    from mlxforge_b200.csrc import ops
    for which in ("B", "C"):
        d, cfg, reqs, expected, tols = models[(which, 12.0)]
        trace = MODES[mode](reqs)
        out_dir = _replay(d, "bfloat16", trace, tmp_path / which)
        ops.check_kernel_status()
        got = TT.read_outputs(trace, out_dir, cfg["vocab_size"])
        d_max, where = TT.worst(got, expected)
        assert d_max <= tols["bfloat16"], (which, mode, d_max, where)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(tmp_path, dtype):
    """Three requests decoded token by token from position 0, together: the first tokens of a
    sequence (a context of one key), 300 steps of decoding across page edges and across the
    widths for which decode steps are captured, a batch that shrinks as requests end."""
    d, cfg, w = make_tiny(tmp_path, "B", "bfloat16", qk_gain=6.0)
    reqs = {f"l{i}": random_prompt(cfg, n, 40 + i) for i, n in enumerate([300, 150, 40])}
    expected = {rid: P.forward_logits(cfg, w, toks) for rid, toks in reqs.items()}
    P.ROUND = P.round_bf16
    try:
        noise = max(float(np.max(np.abs(P.forward_logits(cfg, w, toks) - expected[rid]))) for rid, toks in reqs.items())
    finally:
        P.ROUND = None
    scale = max(float(np.max(np.abs(e))) for e in expected.values())
    tol = TOL_F32 * max(1.0, scale) if dtype == "float32" else BF16_NOISE_FACTOR * noise
    trace = TT.lockstep(reqs)
    out_dir = _replay(d, dtype, trace, tmp_path)
    got = TT.read_outputs(trace, out_dir, cfg["vocab_size"])
    assert len(got) == sum(len(t) for t in reqs.values())
    d_max, where = TT.worst(got, expected)
    assert d_max <= tol, (f"{dtype}: max abs diff {d_max:.3e} at {where}, first beyond tolerance {tol:.3e} at "
                          f"{TT.first_bad(got, expected, tol)}")
