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

LENGTHS = {"A": [5, 17, 31, 70, 100, 90, 120], "B": [1, 9, 40, 70, 131, 150], "C": [3, 33, 64, 97, 110, 75],
           "D": [2, 19, 66, 130, 99, 120], "E": [300, 45, 520, 700], "F": [260, 610, 130, 333]}
# portions of the two models with serving shapes cross 128 tokens (the tcgen05 attention) and 256
# rows (the tcgen05 gated product), start at odd offsets, and still go down to two tokens
PORTIONS = {"E": (150, 2, 129, 7, 300, 128, 3, 131, 64, 200), "F": (131, 2, 260, 5, 128, 190, 3, 64)}
MIXED_PORTION = {"E": 180, "F": 150}
# Queries and keys are scaled so that the softmax is peaked and a wrong or missing key changes the
# logits.  How far that can go depends on the model: the wider models with head sizes 64 and 128
# amplify rounding so much at a gain of 12 that float32 itself is off by 1e-3 (rounding nothing but
# the activations to float32 in the plain implementation moves F's logits by 6e-4 there) and the
# bfloat16 noise floor is as large as the logits; at 2 the floors are 2e-6 and about 1 %.
PEAKED_GAIN = {"A": 12.0, "B": 12.0, "C": 12.0, "D": 12.0, "E": 2.0, "F": 2.0}
POISON = float("nan")
"""What the cache pools hold before a replay: a key or a value that is used from a slot which
the trace never wrote (a page that was handed out again, the tail of a last page, a page the
block table does not name) makes the logits NaN."""


def _requests(cfg, which):
    return {f"r{i}": random_prompt(cfg, n, i) for i, n in enumerate(LENGTHS[which])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    out = {}
    for which in TINY:
        for peaked in (False, True):
            gain = PEAKED_GAIN[which] if peaked else 1.0
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
            out[(which, peaked)] = (d, cfg, reqs, expected, tol)
    return out


def _replay(model_dir, dtype, trace, tmp_path, max_tokens=None):
    """Replays on a pool of exactly the tokens the trace holds at its peak, poisoned beforehand.
    Returns (output folder, which kernels ran how often)."""
    from mlxforge_b200.csrc import binding
    from mlxforge_b200.engine.replay import make_runner, replay
    import io
    runner = make_runner(model_dir, dtype, max_tokens or trace.live_tokens_rounded())
    for pool in runner.cache._k + runner.cache._v:
        pool.fill_(POISON)
    out_dir = str(tmp_path / "out")
    log = io.StringIO()
    before = binding.kernel_launches()
    replay(runner, trace.lines(), out_dir, done=log)
    ran = {k: v - before[k] for k, v in binding.kernel_launches().items()}
    assert log.getvalue().splitlines() == [f"done {i}" for i in range(len(trace.steps))]
    runner.cache.check()
    assert all(p.n_held == 0 for p in runner.cache.pools), "pages still held after every request ended"
    return out_dir, ran


def _portions(reqs, which):
    return TT.portions(reqs, PORTIONS[which]) if which in PORTIONS else TT.portions(reqs)


def _mixed(reqs, which):
    return TT.mixed(reqs, max_portion=MIXED_PORTION.get(which, 9))


def _mixed_tight(reqs, which):
    """Two live requests at a time on a pool of their peak: the trace runs more tokens through
    the pool than it holds, so later requests get pages that earlier ones gave back."""
    trace = TT.mixed(reqs, max_live=2, seed=3, max_portion=MIXED_PORTION.get(which, 9))
    assert TT.total_tokens(reqs) > trace.live_tokens_rounded(), "the pool would hold everything at once"
    return trace


MODES = {
    "whole": lambda reqs, which: TT.whole(reqs),
    "decode_tail": lambda reqs, which: TT.decode_tail(reqs),
    "portions": _portions,
    "mixed": _mixed,
    "mixed_tight": _mixed_tight,
}

BF16_ONLY = ("stream_rows", "stream_tmap", "mid_rows", "gemm_tc", "gemm_tc_swiglu", "attn_prefill_mma",
             "attn_prefill_tc", "attn_decode", "attn_decode_tma", "attn_decode_tma_merged", "attn_decode_merge")
# Kernels that a replay of the two serving-shaped models must have gone through (any one of a
# tuple), by mode: a replay that falls back to another kernel fails even if its logits are right.
MUST_RUN = {
    ("E", "whole"): ["attn_prefill_tc", "gemm_tc_swiglu"],
    ("E", "decode_tail"): ["attn_prefill_tc", ("attn_decode_tma", "attn_decode_tma_merged"), "stream_tmap"],
    ("E", "portions"): ["attn_prefill_tc", "attn_prefill_mma", "gemm_tc_swiglu", "stream_tmap"],
    ("E", "mixed"): ["attn_prefill_tc", "attn_prefill_mma", ("attn_decode_tma", "attn_decode_tma_merged"), "stream_tmap"],
    ("E", "mixed_tight"): ["attn_prefill_mma", ("attn_decode_tma", "attn_decode_tma_merged")],
    ("F", "whole"): ["attn_prefill_tc", "gemm_tc_swiglu"],
    ("F", "decode_tail"): ["attn_prefill_tc", ("attn_decode_tma", "attn_decode_tma_merged"), "stream_tmap"],
    ("F", "portions"): ["attn_prefill_tc", "attn_prefill_mma", "gemm_tc_swiglu"],
    ("F", "mixed"): ["attn_prefill_mma", ("attn_decode_tma", "attn_decode_tma_merged")],
    ("F", "mixed_tight"): ["attn_prefill_mma", ("attn_decode_tma", "attn_decode_tma_merged")],
}


def _check_kernels(ran, which, mode, dtype):
    if dtype == "float32":
        assert ran["gemm_f32"] > 0 and ran["attn_generic"] > 0, ran
        assert not any(ran[k] for k in BF16_ONLY), f"the 32-bit path went through a bfloat16 kernel: {ran}"
        return
    for need in MUST_RUN.get((which, mode), []):
        names = need if isinstance(need, tuple) else (need,)
        assert any(ran[n] > 0 for n in names), f"{which} {mode}: none of {names} ran ({ran})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("peaked", [False, True], ids=["plain", "peaked"])
@pytest.mark.parametrize("which", list(TINY))
def test_replay_matches_plain(models, tmp_path, which, peaked, mode, dtype):
    d, cfg, reqs, expected, tols = models[(which, peaked)]
    trace = MODES[mode](reqs, which)
    out_dir, ran = _replay(d, dtype, trace, tmp_path)
    got = TT.read_outputs(trace, out_dir, cfg["vocab_size"])
    assert got, "the trace asked for nothing"
    tol = tols[dtype]
    d_max, where = TT.worst(got, expected)
    assert d_max <= tol, (f"{which} {'peaked' if peaked else 'plain'} {mode} {dtype}: max abs diff {d_max:.3e} at {where}, "
                          f"first beyond tolerance {tol:.3e} at {TT.first_bad(got, expected, tol)}")
    _check_kernels(ran, which, mode, dtype)


@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_replay_with_the_tcgen05_products(models, tmp_path, mode, monkeypatch):
    """The same traces with this engine's own tensor-memory product kernel in place of the
    library's for the many-row products."""
    monkeypatch.setenv("MLXFORGE_GEMM", "tcgen05")
    from mlxforge_b200.csrc import ops
    for which in ("B", "C", "E"):
        d, cfg, reqs, expected, tols = models[(which, True)]
        trace = MODES[mode](reqs, which)
        out_dir, ran = _replay(d, "bfloat16", trace, tmp_path / which)
        ops.check_kernel_status()
        # many-row products by the tcgen05 kernel, those of 17 to 128 rows by its few-row sibling
        assert ran["gemm_tc"] + ran["mid_rows"] > 0 or (mode == "portions" and which != "E"), ran
        assert which != "E" or mode == "mixed" or ran["gemm_tc"] > 0, ran
        got = TT.read_outputs(trace, out_dir, cfg["vocab_size"])
        d_max, where = TT.worst(got, expected)
        assert d_max <= tols["bfloat16"], (which, mode, d_max, where)


def test_replay_with_the_mid_rows_product(models, tmp_path, monkeypatch):
    """Steps of 17 to 128 tokens (portions of prompts beside decoded tokens) through this engine's
    own product for that many rows instead of the library's."""
    monkeypatch.setenv("MLXFORGE_MID_ROWS", "1")
    from mlxforge_b200.csrc import ops
    for which, mode in (("E", "mixed"), ("F", "portions"), ("C", "whole")):
        d, cfg, reqs, expected, tols = models[(which, True)]
        trace = MODES[mode](reqs, which)
        out_dir, ran = _replay(d, "bfloat16", trace, tmp_path / which)
        ops.check_kernel_status()
        assert ran["mid_rows"] > 0, ran
        got = TT.read_outputs(trace, out_dir, cfg["vocab_size"])
        d_max, where = TT.worst(got, expected)
        assert d_max <= tols["bfloat16"], (which, mode, d_max, where)


@pytest.mark.parametrize("which,lengths", [("B", [300, 150, 40]), ("E", [700, 290, 40])])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(tmp_path, dtype, which, lengths):
    """Three requests decoded token by token from position 0, together: the first tokens of a
    sequence (a context of one key), 300 steps of decoding across page edges and across the
    widths for which decode steps are captured, a batch that shrinks as requests end."""
    d, cfg, w = make_tiny(tmp_path, which, "bfloat16", qk_gain=6.0 if which == "B" else 2.0)
    reqs = {f"l{i}": random_prompt(cfg, n, 40 + i) for i, n in enumerate(lengths)}
    expected = {rid: P.forward_logits(cfg, w, toks) for rid, toks in reqs.items()}
    P.ROUND = P.round_bf16
    try:
        noise = max(float(np.max(np.abs(P.forward_logits(cfg, w, toks) - expected[rid]))) for rid, toks in reqs.items())
    finally:
        P.ROUND = None
    scale = max(float(np.max(np.abs(e))) for e in expected.values())
    tol = TOL_F32 * max(1.0, scale) if dtype == "float32" else BF16_NOISE_FACTOR * noise
    trace = TT.lockstep(reqs)
    out_dir, _ = _replay(d, dtype, trace, tmp_path)
    got = TT.read_outputs(trace, out_dir, cfg["vocab_size"])
    assert len(got) == sum(len(t) for t in reqs.values())
    d_max, where = TT.worst(got, expected)
    assert d_max <= tol, (f"{dtype}: max abs diff {d_max:.3e} at {where}, first beyond tolerance {tol:.3e} at "
                          f"{TT.first_bad(got, expected, tol)}")
