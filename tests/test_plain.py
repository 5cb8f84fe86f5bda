"""The plain implementation itself: the position encoding against the reference's
committed fixtures, and properties every part must have.  CPU only."""
import os

import numpy as np

import plain_llama as P
from helpers import TINY_A, TINY_B, random_prompt, random_weights


def test_rotation_matches_reference_fixture():
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "rope_anchor.npz"))
    cfg = {"head_dim": 64, "hidden_size": 2048, "num_attention_heads": 32, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                            "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}}
    f = P.rope_frequencies(cfg)
    assert np.max(np.abs(f - g["rope_freqs"]) / g["rope_freqs"]) < 1e-6
    out = P.apply_rope(g["q_pre"].astype(np.float64), np.arange(6), f)
    # the fixture is float16 of values up to ~15: half a unit in the last place is 0.004
    assert np.max(np.abs(out - g["q_rope"])) < 0.01
    # the interleaved pairing would be far off: the half-split pairing is the right one
    x = g["q_pre"].astype(np.float64)
    ang = np.arange(6)[:, None] / f[None, :].astype(np.float64)
    inter = np.empty_like(x)
    inter[..., 0::2] = x[..., 0::2] * np.cos(ang) - x[..., 1::2] * np.sin(ang)
    inter[..., 1::2] = x[..., 0::2] * np.sin(ang) + x[..., 1::2] * np.cos(ang)
    assert np.max(np.abs(inter - g["q_rope"])) > 1.0


def test_rms_norm_and_swiglu_formulas():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 10))
    w = rng.standard_normal(10)
    y = P.rms_norm(x, w, 1e-5)
    for r in range(3):
        assert np.allclose(y[r], x[r] / np.sqrt((x[r] ** 2).mean() + 1e-5) * w)
    wg, wu, wd = rng.standard_normal((6, 10)), rng.standard_normal((6, 10)), rng.standard_normal((10, 6))
    g, u = x @ wg.T, x @ wu.T
    assert np.allclose(P.swiglu_mlp(x, wg, wu, wd), (g * (1 / (1 + np.exp(-g))) * u) @ wd.T)


def test_attention_is_causal_and_grouped():
    rng = np.random.default_rng(1)
    nh, nkv, T, hd = 4, 2, 9, 8
    q, k, v = rng.standard_normal((nh, T, hd)), rng.standard_normal((nkv, T, hd)), rng.standard_normal((nkv, T, hd))
    out = P.attention(q, k, v, 0.3).reshape(T, nh, hd)
    k2, v2 = k.copy(), v.copy()
    k2[:, 5:] += 10.0
    v2[:, 5:] -= 3.0
    out2 = P.attention(q, k2, v2, 0.3).reshape(T, nh, hd)
    assert np.allclose(out[:5], out2[:5]) and not np.allclose(out[5:], out2[5:])
    assert np.allclose(out[0, 0], v[0, 0]) and np.allclose(out[0, 3], v[1, 0]), "heads 0,1 read KV head 0; 2,3 read 1"
    # a window of 3 keeps keys j-2..j
    win = P.attention(q, k, v, 0.3, window=3).reshape(T, nh, hd)
    s = (q[0, 8] @ k[0, 6:9].T) * 0.3
    p = np.exp(s - s.max())
    assert np.allclose(win[8, 0], (p / p.sum()) @ v[0, 6:9])


def test_prefix_invariance_of_the_whole_model():
    """Logits at a position depend only on the tokens up to it."""
    for cfg, seed in ((TINY_A, 0), (TINY_B, 1)):
        w = {k: v.astype(np.float64) for k, v in random_weights(cfg, seed, 0.1).items()}
        toks = random_prompt(cfg, 40, 3)
        full = P.forward_logits(cfg, w, toks)
        part = P.forward_logits(cfg, w, toks[:17])
        assert np.max(np.abs(full[:17] - part)) < 1e-12
        assert full.shape == (40, cfg["vocab_size"])


def test_sampler_functions():
    row = np.array([0.1, 2.0, -1.0, 2.0, 0.5])
    assert P.greedy(row) == 1, "ties go to the lowest index"
    assert P.sample_token(row, 0.0, 0.9)[0] == 1
    p = np.exp(row / 0.7 - (row / 0.7).max())
    p /= p.sum()
    cdf = np.cumsum(p)
    for u in (0.0, 0.05, 0.3, 0.6, 0.99):
        assert P.sample_token(row, 0.7, u)[0] == int(np.searchsorted(cdf, u, side="right"))
    f = P.filter_logits(row, 1.0, top_k=2)
    assert np.isinf(f[[0, 2, 4]]).all() and np.isfinite(f[[1, 3]]).all()
    f = P.filter_logits(np.array([3.0, 2.0, 1.0, 0.0]), 1.0, top_p=0.7)
    assert np.isfinite(f[:2]).all() and np.isinf(f[2:]).all()       # 0.64 < 0.7 keeps the second, 0.88 stops
    f = P.filter_logits(np.array([3.0, 2.0, 1.0, 0.0]), 1.0, min_p=0.2)
    assert np.isfinite(f[:2]).all() and np.isinf(f[2:]).all()       # e^-1 = .37 stays, e^-2 = .14 goes
    x = P.apply_penalties(np.array([2.0, -2.0, 1.0, 1.0]), [0, 1, 1], repetition=2.0, frequency=0.5, presence=0.25)
    assert np.allclose(x, [1.0 - 0.5 - 0.25, -4.0 - 1.0 - 0.25, 1.0, 1.0])
    us = [P.uniform_for(3, i) for i in range(2000)]
    assert 0.0 <= min(us) and max(us) < 1.0 and abs(np.mean(us) - 0.5) < 0.03
    assert P.uniform_for(3, 5) == P.uniform_for(3, 5) != P.uniform_for(4, 5)


def test_engine_draw_is_the_plain_draw():
    from mlxforge_b200.sampling import uniform_draw
    for seed in (0, 1, 12345, 2**40 + 3):
        for i in range(50):
            assert uniform_draw(seed, i) == P.uniform_for(seed, i)


def test_rms_norm_against_the_reference_fixture():
    """``embeddings.npy -> attn_norm0.npy`` of the reference's fixtures (six positions of
    Llama-3.2-1B, layer 0's first norm, float16; tests/golden/make_rmsnorm_golden.py).  The
    norm's weight is not a fixture, but it is one vector for all positions: the weight that
    position 0 implies has to reproduce positions 1..5.  The rows' mean squares differ by a
    factor of two and are only thirty times eps, so a missing or misplaced eps, a sum in place
    of the mean, a mean over the wrong axis or a centred norm all miss by several times the
    float16 rounding that the right formula (src/model/decoder_model.cpp:206-208) stays within.
    (A weight applied as ``1 + w`` cannot be told from ``w`` without the checkpoint.)"""
    a = np.load(os.path.join(os.path.dirname(__file__), "golden", "rmsnorm_anchor.npz"))
    x, y = a["x"].astype(np.float64), a["y"].astype(np.float64)
    eps = 1e-5

    def miss(unit_norm):
        u = unit_norm(x)
        ok = np.abs(u[0]) > 1e-3                      # channels where position 0 says something about the weight
        w = y[0] / np.where(ok, u[0], 1.0)
        return float(np.abs(u[1:] * w - y[1:])[:, ok].max())

    ones = np.ones(x.shape[1])
    assert miss(lambda v: P.rms_norm(v, ones, eps)) < 2.5e-3
    wrong = {
        "no eps": lambda v: v / np.sqrt((v * v).mean(-1, keepdims=True)),
        "eps outside the root": lambda v: v / (np.sqrt((v * v).mean(-1, keepdims=True)) + eps),
        "sum for mean": lambda v: v / np.sqrt((v * v).sum(-1, keepdims=True) + eps),
        "over positions": lambda v: v / np.sqrt((v * v).mean(0, keepdims=True) + eps),
        "centred": lambda v: (v - v.mean(-1, keepdims=True)) / np.sqrt(v.var(-1, keepdims=True) + eps),
    }
    for name, f in wrong.items():
        assert miss(f) > 6e-3, name
