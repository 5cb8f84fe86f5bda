"""Each part of a layer alone: built from its registry with nothing but its own sizes and
constants, bound to random tensors, run on steps of a small mixed batch (portions of two
sequences, then single tokens) over a cache of its own, and compared with the plain
implementation's function for that part on the whole sequences.  No model is involved:
the parts are given a runtime, a step batch and a cache lane, which is all they ever see."""
from types import SimpleNamespace

import numpy as np
import pytest

import plain_llama as P
from helpers import bf16_round

pytestmark = pytest.mark.gpu

H, NH, NKV, HD, INTER, EPS, THETA = 88, 6, 2, 32, 136, 3e-6, 50000.0
LENGTHS = [45, 23]
# what each step brings of (sequence 0, sequence 1): portions, a sequence left out, single tokens
STEPS = [(20, 0), (7, 5), (0, 16), (17, 1), (1, 1)]


def torch_dtype(name):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def dev(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    import torch
    return t.detach().to("cpu", torch.float32).numpy().astype(np.float64)


def tol(dtype, scale):
    return (2e-5 if dtype == "float32" else 3e-2) * max(1.0, scale)


class Harness:
    """A runtime, a cache for one paged need and the runner's metadata builder: what a mixer needs around it."""

    def __init__(self, dtype, need=None):
        from mlxforge_b200.cache.manager import CacheLayout, CacheManager, GroupLayout
        from mlxforge_b200.engine.runtime import Runtime
        from mlxforge_b200.engine.step import ModelRunner
        self.rt = Runtime(torch_dtype(dtype))
        paged = (GroupLayout(need, 1),) if need is not None else ()
        lanes = (("paged", 0, 0),) if need is not None else (None,)
        self.cache = CacheManager(CacheLayout(paged=paged, state=(), item_lane=lanes), page_size=16, max_tokens=256,
                                  max_seqs=4, dtype=torch_dtype(dtype), device="cuda")
        stub = SimpleNamespace(graph_safe=False, spec=SimpleNamespace(vocab_size=1 << 20))
        self.runner = ModelRunner(stub, self.cache, self.rt)
        self.seqs = [self.cache.open_sequence() for _ in LENGTHS]

    def steps(self):
        """Yields (batch, rows): rows[i] = (sequence, position) of the step's i-th token."""
        from mlxforge_b200.engine.step import StepEntry
        done = [0, 0]
        for counts in STEPS:
            entries, per_seq = [], []
            for s, n in enumerate(counts):
                if n:
                    entries.append(StepEntry(self.seqs[s], [0] * n, []))
                    per_seq.append((s, n))
            self.cache.reserve([(e.seq, len(e.tokens)) for e in entries])
            batch = self.runner._build(entries)
            # the batch lays single-token sequences first
            order = sorted(range(len(per_seq)), key=lambda i: (per_seq[i][1] != 1, i))
            rows = [(per_seq[i][0], done[per_seq[i][0]] + j) for i in order for j in range(per_seq[i][1])]
            yield batch, rows
            for e in entries:
                self.cache.commit(e.seq, len(e.tokens))
            for s, n in per_seq:
                done[s] += n
        assert done == LENGTHS


def rand(rng, *shape, std=1.0):
    return bf16_round(rng.standard_normal(shape).astype(np.float32) * std)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    import torch
    from mlxforge_b200.parts.base import NORMS, PartSpec, build_part
    h = Harness(dtype)
    rng = np.random.default_rng(0)
    part = build_part(NORMS, PartSpec("rmsnorm", {"size": H, "eps": EPS}, prefix="n."), h.rt)
    assert list(part.tensor_specs()) == ["n.weight"]
    w = (1 + 0.2 * rng.standard_normal(H)).astype(np.float32)
    part.bind({"n.weight": dev(w)})
    resid, delta = rng.standard_normal((9, H)).astype(np.float32) * 2, rand(rng, 9, H)
    r = dev(resid)
    out = part.add_forward(r, dev(delta, torch_dtype(dtype)))
    want = P.rms_norm(resid.astype(np.float64) + delta, w.astype(np.float64), EPS)
    assert np.max(np.abs(host(out) - want)) < tol(dtype, 1.0)
    assert np.max(np.abs(host(r) - (resid.astype(np.float64) + delta))) < 1e-6, "the residual stream moved on, in 32-bit"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    from mlxforge_b200.parts.base import FEED_FORWARDS, PartSpec, build_part
    h = Harness(dtype)
    rng = np.random.default_rng(1)
    part = build_part(FEED_FORWARDS, PartSpec("swiglu", {"hidden_size": H, "intermediate_size": INTER}, prefix="f."), h.rt)
    w = {n: rand(rng, *s.shape, std=0.2) for n, s in part.tensor_specs().items()}
    part.bind({n: dev(a, torch_dtype(dtype)) for n, a in w.items()})
    x = rand(rng, 11, H)
    out = part.forward(dev(x, torch_dtype(dtype)), None)
    f = np.float64
    want = P.swiglu_mlp(x.astype(f), w["f.gate_proj.weight"].astype(f), w["f.up_proj.weight"].astype(f),
                        w["f.down_proj.weight"].astype(f))
    assert np.max(np.abs(host(out) - want)) < tol(dtype, np.abs(want).max())


@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_head_parts(tied):
    import torch
    from mlxforge_b200.parts.base import EMBEDDINGS, HEADS, PartSpec, build_part
    h = Harness("bfloat16")
    rng = np.random.default_rng(2)
    V = 301
    emb = build_part(EMBEDDINGS, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, prefix="e."), h.rt)
    head = build_part(HEADS, PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "tied_to": "e.weight",
                                                      "require_own": not tied}, prefix="h."), h.rt)
    table, own = rand(rng, V, H), rand(rng, V, H)
    tensors = {"e.weight": dev(table, torch.bfloat16)}
    if not tied:
        tensors["h.weight"] = dev(own, torch.bfloat16)
    emb.bind(tensors)
    head.bind(tensors)
    toks = rng.integers(0, V, size=6).astype(np.int32)
    out = torch.empty((6, H), dtype=torch.float32, device="cuda")
    emb.forward(dev(toks), out)
    assert np.array_equal(host(out), table[toks].astype(np.float64))
    x = rand(rng, 4, H)
    logits = torch.empty((4, V), dtype=torch.float32, device="cuda")
    head.forward(dev(x, torch.bfloat16), logits)
    want = x.astype(np.float64) @ (table if tied else own).astype(np.float64).T
    assert np.max(np.abs(host(logits) - want)) < 1e-3 * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_position_encoding_part(dtype):
    """The rotary part alone: rotated queries out, rotated keys and plain values into the pages
    that the step's block table names, for portions and single tokens."""
    import torch
    from mlxforge_b200.parts.base import POSITIONS, PagedKV, PartSpec, build_part
    need = PagedKV(NKV, HD, 0)
    h = Harness(dtype, need)
    rng = np.random.default_rng(3)
    part = build_part(POSITIONS, PartSpec("rope", {"head_dim": HD, "rotary_dim": HD, "theta": THETA, "scaling": None}), h.rt)
    freqs = P.rope_frequencies({"head_dim": HD, "hidden_size": H, "num_attention_heads": NH, "rope_theta": THETA})
    qkv_all = [rand(rng, n, (NH + 2 * NKV) * HD) for n in LENGTHS]
    lane = h.cache.lane(0)
    for batch, rows in h.steps():
        qkv = np.stack([qkv_all[s][p] for s, p in rows])
        q_out = torch.full((len(rows), NH * HD), float("nan"), dtype=torch_dtype(dtype), device="cuda")
        part.rotate_and_store(dev(qkv, torch_dtype(dtype)), batch, q_out, lane, NH, NKV, True)
        got_q = host(q_out).reshape(len(rows), NH, HD)
        for i, (s, p) in enumerate(rows):
            q = qkv_all[s][p][:NH * HD].reshape(NH, 1, HD).astype(np.float64)
            want = P.apply_rope(q, [p], freqs)[:, 0]
            assert np.max(np.abs(got_q[i] - want)) < tol(dtype, 1.0), (s, p)
    kp, vp = host(lane.k), host(lane.v)
    for s, n in enumerate(LENGTHS):
        for p in range(n):
            pg, slot = h.seqs[s].blocks[0][p // 16], p % 16
            k = qkv_all[s][p][NH * HD:(NH + NKV) * HD].reshape(NKV, 1, HD).astype(np.float64)
            assert np.max(np.abs(kp[pg, :, slot] - P.apply_rope(k, [p], freqs)[:, 0])) < tol(dtype, 1.0), (s, p)
            assert np.array_equal(vp[pg, :, slot], qkv_all[s][p][(NH + NKV) * HD:].reshape(NKV, HD)), (s, p)


def _attention_part(h, window=0):
    from mlxforge_b200.parts.base import MIXERS, PartSpec, build_part
    rope = PartSpec("rope", {"head_dim": HD, "rotary_dim": HD, "theta": THETA, "scaling": None})
    return build_part(MIXERS, PartSpec("attention", {"hidden_size": H, "n_heads": NH, "n_kv_heads": NKV, "head_dim": HD,
                                                     "softmax_scale": HD ** -0.5, "window": window, "position": rope},
                                       prefix="a."), h.rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [0, 11])
def test_mixer_part(dtype, window):
    """The attention mixer alone, over a cache it fills itself step by step."""
    from mlxforge_b200.parts.base import PagedKV
    h = Harness(dtype, PagedKV(NKV, HD, window))
    rng = np.random.default_rng(4)
    part = _attention_part(h, window)
    assert part.cache_need() == PagedKV(NKV, HD, window)
    w = {n: rand(rng, *s.shape, std=0.15) for n, s in part.tensor_specs().items()}
    part.bind({n: dev(a, torch_dtype(dtype)) for n, a in w.items()})
    xs = [rand(rng, n, H) for n in LENGTHS]
    f = np.float64
    freqs = P.rope_frequencies({"head_dim": HD, "hidden_size": H, "num_attention_heads": NH, "rope_theta": THETA})
    want = []
    for s, n in enumerate(LENGTHS):
        q, k, v = P.project_qkv(xs[s].astype(f), w["a.q_proj.weight"].astype(f), w["a.k_proj.weight"].astype(f),
                                w["a.v_proj.weight"].astype(f), NH, NKV, HD)
        q, k = P.apply_rope(q, range(n), freqs), P.apply_rope(k, range(n), freqs)
        want.append(P.attention(q, k, v, HD ** -0.5, window) @ w["a.o_proj.weight"].astype(f).T)
    lane = h.cache.lane(0)
    for batch, rows in h.steps():
        x = np.stack([xs[s][p] for s, p in rows])
        out = host(part.forward(dev(x, torch_dtype(dtype)), batch, lane, True))
        for i, (s, p) in enumerate(rows):
            assert np.max(np.abs(out[i] - want[s][p])) < tol(dtype, np.abs(want[s]).max()), (s, p)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part(dtype):
    """The pre-norm arrangement of four parts around the residual stream, alone."""
    import torch
    from mlxforge_b200.parts.base import BLOCKS, FEED_FORWARDS, NORMS, PagedKV, PartSpec, build_part
    h = Harness(dtype, PagedKV(NKV, HD, 0))
    rng = np.random.default_rng(5)
    mixer = _attention_part(h)
    ffn = build_part(FEED_FORWARDS, PartSpec("swiglu", {"hidden_size": H, "intermediate_size": INTER}, prefix="f."), h.rt)
    n1 = build_part(NORMS, PartSpec("rmsnorm", {"size": H, "eps": EPS}, prefix="n1."), h.rt)
    n2 = build_part(NORMS, PartSpec("rmsnorm", {"size": H, "eps": EPS}, prefix="n2."), h.rt)
    block = BLOCKS.get("prenorm")({"mixer": mixer, "mixer_norm": n1, "feed_forward": ffn, "feed_forward_norm": n2}, h.rt)
    with pytest.raises(ValueError, match="needs parts in the roles"):
        BLOCKS.get("prenorm")({"mixer": mixer, "mixer_norm": n1}, h.rt)
    w = {}
    for part in block.parts():
        for n, s in part.tensor_specs().items():
            w[n] = (1 + 0.2 * rng.standard_normal(s.shape)).astype(np.float32) if s.role == "vector" \
                else rand(rng, *s.shape, std=0.15)
    for part in block.parts():
        part.bind({n: dev(a, torch.float32 if a.ndim == 1 else torch_dtype(dtype)) for n, a in w.items()})
    xs = [rng.standard_normal((n, H)).astype(np.float32) for n in LENGTHS]
    f = np.float64
    plain_w = {"model.layers.0.input_layernorm.weight": w["n1.weight"], "model.layers.0.post_attention_layernorm.weight": w["n2.weight"]}
    for n in ("q", "k", "v", "o"):
        plain_w[f"model.layers.0.self_attn.{n}_proj.weight"] = w[f"a.{n}_proj.weight"]
    for n in ("gate", "up", "down"):
        plain_w[f"model.layers.0.mlp.{n}_proj.weight"] = w[f"f.{n}_proj.weight"]
    plain_w = {k: v.astype(f) for k, v in plain_w.items()}
    cfg = {"num_attention_heads": NH, "num_key_value_heads": NKV, "head_dim": HD, "hidden_size": H, "rms_norm_eps": EPS,
           "rope_theta": THETA}
    freqs = P.rope_frequencies(cfg)
    want = [P.decoder_block(xs[s].astype(f), plain_w, cfg, 0, range(n), freqs) for s, n in enumerate(LENGTHS)]
    lane = h.cache.lane(0)
    for batch, rows in h.steps():
        resid = dev(np.stack([xs[s][p] for s, p in rows]))
        resid, pending = block.forward(resid, None, batch, lane, True)
        out = host(resid) + host(pending)           # the last delta is left for the next norm to add
        for i, (s, p) in enumerate(rows):
            assert np.max(np.abs(out[i] - want[s][p])) < tol(dtype, np.abs(want[s]).max()), (s, p)
