"""Each CUDA kernel alone against a plain NumPy reference of the same operation,
at sizes other than the engine's test models: head sizes in steps of 16, widths
and vocabularies that are no power of two, odd numbers of heads and groups,
pages in scrambled order, windows, and inputs built so that one far key or one
page's edge decides the result."""
import numpy as np
import pytest

import plain_llama as P
from helpers import bf16_round

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    import torch
    return t.detach().to("cpu", torch.float32).numpy().astype(np.float64)


def torch_dtype(name):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


# ----------------------------------------------------------------------------- embedding, norm, swiglu

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("V,H,T", [(307, 80, 5), (1000, 2048, 33), (50, 24, 1)])
def test_embed(dtype, V, H, T):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(0)
    table = bf16_round(rng.standard_normal((V, H)).astype(np.float32))
    toks = rng.integers(0, V, size=T).astype(np.int32)
    toks[0] = V - 1
    out = torch.empty((T, H), dtype=torch.float32, device="cuda")
    ops.embed(dev(table, torch_dtype(dtype)), dev(toks), out)
    assert np.array_equal(host(out), P.embed(table.astype(np.float64), toks))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,T,eps", [(80, 7, 1e-5), (2048, 3, 1e-6), (1000, 5, 3e-5), (24, 1, 1e-5)])
def test_add_rmsnorm(dtype, H, T, eps):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(1)
    td = torch_dtype(dtype)
    resid = rng.standard_normal((T, H)).astype(np.float32) * 3.0
    delta = bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    w = (1.0 + 0.3 * rng.standard_normal(H)).astype(np.float32)
    tol = 1e-5 if dtype == "float32" else 2.0 ** -7
    # plain norm
    r = dev(resid)
    out = torch.empty((T, H), dtype=td, device="cuda")
    ops.add_rmsnorm(r, None, dev(w), eps, out)
    want = P.rms_norm(resid.astype(np.float64), w.astype(np.float64), eps)
    assert np.max(np.abs(host(out) - want) / (np.abs(want) + 1.0)) < tol
    assert np.array_equal(host(r), resid)
    # add + norm: the residual moves on, in 32-bit
    ops.add_rmsnorm(r, dev(delta, td), dev(w), eps, out)
    summed = resid.astype(np.float64) + delta
    assert np.max(np.abs(host(r) - summed)) < 1e-6
    want = P.rms_norm(summed, w.astype(np.float64), eps)
    assert np.max(np.abs(host(out) - want) / (np.abs(want) + 1.0)) < tol
    # selected rows: nothing is written back
    r2 = dev(resid)
    rows = np.array([T - 1, 0], dtype=np.int32)
    out2 = torch.empty((2, H), dtype=td, device="cuda")
    ops.add_rmsnorm(r2, dev(delta, td), dev(w), eps, out2, dev(rows))
    assert np.array_equal(host(r2), resid)
    assert np.max(np.abs(host(out2) - want[rows]) / (np.abs(want[rows]) + 1.0)) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("I,T,group", [(136, 5, 8), (100, 3, 100), (8192, 2, 8)])
def test_swiglu(dtype, I, T, group):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(2)
    g = bf16_round(rng.standard_normal((T, I)).astype(np.float32) * 2)
    u = bf16_round(rng.standard_normal((T, I)).astype(np.float32))
    n = I // group
    gu = np.stack([g.reshape(T, n, group), u.reshape(T, n, group)], axis=2).reshape(T, 2 * I)
    out = torch.empty((T, I), dtype=torch_dtype(dtype), device="cuda")
    ops.swiglu(dev(gu, torch_dtype(dtype)), out, group)
    want = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u
    # relative to each value: a few float32 (2^-24) or one bfloat16 (2^-8) roundings
    rel = 2.0 ** -21 if dtype == "float32" else 2.0 ** -7
    assert np.all(np.abs(host(out) - want) <= rel * (np.abs(want) + 1e-3))


@pytest.mark.parametrize("M,N,K", [(1, 307, 80), (33, 96, 200), (70, 1000, 17), (128, 64, 64)])
def test_gemm_f32_is_ieee(M, N, K):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(3)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32)
    out = torch.empty((M, N), dtype=torch.float32, device="cuda")
    ops.gemm_f32(dev(a), dev(w), out)
    want = a.astype(np.float64) @ w.astype(np.float64).T
    # a reduced-precision product mode would be off by ~1e-3 relative; IEEE float32 by ~1e-6
    assert np.max(np.abs(host(out) - want)) < 2e-5 * np.sqrt(K)
    # rows do not depend on how many other rows there are
    out1 = torch.empty((1, N), dtype=torch.float32, device="cuda")
    ops.gemm_f32(dev(a[M // 2:M // 2 + 1]), dev(w), out1)
    assert torch.equal(out1[0], out[M // 2])


# ----------------------------------------------------------------------------- paged cache helpers

class Paged:
    """Sequences with keys and values laid out in scrambled pages, and the same
    data as plain per-sequence arrays for the reference."""

    def __init__(self, lengths, nkv, hd, page=16, dtype="float32", seed=0, extra_pages=7):
        import torch
        rng = np.random.default_rng(seed)
        self.page, self.nkv, self.hd = page, nkv, hd
        blocks = [(n + page - 1) // page for n in lengths]
        n_pages = sum(blocks) + extra_pages
        perm = rng.permutation(n_pages)
        self.k = [bf16_round(rng.standard_normal((n, nkv, hd)).astype(np.float32)) for n in lengths]
        self.v = [bf16_round(rng.standard_normal((n, nkv, hd)).astype(np.float32)) for n in lengths]
        # unused pages and the tails of last pages hold NaN: reading them shows
        kp = np.full((n_pages, nkv, page, hd), np.nan, dtype=np.float32)
        vp = np.full((n_pages, nkv, page, hd), np.nan, dtype=np.float32)
        self.table = np.full((len(lengths), max(blocks)), -1, dtype=np.int32)
        at = 0
        for s, n in enumerate(lengths):
            for b in range(blocks[s]):
                pg = perm[at]
                at += 1
                self.table[s, b] = pg
                m = min(page, n - b * page)
                kp[pg, :, :m] = self.k[s][b * page:b * page + m].transpose(1, 0, 2)
                vp[pg, :, :m] = self.v[s][b * page:b * page + m].transpose(1, 0, 2)
        td = torch_dtype(dtype)
        self.k_pool, self.v_pool = dev(kp, td), dev(vp, td)
        self.table_dev = dev(self.table)

    def reference(self, q, seq, pos, scale, window=0):
        """q [nh, hd] -> [nh, hd] over keys [lo, pos] of sequence seq."""
        nh = q.shape[0]
        rep = nh // self.nkv
        lo = max(0, pos - window + 1) if window > 0 else 0
        out = np.empty_like(q, dtype=np.float64)
        for h in range(nh):
            k = self.k[seq][lo:pos + 1, h // rep].astype(np.float64)
            v = self.v[seq][lo:pos + 1, h // rep].astype(np.float64)
            s = (k @ q[h].astype(np.float64)) * scale
            p = np.exp(s - s.max())
            out[h] = (p / p.sum()) @ v
        return out


ATTN_CASES = [
    # nh, nkv, hd, lengths, window
    (4, 2, 16, [1, 17, 40], 0),
    (6, 1, 32, [300, 5, 129], 0),
    (5, 5, 48, [64, 65, 200], 0),
    (32, 8, 64, [1000, 257], 0),
    (8, 2, 128, [130, 31], 0),
    (3, 1, 256, [70], 0),
    (40, 2, 64, [90, 33], 0),          # 20 query heads per KV head: two groups of 16
    (4, 2, 32, [300, 40, 129], 37),    # a window
    (8, 2, 64, [3000, 700, 45], 0),    # head size 64 over several splits of the keys
    (8, 2, 64, [1500, 300], 600),      # a window that spans splits and tiles
    (4, 4, 64, [2100, 129], 100),      # a window inside one tile, far from the start
]


@pytest.mark.parametrize("case", ATTN_CASES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_generic(case, dtype):
    import torch
    from mlxforge_b200.csrc import ops
    nh, nkv, hd, lengths, window = case
    pc = Paged(lengths, nkv, hd, dtype=dtype, seed=hd)
    rng = np.random.default_rng(5)
    # queries: the last token of every sequence, plus a run of tokens in the middle of the first
    toks = [(s, n - 1) for s, n in enumerate(lengths)] + [(0, p) for p in range(max(0, lengths[0] - 5), lengths[0] - 1)]
    q = bf16_round(rng.standard_normal((len(toks), nh, hd)).astype(np.float32))
    out = torch.empty((len(toks), nh * hd), dtype=torch_dtype(dtype), device="cuda")
    scale = hd ** -0.5
    ops.attention_generic(dev(q.reshape(len(toks), -1), torch_dtype(dtype)), pc.k_pool, pc.v_pool, out,
                          dev(np.array([p for _, p in toks], dtype=np.int32)),
                          dev(np.array([s for s, _ in toks], dtype=np.int32)), pc.table_dev, pc.page, nh, nkv, hd,
                          scale, window)
    got = host(out).reshape(len(toks), nh, hd)
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    for i, (s, p) in enumerate(toks):
        want = pc.reference(q[i], s, p, scale, window)
        assert np.max(np.abs(got[i] - want)) < tol, (i, s, p)


DECODE_CASES = ATTN_CASES + [(32, 8, 64, [2100, 700, 1, 513, 512], 0), (4, 1, 64, [900, 40], 300),
                                               (8, 2, 64, [5000, 4097, 2048, 2049, 300], 0),
                                               (8, 2, 64, [5000, 2300, 640], 2500),
                                               (8, 8, 64, [600 + 7 * i for i in range(30)], 0),    # two items to a block
                                               (8, 8, 64, [600 + 7 * i for i in range(44)], 0),    # more: merge kernel
                                               # head size 128: two boxes per granule, one block per SM
                                               (8, 2, 128, [3000, 700, 45], 0), (24, 8, 128, [5000, 2300, 640], 2500),
                                               (12, 4, 128, [600 + 7 * i for i in range(20)], 0),
                                               (16, 1, 128, [900, 40, 1], 300),                    # 16 heads to a group: two stages
                                               (8, 8, 128, [600 + 7 * i for i in range(44)], 0)]
# head sizes 64 and 128 have three forms of the kernel; the others one
DECODE_FORMS = [(c, f) for c in DECODE_CASES for f in (("tma", "tma, merge kernel", "no tma") if c[2] in (64, 128) else ("tma",))]


@pytest.mark.parametrize("case,tma", DECODE_FORMS)
def test_attention_decode(case, tma):
    """Head sizes 64 and 128 have the TMA kernel, which merges its splits itself (the block that finishes a
    group's last split; run twice here: the tickets must be back at zero) or leaves them to the
    merge kernel, and the kernel without tensor copies."""
    import torch
    from mlxforge_b200.csrc import ops
    nh, nkv, hd, lengths, window = case
    old = ops.set_decode_tma(tma != "no tma")
    old_merge = ops.set_decode_merge_inside(tma == "tma")
    try:
        for _ in range(2):
            _attention_decode_case(case)
            ops.check_kernel_status()
    finally:
        ops.set_decode_tma(old)
        ops.set_decode_merge_inside(old_merge)


def _attention_decode_case(case):
    import torch
    from mlxforge_b200.csrc import ops
    nh, nkv, hd, lengths, window = case
    pc = Paged(lengths, nkv, hd, dtype="bfloat16", seed=hd + 1)
    rng = np.random.default_rng(6)
    n = len(lengths)
    q = bf16_round(rng.standard_normal((n, nh, hd)).astype(np.float32))
    scale = hd ** -0.5
    pos = np.array([m - 1 for m in lengths], dtype=np.int32)
    max_ctx = max(lengths) + 3
    n_o, n_ml = ops.attention_decode_scratch(n, nh, hd, max_ctx)
    out = torch.full((n, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.attention_decode(dev(q.reshape(n, -1), torch.bfloat16), pc.k_pool, pc.v_pool, out,
                         torch.full((n_o,), float("nan"), dtype=torch.float32, device="cuda"),
                         torch.full((n_ml,), float("nan"), dtype=torch.float32, device="cuda"),
                         dev(pos), dev(np.arange(n, dtype=np.int32)), pc.table_dev, pc.page, nh, nkv, hd, scale,
                         window, max_ctx)
    got = host(out).reshape(n, nh, hd)
    for s in range(n):
        want = pc.reference(q[s], s, int(pos[s]), scale, window)
        assert np.max(np.abs(got[s] - want)) < 1.5e-2, (s, np.max(np.abs(got[s] - want)))


@pytest.mark.parametrize("kernel", ["generic32", "generic16", "decode"])
def test_one_far_key_decides(kernel):
    """Among a thousand keys one, far back and at the first slot of a page, matches
    the query: the output must be that key's value.  A kernel that drops a key, a
    page or a split shows here, where random scores would hide it."""
    import torch
    from mlxforge_b200.csrc import ops
    nh, nkv, hd, n = 8, 2, 64, 1000
    dtype = "float32" if kernel == "generic32" else "bfloat16"
    for special in (0, 16, 255, 256, 511, 640, 999):
        pc = Paged([n], nkv, hd, dtype="float32", seed=special)
        q = np.zeros((1, nh, hd), dtype=np.float32)
        for h in range(nh):
            pc.k[0][:, h // 4] *= 0.05
            q[0, h] = 1.0
        pc.k[0][special, :, :] = 4.0            # score 4 * 64 / 8 = 32 against ~0 for the rest
        pc2 = Paged.__new__(Paged)
        # rebuild the pools from the edited arrays
        pc2.__dict__.update(pc.__dict__)
        kp = np.full(tuple(pc.k_pool.shape), np.nan, dtype=np.float32)
        for b in range(pc.table.shape[1]):
            m = min(16, n - b * 16)
            kp[pc.table[0, b], :, :m] = pc.k[0][b * 16:b * 16 + m].transpose(1, 0, 2)
        td = torch_dtype(dtype)
        k_pool, v_pool = dev(kp, td), pc.v_pool.to(td)
        out = torch.empty((1, nh * hd), dtype=td, device="cuda")
        args = (dev(np.array([n - 1], dtype=np.int32)), dev(np.array([0], dtype=np.int32)), pc.table_dev, 16, nh,
                nkv, hd, hd ** -0.5, 0)
        if kernel == "decode":
            n_o, n_ml = ops.attention_decode_scratch(1, nh, hd, n)
            ops.attention_decode(dev(q.reshape(1, -1), td), k_pool, v_pool, out,
                                 torch.empty(n_o, dtype=torch.float32, device="cuda"),
                                 torch.empty(n_ml, dtype=torch.float32, device="cuda"), *args, n)
        else:
            ops.attention_generic(dev(q.reshape(1, -1), td), k_pool, v_pool, out, *args)
        got = host(out).reshape(nh, hd)
        for h in range(nh):
            assert np.max(np.abs(got[h] - pc.v[0][special, h // 4])) < 2e-2, (special, h)


def _decisive_pools(pc, n, td):
    """The pools of ``pc`` rebuilt from its (edited) key arrays; tails and unused pages stay NaN."""
    kp = np.full(tuple(pc.k_pool.shape), np.nan, dtype=np.float32)
    for b in range(pc.table.shape[1]):
        m = min(pc.page, n - b * pc.page)
        kp[pc.table[0, b], :, :m] = pc.k[0][b * pc.page:b * pc.page + m].transpose(1, 0, 2)
    return dev(kp, td), pc.v_pool.to(td)


DECISIVE_KERNELS = {
    # name: (head size, prefill?, tcgen05 prefill, decode with tensor copies, merge inside)
    "prefill tcgen05 64": (64, True, True, True, True),
    "prefill tcgen05 128": (128, True, True, True, True),
    "prefill mma.sync 64": (64, True, False, True, True),
    "prefill mma.sync 48": (48, True, False, True, True),
    "decode tensor copies": (64, False, True, True, True),
    "decode tensor copies, merge kernel": (64, False, True, True, False),
    "decode 64 without tensor copies": (64, False, True, False, True),
    "decode 128": (128, False, True, True, True),
    "decode 128, merge kernel": (128, False, True, True, False),
    "decode 128 without tensor copies": (128, False, True, False, True),
}


@pytest.mark.parametrize("hd", [64, 128])
def test_decode_attention_reads_a_stage_before_the_next_copy_lands(hd):
    """The decode attention's ring of keys and values is read by ordinary loads and refilled by the copy
    engine, as the streamed products' ring is: with queries of zero every key weighs the same, the values
    say which tile of 128 keys they belong to, and a granule of 16 values read from the copy that came
    next moves the average by more than rounding does.  Many launches, eight sequences each.  (This kernel
    has not been seen to fail without its fence, as the streamed product has; the test guards the ring.)"""
    import torch
    from mlxforge_b200.csrc import ops
    n_seq, ctx, nh, nkv, page = 8, 1024, 8, 2, 16
    pages_per_seq = ctx // page
    n_pages = n_seq * pages_per_seq
    gen = torch.Generator(device="cuda").manual_seed(3)
    order = torch.randperm(n_pages, generator=gen, device="cuda").to(torch.int32)
    table = order.view(n_seq, pages_per_seq).contiguous()
    k_pool = torch.randn((n_pages, nkv, page, hd), generator=gen, device="cuda").to(torch.bfloat16)
    v_pool = torch.empty((n_pages, nkv, page, hd), dtype=torch.bfloat16, device="cuda")
    key = torch.arange(ctx, device="cuda")
    code = (((key // 128) % 7) * 32).to(torch.float32)                     # 0 .. 192 by tile of 128 keys
    for s_ in range(n_seq):
        for h in range(nkv):
            vals = code + 8.0 * h + s_                                          # exact in bfloat16 (integers up to 215)
            v_pool[table[s_].long(), h] = vals.view(pages_per_seq, page, 1).expand(-1, -1, hd).to(torch.bfloat16)
    q = torch.zeros((n_seq, nh * hd), dtype=torch.bfloat16, device="cuda")
    positions = torch.full((n_seq,), ctx - 1, dtype=torch.int32, device="cuda")
    seq_of = torch.arange(n_seq, dtype=torch.int32, device="cuda")
    n_o, n_ml = ops.attention_decode_scratch(n_seq, nh, hd, ctx)
    part_o = torch.empty(n_o, dtype=torch.float32, device="cuda")
    part_ml = torch.empty(n_ml, dtype=torch.float32, device="cuda")
    want = torch.empty((n_seq, nh, hd), dtype=torch.float64, device="cuda")
    for s_ in range(n_seq):
        for h in range(nh):
            want[s_, h] = float(code.double().mean()) + 8.0 * (h // (nh // nkv)) + s_
    out = torch.empty((n_seq, nh * hd), dtype=torch.bfloat16, device="cuda")
    from mlxforge_b200.csrc import binding
    before = binding.kernel_launches()
    for launch in range(60):
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        ops.attention_decode(q, k_pool, v_pool, out, part_o, part_ml, positions, seq_of, table, page, nh, nkv, hd,
                             hd ** -0.5, 0, ctx)
        torch.cuda.synchronize()
        err = (out.double().view(n_seq, nh, hd) - want).abs()
        assert float(err.max()) < 0.6, f"launch {launch}: an average is off by {float(err.max()):.2f} (a stale granule moves it by 0.5 to 3)"
    ops.check_kernel_status()
    after = binding.kernel_launches()
    assert (after["attn_decode_tma"] + after["attn_decode_tma_merged"]) - (before["attn_decode_tma"] + before["attn_decode_tma_merged"]) == 60


@pytest.mark.parametrize("window", [0, 600])
@pytest.mark.parametrize("kernel", list(DECISIVE_KERNELS))
def test_one_key_decides_at_every_edge(kernel, window):
    """One key among 1400 matches the queries; everything else scores about zero.  Rows that may
    see it must return its value, rows that may not must return the average of what they do
    see.  The key is put at the window's first position of some row and just before it, at a
    query's own position and just after it (the causal edge), at the first and last slot of a
    page, on both sides of the borders of 64-key and 128-key tiles and of 128-query tiles, and
    in another split of the keys than the query.  With random scores an edge that is off by one
    key moves the output by a thousandth, far inside any tolerance; here it moves it by about 1."""
    import torch
    from mlxforge_b200.csrc import ops
    hd, prefill, tc, tma, merge_inside = DECISIVE_KERNELS[kernel]
    nh, nkv, n = 4, 2, 1400
    q_len = 300 if prefill else 1
    first = n - q_len                                   # position of the first query row
    # key positions to try: relative to the rows' windows, to the causal edge, to pages and tiles
    specials = {n - 1, n - 2, first, first + 1, first + 127, first + 128, first + 129, 1023, 1024, 1039, 1040, 511, 512}
    if window:
        specials |= {n - window, n - window - 1, first - window + 1, first - window, first - window + 128,
                     n - window - 16, 800, 801}
    else:
        specials |= {0, 15, 16, 63, 64, 127, 128}
    old_tma, old_merge = ops.set_decode_tma(tma), ops.set_decode_merge_inside(merge_inside)
    ops.set_prefill_tcgen05(tc)
    try:
        for special in sorted(p for p in specials if 0 <= p < n):
            pc = Paged([n], nkv, hd, dtype="float32", seed=special % 97)
            pc.k[0][:] *= 0.05
            pc.k[0][special] = 4.0                      # score 4 * hd / sqrt(hd) >= 27 against ~0 for the rest
            k_pool, v_pool = _decisive_pools(pc, n, torch.bfloat16)
            q = np.ones((q_len, nh, hd), dtype=np.float32)
            out = torch.full((q_len, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
            qd = dev(q.reshape(q_len, -1), torch.bfloat16)
            scale = hd ** -0.5
            if prefill:
                ops.attention_prefill(qd, k_pool, v_pool, out, dev(np.array([0], dtype=np.int32)),
                                      dev(np.array([q_len], dtype=np.int32)), dev(np.array([n], dtype=np.int32)), 0,
                                      q_len, pc.table_dev, pc.page, nh, nkv, hd, scale, window)
            else:
                n_o, n_ml = ops.attention_decode_scratch(1, nh, hd, n)
                ops.attention_decode(qd, k_pool, v_pool, out, torch.empty(n_o, dtype=torch.float32, device="cuda"),
                                     torch.empty(n_ml, dtype=torch.float32, device="cuda"),
                                     dev(np.array([n - 1], dtype=np.int32)), dev(np.array([0], dtype=np.int32)),
                                     pc.table_dev, pc.page, nh, nkv, hd, scale, window, n)
            ops.check_kernel_status()
            got = host(out).reshape(q_len, nh, hd)
            for j in range(q_len):
                pos = first + j
                lo = max(0, pos - window + 1) if window else 0
                want = pc.reference(q[j], 0, pos, scale, window)
                d = np.max(np.abs(got[j] - want))
                assert d < 2e-2, (kernel, window, special, "row", j, "pos", pos, "sees it" if lo <= special <= pos else "must not see it", d)
    finally:
        ops.set_decode_tma(old_tma)
        ops.set_decode_merge_inside(old_merge)
        ops.set_prefill_tcgen05(True)


# ----------------------------------------------------------------------------- rope + cache write

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (6, 1, 32, 32), (5, 5, 48, 48), (3, 1, 64, 32), (2, 2, 32, 0)])
def test_rope_kv_write(dtype, nh, nkv, hd, rot):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(7)
    td = torch_dtype(dtype)
    page, n_pages = 16, 12
    # two sequences: tokens 30..36 of the first (crossing a page edge at 32), token 5 of the second
    seqs = np.array([0] * 7 + [1], dtype=np.int32)
    poss = np.array(list(range(30, 37)) + [5], dtype=np.int32)
    table = np.array([[7, 2, 9], [4, -1, -1]], dtype=np.int32)
    T = len(seqs)
    qkv = bf16_round(rng.standard_normal((T, (nh + 2 * nkv) * hd)).astype(np.float32))
    freqs = np.power(np.float32(10000.0), np.arange(0, max(rot, 2), 2, dtype=np.float32) / np.float32(max(rot, 2)))
    k_pool = torch.zeros((n_pages, nkv, page, hd), dtype=td, device="cuda")
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty((T, nh * hd), dtype=td, device="cuda")
    ops.rope_kv_write(dev(qkv, td), dev(poss), dev(seqs), dev(table), page, dev(freqs) if rot else None, q_out,
                      k_pool, v_pool, nh, nkv, hd, rot, True, dtype == "float32")
    x = qkv.astype(np.float64).reshape(T, nh + 2 * nkv, hd)

    def rotate(heads):   # [T, h, hd]
        if rot == 0:
            return heads
        r = P.apply_rope(heads[..., :rot].transpose(1, 0, 2), poss, freqs).transpose(1, 0, 2)
        return np.concatenate([r, heads[..., rot:]], axis=-1)

    tol = 1e-5 if dtype == "float32" else 2.0 ** -6
    assert np.max(np.abs(host(q_out).reshape(T, nh, hd) - rotate(x[:, :nh]))) < tol * 4
    want_k, want_v = rotate(x[:, nh:nh + nkv]), x[:, nh + nkv:]
    kp, vp = host(k_pool), host(v_pool)
    written = np.zeros((n_pages, page), dtype=bool)
    for t in range(T):
        pg, slot = table[seqs[t], poss[t] // page], poss[t] % page
        written[pg, slot] = True
        assert np.max(np.abs(kp[pg, :, slot] - want_k[t])) < tol * 4
        assert np.max(np.abs(vp[pg, :, slot] - want_v[t])) < 1e-6
    untouched = ~written                      # pools are [page][kv head][slot][channel]
    assert np.all(kp.transpose(0, 2, 1, 3)[untouched] == 0) and np.all(vp.transpose(0, 2, 1, 3)[untouched] == 0), \
        "nothing else in the pools was touched"


# ----------------------------------------------------------------------------- few-row products

@pytest.mark.parametrize("M", [17, 32, 33, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(304, 80), (2048, 2048), (3072, 2048), (1000, 136), (96, 200), (130, 64), (5000, 520),
                                 (2048, 8192), (40000, 512), (300, 3080)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_mid_linear(M, N, K, out_dtype):
    """The product for 17 to 128 rows: matrices of a few tiles that every block gets a piece of
    (partial sums, tickets), of many tiles, tiles that end beyond N, K tails; run twice on the
    same scratch, which starts full of NaN (the tickets must be back at zero, nothing stale read)."""
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(M * 7 + N)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = bf16_round((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32))
    want = x.astype(np.float64) @ w.astype(np.float64).T
    td = torch_dtype(out_dtype)
    scratch = torch.full((ops.mid_rows_scratch(M),), float("nan"), dtype=torch.float32, device="cuda")
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    torch.cuda.synchronize()      # the kernel fetches W before it waits for the kernel before it: W must be there
    for _ in range(2):
        out = torch.full((M, N), float("nan"), dtype=td, device="cuda")
        ops.mid_linear(xd, wd, out, scratch)
        ops.check_kernel_status()
        got = host(out)
        tol = 2e-5 * np.sqrt(K) if out_dtype == "float32" else 2.0 ** -7 * max(1.0, np.abs(want).max())
        assert np.max(np.abs(got - want)) < tol, np.max(np.abs(got - want))


@pytest.mark.parametrize("M,I,K", [(17, 136, 80), (64, 8192, 2048), (100, 64, 96), (128, 1000, 520)])
def test_mid_linear_swiglu(M, I, K):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(M + I)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    wg = bf16_round((rng.standard_normal((I, K)) / np.sqrt(K)).astype(np.float32))
    wu = bf16_round((rng.standard_normal((I, K)) / np.sqrt(K)).astype(np.float32))
    gu = np.stack([wg.reshape(I // 8, 8, K), wu.reshape(I // 8, 8, K)], axis=1).reshape(2 * I, K)
    g = x.astype(np.float64) @ wg.astype(np.float64).T
    u = x.astype(np.float64) @ wu.astype(np.float64).T
    want = g / (1.0 + np.exp(-g)) * u
    scratch = torch.full((ops.mid_rows_scratch(M),), float("nan"), dtype=torch.float32, device="cuda")
    xd, gud = dev(x, torch.bfloat16), dev(gu, torch.bfloat16)
    torch.cuda.synchronize()      # the kernel fetches W before it waits for the kernel before it: W must be there
    for _ in range(2):
        out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.mid_linear(xd, gud, out, scratch, swiglu=True)
        ops.check_kernel_status()
        assert np.max(np.abs(host(out) - want)) < 2.0 ** -6 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("M,N,K", [(16, 2048, 8192), (16, 16384, 2048), (8, 16384, 2048), (12, 16384, 3072), (16, 28672, 4096),
                                   (3, 128256, 64), (16, 50000, 128), (8, 20000, 1536), (13, 2050, 192)])
@pytest.mark.parametrize("tensor_copies", [True, False])
def test_stream_linear_reads_a_stage_before_the_next_copy_lands(M, N, K, tensor_copies):
    """A stage of the ring is read by ordinary loads and overwritten by the copy engine: the reads must be
    done before the stage is handed back.  Weights that say which tile and which quarter of K they come
    from, rows of x that each pick one sixteenth of K, float32 sums of small integers: every output is
    exact, and a lane that read the next copy's bytes shows as another tile's or quarter's value.  (Without
    the proxy fence before the hand-back the first size was wrong in 595 of 600 launches.)"""
    import torch
    from mlxforge_b200.csrc import ops
    k = torch.arange(K, device="cuda")
    x = (k[None, :] // -(-K // 16) == torch.arange(M, device="cuda")[:, None]).to(torch.bfloat16)
    n = torch.arange(N, device="cuda")
    w = (((n[:, None] // 16) % 64) + 64 * (k[None, :] * 4 // K)).to(torch.bfloat16)        # at most 255: exact in bfloat16
    want = x.double() @ w.double().T
    out = torch.empty((M, N), dtype=torch.float32, device="cuda")
    ops.set_stream_tensor_copies(tensor_copies)      # False: the ring of row-segment copies, which has the same fence
    try:
        for launch in range(30):
            out.fill_(float("nan"))
            torch.cuda.synchronize()
            ops.stream_linear(x, w, out)
            torch.cuda.synchronize()
            wrong = (out.double() != want).nonzero()
            assert wrong.numel() == 0, (f"launch {launch}: {wrong.shape[0]} wrong sums, first at row {int(wrong[0, 0])} column "
                                        f"{int(wrong[0, 1])}: {float(out[wrong[0, 0], wrong[0, 1]])} for "
                                        f"{float(want[wrong[0, 0], wrong[0, 1]])}")
        ops.check_kernel_status()
    finally:
        ops.set_stream_tensor_copies(True)


@pytest.mark.parametrize("M,N,K", [(1, 304, 80), (8, 2048, 2048), (5, 307, 136), (16, 96, 200), (9, 1000, 64),
                                   (3, 128256, 64), (8, 16, 8192), (2, 5000, 520), (7, 40, 1032), (16, 4737, 1536),
                                   (3, 9000, 512), (11, 4744, 1024), (8, 300, 3072), (13, 2050, 192), (8, 3000, 576),
                                   (16, 700, 1088), (4, 5000, 320)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("tensor_copies", [True, False])
def test_stream_linear(M, N, K, out_dtype, tensor_copies):
    """The bulk-copy version: tiles that end inside a stage, K tails, more tiles than blocks;
    with one tensor copy per stage (widths of whole stages) and with a copy per row segment."""
    from mlxforge_b200.csrc import ops
    ops.set_stream_tensor_copies(tensor_copies)
    try:
        _check_stream_linear(M, N, K, out_dtype)
    finally:
        ops.set_stream_tensor_copies(True)


def _check_stream_linear(M, N, K, out_dtype):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(M * 1000 + N)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = bf16_round(rng.standard_normal((N, K)).astype(np.float32))
    out = torch.full((M, N), float("nan"), dtype=torch_dtype(out_dtype), device="cuda")
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    torch.cuda.synchronize()      # the kernel fetches W before it waits for the kernel before it: W must be there
    ops.stream_linear(xd, wd, out)
    ops.check_kernel_status()
    want = x.astype(np.float64) @ w.astype(np.float64).T
    tol = 3e-6 * np.sqrt(K) * 4 if out_dtype == "float32" else 2.0 ** -8 * np.abs(want).max() + 1e-3
    assert np.max(np.abs(host(out) - want)) < tol
    if M > 1:
        # a row's result does not depend on how many rows there are.  (The same W on the device: a
        # W converted by the kernel launched just before would be read before that kernel is done.)
        out1 = torch.empty((1, N), dtype=torch_dtype(out_dtype), device="cuda")
        x1 = dev(x[M - 1:M], torch.bfloat16)
        torch.cuda.synchronize()
        ops.stream_linear(x1, wd, out1)
        assert torch.equal(out1[0], out[M - 1])
    # the swiglu epilogue, when the shape allows it
    if N % 16 == 0 and out_dtype == "bfloat16":
        I = N // 2
        wg, wu = w[:I] * 0.2, w[I:] * 0.2
        gu = bf16_round(np.stack([wg.reshape(I // 8, 8, K), wu.reshape(I // 8, 8, K)], axis=1).reshape(N, K))
        act = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device="cuda")
        gud = dev(gu, torch.bfloat16)
        torch.cuda.synchronize()
        ops.stream_linear(xd, gud, act, swiglu=True)
        gg = x.astype(np.float64) @ bf16_round(wg).astype(np.float64).T
        uu = x.astype(np.float64) @ bf16_round(wu).astype(np.float64).T
        want = gg / (1 + np.exp(-gg)) * uu
        assert np.all(np.abs(host(act) - want) <= 2.0 ** -7 * (np.abs(want) + 1e-2))
    ops.check_kernel_status()


def test_few_row_products_refuse_what_they_cannot_do():
    import torch
    from mlxforge_b200.csrc import ops
    from mlxforge_b200.csrc.binding import KernelError
    x = torch.zeros((2, 12), dtype=torch.bfloat16, device="cuda")          # K no multiple of 8
    w = torch.zeros((16, 12), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(KernelError, match="refused"):
        ops.stream_linear(x, w, torch.zeros((2, 16), dtype=torch.bfloat16, device="cuda"))
    x = torch.zeros((17, 16), dtype=torch.bfloat16, device="cuda")         # more rows than the streamed product takes
    with pytest.raises(KernelError, match="refused"):
        ops.stream_linear(x, torch.zeros((16, 16), dtype=torch.bfloat16, device="cuda"),
                          torch.zeros((17, 16), dtype=torch.bfloat16, device="cuda"))
    x = torch.zeros((129, 16), dtype=torch.bfloat16, device="cuda")        # and than the 17-to-128-row product takes
    with pytest.raises(KernelError, match="refused"):
        ops.mid_linear(x, torch.zeros((16, 16), dtype=torch.bfloat16, device="cuda"),
                       torch.zeros((129, 16), dtype=torch.bfloat16, device="cuda"),
                       torch.zeros(ops.mid_rows_scratch(129), dtype=torch.float32, device="cuda"))


# ----------------------------------------------------------------------------- prefill attention

@pytest.mark.parametrize("case", ATTN_CASES)
def test_attention_prefill(case):
    """Portions of several sequences in one launch: a whole prompt, the tail of a
    longer context, a two-token portion; checked row by row against the plain formula."""
    import torch
    from mlxforge_b200.csrc import ops
    nh, nkv, hd, lengths, window = case
    pc = Paged(lengths, nkv, hd, dtype="bfloat16", seed=hd + 2)
    rng = np.random.default_rng(8)
    # per sequence: how many of its last tokens are the new ones
    q_lens = [n if i == 0 else (2 if i == 1 else min(n, 67)) for i, n in enumerate(lengths)]
    q_lens = [min(ql, n) for ql, n in zip(q_lens, lengths)]
    starts = np.cumsum([3] + q_lens[:-1]).astype(np.int32)        # 3 unrelated rows come first
    T = 3 + sum(q_lens)
    q = bf16_round(rng.standard_normal((T, nh, hd)).astype(np.float32))
    out = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    scale = hd ** -0.5
    # a table with one more leading row than sequences, to exercise table_row0
    table = np.concatenate([np.full((1, pc.table.shape[1]), -1, dtype=np.int32), pc.table])
    ops.attention_prefill(dev(q.reshape(T, -1), torch.bfloat16), pc.k_pool, pc.v_pool, out, dev(starts),
                          dev(np.array(q_lens, dtype=np.int32)), dev(np.array(lengths, dtype=np.int32)), 1,
                          max(q_lens), dev(table), pc.page, nh, nkv, hd, scale, window)
    got = host(out).reshape(T, nh, hd)
    assert np.isnan(got[:3]).all(), "rows that belong to no portion are left alone"
    for s, (n, ql) in enumerate(zip(lengths, q_lens)):
        for j in range(ql):
            pos = n - ql + j
            want = pc.reference(q[starts[s] + j], s, pos, scale, window)
            d = np.max(np.abs(got[starts[s] + j] - want))
            assert d < 1.5e-2, (s, j, pos, d)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("nh,nkv,lengths,q_lens,window", [
    (8, 2, [700, 130, 513], [700, 130, 300], 0),          # whole prompts and the tail of a longer context
    (4, 4, [300, 640], [300, 200], 100),                  # a window shorter than a key tile
    (4, 1, [128, 2000, 5], [128, 129, 2], 0),             # exactly one tile; one query past a tile; two tokens
    (4, 2, [1500], [1100], 700),                          # a window over several key tiles
    (32, 8, [2048], [2048], 0),
])
def test_attention_prefill_tcgen05(nh, nkv, lengths, q_lens, window, hd):
    """The tcgen05 kernel (head size 64 or 128, a portion of 128 tokens or more in the launch):
    every row of every portion against the plain formula, unused pages and page tails full of NaN."""
    import torch
    from mlxforge_b200.csrc import ops
    if hd == 128 and nh == 32:
        nh, nkv = 8, 2                                             # the plain formula is slow
    pc = Paged(lengths, nkv, hd, dtype="bfloat16", seed=len(lengths) + nh)
    rng = np.random.default_rng(18)
    starts = np.cumsum([3] + q_lens[:-1]).astype(np.int32)        # 3 unrelated rows come first
    T = 3 + sum(q_lens) + 2                                        # and 2 after
    q = bf16_round(rng.standard_normal((T, nh, hd)).astype(np.float32))
    scale = hd ** -0.5
    table = np.concatenate([np.full((1, pc.table.shape[1]), -1, dtype=np.int32), pc.table])
    args = (dev(q.reshape(T, -1), torch.bfloat16), pc.k_pool, pc.v_pool)
    meta = (dev(starts), dev(np.array(q_lens, dtype=np.int32)), dev(np.array(lengths, dtype=np.int32)), 1,
            max(q_lens), dev(table), pc.page, nh, nkv, hd, scale, window)
    outs = []
    for tc in (True, False):
        ops.set_prefill_tcgen05(tc)
        try:
            out = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.attention_prefill(*args, out, *meta)
            ops.check_kernel_status()
        finally:
            ops.set_prefill_tcgen05(True)
        outs.append(host(out).reshape(T, nh, hd))
    got, other = outs
    assert np.isnan(got[:3]).all() and np.isnan(got[-2:]).all(), "rows that belong to no portion are left alone"
    step = 1 if sum(q_lens) <= 800 else 7                          # the plain formula is slow: every 7th row of long ones
    for s, (n, ql) in enumerate(zip(lengths, q_lens)):
        rows = sorted(set(range(0, ql, step)) | {0, ql - 1, min(ql - 1, 127), min(ql - 1, 128)})
        for j in rows:
            pos = n - ql + j
            want = pc.reference(q[starts[s] + j], s, pos, scale, window)
            d = np.max(np.abs(got[starts[s] + j] - want))
            assert d < 1.5e-2, (s, j, pos, d)
        sl = slice(starts[s], starts[s] + ql)
        assert np.max(np.abs(got[sl] - other[sl])) < 2e-2, "the two kernels agree on every row"


# ----------------------------------------------------------------------------- tcgen05 product

@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (2048, 3072, 2048), (300, 520, 136), (17, 96, 80),
                                   (129, 257, 72), (1000, 128, 4096), (64, 16384, 512),
                                   # tiles that hang over M, N and K in the middle of a block's run of
                                   # tiles: every barrier is used again after such a box
                                   (300, 30000, 72), (200, 20000, 200)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_gemm_tcgen05(M, N, K, out_dtype):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(M + N + K)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = bf16_round(rng.standard_normal((N, K)).astype(np.float32))
    out = torch.full((M, N), float("nan"), dtype=torch_dtype(out_dtype), device="cuda")
    ops.gemm_bf16(dev(x, torch.bfloat16), dev(w, torch.bfloat16), out)
    ops.check_kernel_status()
    want = x.astype(np.float64) @ w.astype(np.float64).T
    got = host(out)
    assert np.isfinite(got).all()
    # Forward error bound of a float32 sum: each of the K additions may lose 2^-23 (the
    # tensor cores truncate) of the running magnitude, which sum(|x||w|) bounds.  A wrong
    # tile, a dropped k-step or a 16-bit accumulator would be orders of magnitude beyond it.
    bound = 2.0 ** -19 * (np.abs(x).astype(np.float64) @ np.abs(w).astype(np.float64).T) + 1e-6
    if out_dtype == "bfloat16":
        bound = bound + 2.0 ** -8 * np.abs(want)
    assert np.all(np.abs(got - want) <= bound), float(np.max(np.abs(got - want) / bound))


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (2048, 8192, 2048), (77, 136, 80)])
def test_gemm_tcgen05_swiglu(M, I, K):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(I)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    wg = bf16_round(rng.standard_normal((I, K)).astype(np.float32) * 0.1)
    wu = bf16_round(rng.standard_normal((I, K)).astype(np.float32) * 0.1)
    gu = np.stack([wg.reshape(I // 8, 8, K), wu.reshape(I // 8, 8, K)], axis=1).reshape(2 * I, K)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_bf16(dev(x, torch.bfloat16), dev(gu, torch.bfloat16), out, swiglu=True)
    ops.check_kernel_status()
    g = x.astype(np.float64) @ wg.astype(np.float64).T
    u = x.astype(np.float64) @ wu.astype(np.float64).T
    silu = g / (1 + np.exp(-g))
    want = silu * u
    # float32 accumulation errors of the two sums (each at most 2^-19 of sum(|x||w|): K
    # additions that may each lose 2^-23 of the running magnitude), carried through
    # silu(g) * u (|silu'| <= 1.1), plus one bfloat16 rounding of the result
    eg = 2.0 ** -19 * (np.abs(x).astype(np.float64) @ np.abs(wg).astype(np.float64).T)
    eu = 2.0 ** -19 * (np.abs(x).astype(np.float64) @ np.abs(wu).astype(np.float64).T)
    bound = 1.1 * eg * (np.abs(u) + eu) + np.abs(silu) * eu + 2.0 ** -8 * np.abs(want) + 1e-6
    assert np.all(np.abs(host(out) - want) <= bound)


def _coded_operands(M, N, K, groups=16):
    """x rows that each pick one of ``groups`` ranges of K, weights that say which 128 rows and which
    eighth of K they come from (integers up to 255): every sum is exact in float32, and a tile or a
    stage taken from elsewhere shows as another value."""
    import torch
    k = torch.arange(K, device="cuda")
    m = torch.arange(M, device="cuda")
    x = ((k[None, :] * groups // K) == (m[:, None] % groups)).to(torch.bfloat16)
    n = torch.arange(N, device="cuda")
    w = (((n[:, None] // 128) % 32) + 32 * (k[None, :] * 8 // K)).to(torch.bfloat16)
    return x, w


@pytest.mark.parametrize("M,N,K", [(2048, 3072, 2048), (2048, 2048, 8192), (512, 16384, 2048), (300, 1000, 1536)])
def test_gemm_tcgen05_is_exact_launch_after_launch(M, N, K):
    """The many-row product's rings (operands by TMA, two accumulators in tensor memory) under repeated
    launches with coded operands: exact sums, every launch."""
    import torch
    from mlxforge_b200.csrc import ops
    x, w = _coded_operands(M, N, K)
    assert ops.gemm_ok(x, w)
    want = x.double() @ w.double().T
    out = torch.empty((M, N), dtype=torch.float32, device="cuda")
    for launch in range(25):
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        ops.gemm_bf16(x, w, out)
        torch.cuda.synchronize()
        assert bool((out.double() == want).all()), f"launch {launch}"
    ops.check_kernel_status()


@pytest.mark.parametrize("M,N,K", [(64, 3072, 2048), (64, 2048, 8192), (128, 16384, 2048), (17, 2048, 2048)])
def test_mid_linear_is_exact_launch_after_launch(M, N, K):
    """The same for the product of 17 to 128 rows, whose tiles are shared between blocks and reduced by
    whoever takes a tile's last ticket."""
    import torch
    from mlxforge_b200.csrc import ops
    x, w = _coded_operands(M, N, K)
    want = x.double() @ w.double().T
    out = torch.empty((M, N), dtype=torch.float32, device="cuda")
    scratch = torch.empty(ops.mid_rows_scratch(M), dtype=torch.float32, device="cuda")
    for launch in range(25):
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        ops.mid_linear(x, w, out, scratch)
        torch.cuda.synchronize()
        assert bool((out.double() == want).all()), f"launch {launch}"
    ops.check_kernel_status()


@pytest.mark.parametrize("hd,tcgen05", [(64, True), (128, True), (64, False)])
def test_prefill_attention_rings_launch_after_launch(hd, tcgen05):
    """Prefill attention of 2048 tokens with queries of zero (every visible key weighs the same) and values
    that say which tile of 64 keys they belong to: row p must return the average of the codes of keys
    0..p, launch after launch; a tile of values read from another turn of the ring moves it by 1 or more."""
    import torch
    from mlxforge_b200.csrc import ops
    T, nh, nkv, page = 2048, 8, 2, 16
    n_pages = T // page
    gen = torch.Generator(device="cuda").manual_seed(1)
    table = torch.randperm(n_pages, generator=gen, device="cuda").to(torch.int32).view(1, n_pages).contiguous()
    k_pool = torch.randn((n_pages, nkv, page, hd), generator=gen, device="cuda").to(torch.bfloat16)
    v_pool = torch.empty((n_pages, nkv, page, hd), dtype=torch.bfloat16, device="cuda")
    key = torch.arange(T, device="cuda")
    code = (((key // 64) % 7) * 32).to(torch.float32)
    for h in range(nkv):
        v_pool[table[0].long(), h] = (code + 8.0 * h).view(n_pages, page, 1).expand(-1, -1, hd).to(torch.bfloat16)
    q = torch.zeros((T, nh * hd), dtype=torch.bfloat16, device="cuda")
    heads = (torch.arange(nh, device="cuda") // (nh // nkv)).double()
    want = (torch.cumsum(code.double(), 0) / (key + 1).double())[:, None, None] + 8.0 * heads[None, :, None]
    out = torch.empty((T, nh * hd), dtype=torch.bfloat16, device="cuda")

    def i32(v):
        return torch.tensor([v], dtype=torch.int32, device="cuda")

    ops.set_prefill_tcgen05(tcgen05)
    try:
        for launch in range(25):
            out.fill_(float("nan"))
            torch.cuda.synchronize()
            ops.attention_prefill(q, k_pool, v_pool, out, i32(0), i32(T), i32(T), 0, T, table, page, nh, nkv, hd, hd ** -0.5, 0)
            torch.cuda.synchronize()
            err = float((out.double().view(T, nh, hd) - want).abs().max())
            assert err < 0.6, f"launch {launch}: an average is off by {err:.2f}"
        ops.check_kernel_status()
    finally:
        ops.set_prefill_tcgen05(True)

