"""The decode attention entry point that takes no scratch memory from its caller.

Some users of the library cannot allocate device memory: a C host without an
allocator of its own, a service that got its memory once at start-up, code that
must not call cudaMalloc because it stalls the device.  For them
``mf_attention_decode_static`` keeps the partial results of the key splits in
an array inside the library.  This test calls it through its exported C symbol
and checks that it gives what the ordinary entry point gives, twice in a row
(the array is shared between calls and keeps the first call's contents), and
that a call beyond the array's size is refused with a message.

The file name makes pytest collect it last, so a run that stops at the first
failure has already run every other test.
"""
import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

STATIC_BYTES = 8 * 1024 * 1024
MF_ERR_SCRATCH_LIMIT = 10003


def _symbols():
    from mlxforge_b200.csrc.binding import library
    lib = library()
    fn = lib.mf_attention_decode_static
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                   c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p, c_char_p, c_int]
    fn.restype = c_int
    size = lib.mf_attention_decode_static_bytes
    size.argtypes = [c_int, c_int, c_int, c_int]
    size.restype = c_longlong
    return fn, size


def _case(seed, lengths, nh, nkv, hd, page=16):
    import torch
    rng = np.random.default_rng(seed)
    n = len(lengths)
    blocks = [(m + page - 1) // page for m in lengths]
    n_pages = sum(blocks) + 3
    perm = rng.permutation(n_pages)
    table = np.full((n, max(blocks)), -1, dtype=np.int32)
    at = 0
    for s in range(n):
        for b in range(blocks[s]):
            table[s, b] = perm[at]
            at += 1
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn((n_pages, nkv, page, hd), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((n_pages, nkv, page, hd), generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn((n, nh * hd), generator=g, device="cuda").to(torch.bfloat16)
    pos = torch.tensor([m - 1 for m in lengths], dtype=torch.int32, device="cuda")
    seq = torch.arange(n, dtype=torch.int32, device="cuda")
    return q, k, v, pos, seq, torch.from_numpy(table).cuda(), max(lengths)


def _free_bytes():
    """Free device memory as the driver sees it (torch's cached blocks count as taken, so an
    allocation by torch that is served from its cache does not move this number, while a
    cudaMalloc by anyone does)."""
    import torch
    return torch.cuda.mem_get_info()[0]


@pytest.mark.parametrize("nh,nkv,hd", [(12, 3, 64), (8, 2, 128)])
def test_static_scratch_entry_point_matches_the_ordinary_one(nh, nkv, hd):
    """Head size 64 goes through the kernel with tensor copies (which merges its splits itself
    or leaves them to the merge kernel), head size 128 through the one without them and the
    merge kernel: both read and write the built-in array."""
    import torch
    from mlxforge_b200.csrc import ops
    fn, size = _symbols()
    page = 16
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    # the second call is smaller than the first: it runs over what the first left in the array
    for seed, lengths in ((1, [700, 33, 256, 1]), (2, [45, 300])):
        q, k, v, pos, seq, table, max_ctx = _case(seed, lengths, nh, nkv, hd, page)
        n = len(lengths)
        scale = hd ** -0.5
        n_o, n_ml = ops.attention_decode_scratch(n, nh, hd, max_ctx)
        want = torch.empty((n, nh * hd), dtype=torch.bfloat16, device="cuda")
        ops.attention_decode(q, k, v, want, torch.empty(n_o, dtype=torch.float32, device="cuda"),
                             torch.empty(n_ml, dtype=torch.float32, device="cuda"), pos, seq, table, page, nh, nkv,
                             hd, scale, 0, max_ctx)
        got = torch.full_like(want, float("nan"))
        assert 0 < size(n, nh, hd, max_ctx) <= STATIC_BYTES
        err = ctypes.create_string_buffer(256)
        torch.cuda.synchronize()
        free_before = _free_bytes()
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), got.data_ptr(), n, nh, nkv, hd, pos.data_ptr(),
                seq.data_ptr(), table.data_ptr(), table.shape[1], page, scale, 0, max_ctx, stream, err, 256)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        # its one claim: the call took no device memory (the ordinary call above has already paid
        # for whatever a kernel's first launch on this device costs)
        assert _free_bytes() == free_before, "the entry point that allocates nothing changed the free device memory"
        # the same kernels on the same inputs; the tolerance is that of the other attention tests
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 1.5e-2, diff
        assert torch.isfinite(got.float()).all()


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    import torch
    fn, size = _symbols()
    nh, nkv, hd = 32, 8, 64
    q, k, v, pos, seq, table, _ = _case(3, [40, 50], nh, nkv, hd)
    too_long = 64                          # grow the claimed context until the partials no longer fit
    while size(2, nh, hd, too_long) <= STATIC_BYTES:
        too_long *= 2
    assert size(2, nh, hd, too_long // 2) <= STATIC_BYTES < size(2, nh, hd, too_long)
    out = torch.zeros((2, nh * hd), dtype=torch.bfloat16, device="cuda")
    err = ctypes.create_string_buffer(256)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 2, nh, nkv, hd, pos.data_ptr(),
            seq.data_ptr(), table.data_ptr(), table.shape[1], 16, 0.125, 0, too_long,
            c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    assert rc == MF_ERR_SCRATCH_LIMIT
    msg = err.value.decode()
    assert "bytes of scratch" in msg and str(STATIC_BYTES) in msg
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0, "a refused call launches nothing"
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 2, nh, nkv, 40, pos.data_ptr(),
            seq.data_ptr(), table.data_ptr(), table.shape[1], 16, 0.125, 0, 64,
            c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    assert rc != 0 and "unsupported sizes" in err.value.decode()
