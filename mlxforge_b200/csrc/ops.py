"""Python-side launchers of the CUDA kernels, taking torch tensors.

These are thin: they check what the kernel cannot check for itself, pass raw
pointers and the current stream, and raise ``KernelError`` on a refusal.
"""
from __future__ import annotations

from ctypes import c_void_p
from typing import Optional

import torch

from .binding import KernelError, check, count_launches, library

F32, BF16 = 0, 1


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"tensor dtype {t.dtype} is neither float32 nor bfloat16")


# The current stream's handle without building a torch.cuda.Stream object for it (that costs
# about 15 us a call, and every kernel launch asks): torch's own binding for it, where present.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernel operands must be contiguous CUDA tensors "
                              f"(got device={t.device}, contiguous={t.is_contiguous()})")


def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(table, tokens, out)
    T, H = out.shape
    check(library().mf_embed(table.data_ptr(), dtype_code(table), tokens.data_ptr(), out.data_ptr(), T, H,
                             _stream()), "embed")


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    _need_cuda(resid, delta, weight, out, rows)
    H = resid.shape[-1]
    n = out.shape[0]
    check(library().mf_add_rmsnorm(resid.data_ptr(), _ptr(delta), dtype_code(delta) if delta is not None else F32,
                                   weight.data_ptr(), eps, out.data_ptr(), dtype_code(out), _ptr(rows), n, H,
                                   _stream()), "add_rmsnorm")


def residual_add(resid: torch.Tensor, delta: torch.Tensor) -> None:
    _need_cuda(resid, delta)
    check(library().mf_residual_add(resid.data_ptr(), delta.data_ptr(), dtype_code(delta), resid.numel(),
                                    _stream()), "residual_add")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                  block_table: torch.Tensor, page_size: int, freqs: Optional[torch.Tensor], q_out: torch.Tensor,
                  k_pool: torch.Tensor, v_pool: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                  rotary_dim: int, write_kv: bool, precise: bool) -> None:
    _need_cuda(qkv, positions, seq_of_token, block_table, freqs, q_out, k_pool, v_pool)
    T = qkv.shape[0]
    check(library().mf_rope_kv_write(qkv.data_ptr(), dtype_code(qkv), T, n_heads, n_kv, head_dim, rotary_dim,
                                     positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                                     block_table.shape[1], page_size, _ptr(freqs), q_out.data_ptr(),
                                     k_pool.data_ptr(), v_pool.data_ptr(), int(write_kv), int(precise),
                                     _stream()), "rope_kv_write")


def swiglu(gu: torch.Tensor, out: torch.Tensor, group: int) -> None:
    _need_cuda(gu, out)
    T, I = out.shape
    check(library().mf_swiglu(gu.data_ptr(), out.data_ptr(), dtype_code(gu), T, I, group, _stream()), "swiglu")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    check(library().mf_gemm_f32(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, int(accumulate),
                                _stream()), "gemm_f32")


def attention_generic(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                      positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                      page_size: int, n_heads: int, n_kv: int, head_dim: int, scale: float, window: int) -> None:
    _need_cuda(q, k_pool, v_pool, out, positions, seq_of_token, block_table)
    T = q.shape[0]
    check(library().mf_attention_generic(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                         dtype_code(q), T, n_heads, n_kv, head_dim, positions.data_ptr(),
                                         seq_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                         page_size, scale, window, _stream()), "attention_generic")


def attention_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                      seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, seq_ctx_len: torch.Tensor,
                      table_row0: int, max_q_len: int, block_table: torch.Tensor, page_size: int, n_heads: int,
                      n_kv: int, head_dim: int, scale: float, window: int) -> None:
    """Attention of prompt portions, bfloat16.  ``q`` / ``out`` are the whole step's
    [T, n_heads*head_dim]; the three per-sequence arrays describe the sequences
    that start at row ``table_row0`` of ``block_table``."""
    _need_cuda(q, k_pool, v_pool, out, seq_q_start, seq_q_len, seq_ctx_len, block_table)
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: bfloat16 only")
    check(library().mf_attention_prefill(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                         seq_q_start.data_ptr(), seq_q_len.data_ptr(), seq_ctx_len.data_ptr(),
                                         table_row0, seq_q_len.shape[0], max_q_len, q.shape[0], n_heads, n_kv,
                                         head_dim, block_table.data_ptr(), block_table.shape[1], page_size, scale,
                                         window, kernel_status(q.device).data_ptr(), _stream()), "attention_prefill")


def set_prefill_tcgen05(on: bool) -> None:
    """Whether portions of at least 128 tokens with head size 64 take the tcgen05 attention
    kernel (the default) or every shape the mma.sync one."""
    check(library().mf_set_prefill_tcgen05(1 if on else 0), "set_prefill_tcgen05", launches=0)


def few_rows_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the few-row product kernels take these operands (rows are read in 16-byte pieces)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_STATUS = {}
_TMA_STATUS_SET = False


def kernel_status(device=None) -> torch.Tensor:
    """The device word in which kernels with bounded waits record that a wait ran out."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _STATUS[key] = t
    return t


def kernel_gave_up(code: int, device=None) -> KernelError:
    """What to do when the status word read ``code`` != 0: a kernel with bounded waits gave up,
    so what it wrote is not to be trusted.  Clears the word and everything such a kernel may
    have left half done (the decode-attention tickets), and returns the error to raise."""
    kernel_status(device).zero_()
    check(library().mf_reset_decode_tickets(_stream()), "reset_decode_tickets", launches=0)
    check(library().mf_reset_mid_rows_tickets(_stream()), "reset_mid_rows_tickets", launches=0)
    return KernelError(f"a kernel's bounded wait ran out (code {code}: 1 = copy producer, 2 = consumer); "
                       "the results of the step are invalid")


def check_kernel_status() -> None:
    """Raise if a kernel gave up a bounded wait since the last check (reads the word back, which
    waits for the device: call it where the host waits anyway)."""
    for key, t in _STATUS.items():
        code = int(t.item())
        if code:
            raise kernel_gave_up(code, torch.device("cuda", key))


def stream_max_rows() -> int:
    return int(library().mf_stream_max_rows())


def set_stream_tensor_copies(on: bool) -> None:
    """Whether ``stream_linear`` brings a stage with one tensor copy (widths that are a multiple
    of 64; the default) or always with one copy per row segment."""
    check(library().mf_set_stream_tensor_copies(1 if on else 0), "set_stream_tensor_copies", launches=0)


def stream_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> None:
    """out = x @ w^T for at most ``stream_max_rows()`` rows of bfloat16 x (out bfloat16 or
    float32), the weights streamed by bulk copies (see gemv_stream.cu); with ``swiglu`` the rows
    of w interleave gate and up in groups of 8 and out [M, N/2] is silu(gate) * up.
    The kernel starts fetching ``w`` before it waits for the kernel launched before it, so
    ``w`` must not be the output of that kernel (the engine's weights are written once, at
    load time)."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    want = (M, N // 2) if swiglu else (M, N)
    if w.shape[1] != K or tuple(out.shape) != want:
        raise KernelError(f"stream_linear: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    check(library().mf_stream_linear(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out), M, N, K,
                                     1 if swiglu else 0, kernel_status(x.device).data_ptr(), _stream()),
          "stream_linear")


def mid_rows_range():
    """(fewest, most) rows of x that ``mid_linear`` takes."""
    return int(library().mf_mid_rows_min()), int(library().mf_mid_rows_max())


def mid_rows_scratch(rows: int) -> int:
    """float32 elements of scratch that ``mid_linear`` needs for ``rows`` rows of x."""
    return int(library().mf_mid_rows_scratch(rows))


def mid_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, swiglu: bool = False) -> None:
    """out = x @ w^T for 17 to 128 rows of bfloat16 x on the tcgen05 tensor cores with the weights
    streamed once (see gemm_mid_rows.cu); out bfloat16 or float32; with ``swiglu`` the rows of w
    interleave gate and up in groups of 8 and out is [M, N/2] = silu(gate) * up.  ``scratch``:
    float32, at least ``mid_rows_scratch(M)`` elements.  As with ``stream_linear``, ``w`` must not
    be the output of the kernel launched just before."""
    _need_cuda(x, w, out, scratch)
    M, K = x.shape
    N = w.shape[0]
    want = (M, N // 2) if swiglu else (M, N)
    if w.shape[1] != K or tuple(out.shape) != want:
        raise KernelError(f"mid_linear: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if scratch.dtype != torch.float32 or scratch.numel() < mid_rows_scratch(M):
        raise KernelError("mid_linear: scratch too small")
    check(library().mf_mid_rows_linear(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out), scratch.data_ptr(),
                                       M, N, K, 1 if swiglu else 0, kernel_status(x.device).data_ptr(), _stream()),
          "mid_linear")


def gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands (TMA needs 16-byte row strides)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> None:
    """out = x @ w^T on the tcgen05 tensor cores (bfloat16 operands; out bfloat16 or float32);
    with ``swiglu`` the rows of w interleave gate and up in groups of 8 and out is
    [M, N/2] = silu(gate) * up."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    want = (M, N // 2) if swiglu else (M, N)
    if w.shape[1] != K or tuple(out.shape) != want:
        raise KernelError(f"gemm_bf16: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if swiglu and out.dtype != torch.bfloat16:
        raise KernelError("gemm_bf16: the gated epilogue writes bfloat16")
    epi = 2 if swiglu else (1 if out.dtype == torch.float32 else 0)
    check(library().mf_gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, epi,
                                 kernel_status(x.device).data_ptr(), _stream()), "gemm_bf16")


def set_decode_tma(on: bool) -> bool:
    """Switch the TMA decode-attention kernel (head size 64) on or off; returns the previous
    setting.  Both kernels write the same partial results."""
    return bool(library().mf_set_decode_tma(1 if on else 0, kernel_status().data_ptr()))


def set_decode_merge_inside(on: bool) -> bool:
    """Whether the TMA decode-attention kernel merges its splits itself (the block that finishes a
    group's last split does it) or a merge kernel follows it; returns the previous setting."""
    return bool(library().mf_set_decode_merge_inside(1 if on else 0))


def attention_decode_split(head_dim: int) -> int:
    """Keys per split of the decode kernel for a head size."""
    return int(library().mf_attention_decode_split(head_dim))


def attention_decode_scratch(n_tokens: int, n_heads: int, head_dim: int, max_ctx: int):
    """Element counts of the two float32 scratch buffers the decode kernel needs."""
    splits = (max_ctx + attention_decode_split(head_dim) - 1) // attention_decode_split(head_dim)
    return n_tokens * n_heads * splits * head_dim, n_tokens * n_heads * splits * 2


def attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                     part_o: torch.Tensor, part_ml: torch.Tensor, positions: torch.Tensor,
                     seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int, n_heads: int,
                     n_kv: int, head_dim: int, scale: float, window: int, max_ctx: int,
                     unequal_contexts: bool = False) -> None:
    """Attention of tokens that are each the newest of their sequence (one query per
    sequence), bfloat16, split over the keys; ``part_o`` / ``part_ml`` are float32
    scratch of at least ``attention_decode_scratch`` elements.  ``unequal_contexts``: the
    caller knows that the contexts differ widely in length (see mf_attention_decode_hinted)."""
    _need_cuda(q, k_pool, v_pool, out, part_o, part_ml, positions, seq_of_token, block_table)
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 only")
    n = q.shape[0]
    global _TMA_STATUS_SET
    if not _TMA_STATUS_SET:
        library().mf_set_decode_status(kernel_status(q.device).data_ptr())
        _TMA_STATUS_SET = True
    need_o, need_ml = attention_decode_scratch(n, n_heads, head_dim, max_ctx)
    if part_o.numel() < need_o or part_ml.numel() < need_ml or part_o.dtype != torch.float32:
        raise KernelError("attention_decode: scratch too small")
    check(library().mf_attention_decode_hinted(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                               part_o.data_ptr(), part_ml.data_ptr(), n, n_heads, n_kv, head_dim,
                                               positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                                               block_table.shape[1], page_size, scale, window, max_ctx,
                                               1 if unequal_contexts else 0, _stream()),
          "attention_decode", launches=0)
    # one kernel when the TMA kernel merged its splits itself, two when a merge kernel followed
    count_launches(int(library().mf_attention_decode_launches()))


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], u: Optional[torch.Tensor],
           out: torch.Tensor) -> None:
    """Row r: argmax if temperature is None or temperature[r] <= 0, else an
    inverse-CDF draw from softmax(logits[r] / temperature[r]) with u[r]."""
    _need_cuda(temperature, u, out)
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 CUDA rows")
    n, V = logits.shape
    split = temperature is None and V >= 16384 and n <= 4096       # greedy over a large vocabulary: two kernels
    check(library().mf_sample(logits.data_ptr(), n, V, logits.stride(0), _ptr(temperature), _ptr(u),
                              out.data_ptr(), _stream()), "sample", launches=2 if split else 1)


def apply_penalties(logits: torch.Tensor, params, histories) -> None:
    """Repetition / frequency / presence penalties, in place, over each row's
    history.  The unique ids and their counts are made on the host (the history
    lives there) and sent in one copy."""
    import numpy as np
    n = logits.shape[0]
    ids, counts, off = [], [], [0]
    for r in range(n):
        h = np.asarray(histories[r] if params[r].has_penalties else (), dtype=np.int64)
        added = 0
        if h.size:
            u, c = np.unique(h, return_counts=True)
            ids.append(u.astype(np.int32))
            counts.append(c.astype(np.int32))
            added = u.size
        off.append(off[-1] + added)
    if off[-1] == 0:
        return
    ints = np.concatenate(ids + counts + [np.asarray(off, dtype=np.int32)])
    floats = np.asarray([[p.repetition_penalty for p in params], [p.frequency_penalty for p in params],
                         [p.presence_penalty for p in params]], dtype=np.float32)
    di = torch.from_numpy(ints).to(logits.device)
    df = torch.from_numpy(floats).to(logits.device)
    m = off[-1]
    check(library().mf_apply_penalties(logits.data_ptr(), n, logits.stride(0), di[:m].data_ptr(),
                                       di[m:2 * m].data_ptr(), di[2 * m:].data_ptr(), df[0].data_ptr(),
                                       df[1].data_ptr(), df[2].data_ptr(), _stream()), "apply_penalties")


def filter_logits(logits: torch.Tensor, params) -> None:
    """top-k, top-p and min-p of every non-greedy row, in place (removed entries -inf)."""
    import numpy as np
    n, V = logits.shape
    floats = np.asarray([[0.0 if p.greedy else p.temperature for p in params], [p.top_p for p in params],
                         [p.min_p for p in params]], dtype=np.float32)
    ks = np.asarray([p.top_k for p in params], dtype=np.int32)
    df = torch.from_numpy(floats).to(logits.device)
    dk = torch.from_numpy(ks).to(logits.device)
    check(library().mf_filter_logits(logits.data_ptr(), n, V, logits.stride(0), df[0].data_ptr(), dk.data_ptr(),
                                     df[1].data_ptr(), df[2].data_ptr(), _stream()), "filter_logits")


def set_dependent_launch(on: bool) -> bool:
    """Switch programmatic dependent launch of the decode-path kernels on or off;
    returns the previous setting.  Results do not depend on it."""
    return bool(library().mf_set_pdl(1 if on else 0))
