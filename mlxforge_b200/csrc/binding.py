"""ctypes binding of the engine's CUDA library.

Every entry point takes raw device pointers and the CUDA stream to launch on
and allocates nothing; the wrappers here pass ``tensor.data_ptr()`` and the
current torch stream.  There is no other implementation behind these names:
if the library cannot be built or loaded, ``kernels()`` raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

from . import build as _build

_P = c_void_p
_LIB: Optional[ctypes.CDLL] = None

_SIGNATURES = {
    "mf_embed": [_P, c_int, _P, _P, c_int, c_int, _P],
    "mf_add_rmsnorm": [_P, _P, c_int, _P, c_float, _P, c_int, _P, c_int, c_int, _P],
    "mf_rope_kv_write": [_P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, c_int, c_int, _P, _P, _P,
                         _P, c_int, c_int, _P],
    "mf_swiglu": [_P, _P, c_int, c_int, c_int, c_int, _P],
    "mf_residual_add": [_P, _P, c_int, c_longlong, _P],
    "mf_gemm_f32": [_P, _P, _P, c_int, c_int, c_int, c_int, _P],
    "mf_attention_generic": [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, c_int, c_int,
                             c_float, c_int, _P],
    "mf_sample": [_P, c_int, c_int, c_longlong, _P, _P, _P, _P],
    "mf_set_pdl": [c_int],
    "mf_set_decode_tma": [c_int, _P],
    "mf_set_decode_status": [_P],
    "mf_set_decode_merge_inside": [c_int],
    "mf_attention_decode_launches": [],
    "mf_gemm_bf16": [_P, _P, _P, c_int, c_int, c_int, c_int, _P, _P],
    "mf_stream_max_rows": [],
    "mf_set_stream_tensor_copies": [c_int],
    "mf_stream_linear": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "mf_attention_prefill": [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int,
                             c_int, c_float, c_int, _P, _P],
    "mf_set_prefill_tcgen05": [c_int],
    "mf_attention_decode_split": [c_int],
    "mf_attention_decode": [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, _P, _P, c_int, c_int,
                            c_float, c_int, c_int, _P],
    "mf_attention_decode_hinted": [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, _P, _P, c_int, c_int,
                                   c_float, c_int, c_int, c_int, _P],
    "mf_apply_penalties": [_P, c_int, c_longlong, _P, _P, _P, _P, _P, _P, _P],
    "mf_filter_logits": [_P, c_int, c_int, c_longlong, _P, _P, _P, _P, _P],
    "mf_kernel_kinds": [],
    "mf_reset_decode_tickets": [_P],
    "mf_reset_mid_rows_tickets": [_P],
    "mf_mid_rows_min": [],
    "mf_set_mid_rows_chunks": [c_int],
    "mf_mid_rows_max": [],
    "mf_mid_rows_linear": [_P, _P, _P, c_int, _P, c_int, c_int, c_int, c_int, _P, _P],
}

MF_ERRORS = {10001: "a size or option this kernel does not take", 10002: "an unsupported dtype"}


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The loaded CUDA library; built on first use.  Raises if it cannot be had."""
    global _LIB
    if _LIB is None:
        path = _build.library_path()
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"mlxforge_b200: cannot load its CUDA library {path}: {e}") from e
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
        lib.mf_kernel_name.argtypes = [c_int]
        lib.mf_kernel_name.restype = ctypes.c_char_p
        lib.mf_kernel_launches.argtypes = [c_int]
        lib.mf_kernel_launches.restype = c_longlong
        lib.mf_mid_rows_scratch.argtypes = [c_int]
        lib.mf_mid_rows_scratch.restype = c_longlong
        _LIB = lib
    return _LIB


def declare(name: str, argtypes) -> None:
    """Add the signature of a further entry point (used by kernel modules that
    come with their own .cu file)."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None:
        fn = getattr(_LIB, name)
        fn.argtypes = argtypes
        fn.restype = c_int


_LAUNCHES = 0


def launch_count() -> int:
    """Kernel launches of this library so far in this process (every entry point
    reports how many kernels it launched; graph replays add their kernel nodes)."""
    return _LAUNCHES


def count_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def kernel_launches() -> dict:
    """How often each kind of kernel has been launched by this process, by name (a launch
    recorded into a CUDA graph counts once, its replays do not).  Tests of whole models use
    the difference of two readings to say which kernels a model's steps went through."""
    lib = library()
    return {lib.mf_kernel_name(i).decode(): int(lib.mf_kernel_launches(i)) for i in range(lib.mf_kernel_kinds())}


def check(code: int, what: str, launches: int = 1) -> None:
    if code == 0:
        global _LAUNCHES
        _LAUNCHES += launches
        return
    if code in MF_ERRORS:
        raise KernelError(f"{what}: refused: {MF_ERRORS[code]}")
    raise KernelError(f"{what}: CUDA error {code} ({_cuda_error_name(code)})")


def _cuda_error_name(code: int) -> str:
    try:
        import torch
        rt = torch.cuda.cudart()
        return str(rt.cudaGetErrorString(rt.cudaError(code)))
    except Exception:
        return "see cudaError_t"
