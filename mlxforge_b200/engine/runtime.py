"""What every part needs from the engine at run time: the compute dtype, the
device, scratch buffers that are allocated once and reused by every step, and
the matrix product (the one operation whose kernel depends on the dtype and on
how many rows there are).
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from ..csrc import ops


class Runtime:
    """``dtype`` float32 is the true 32-bit path (IEEE products on the CUDA cores,
    angles in double); bfloat16 is the serving path (bfloat16 operands, 32-bit
    accumulation, 32-bit residual stream, norms, softmax and logits)."""

    def __init__(self, dtype: torch.dtype, device: str = "cuda"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.device = torch.device(device)
        self.precise = dtype == torch.float32
        # the library's bfloat16 products must add their partial sums in 32-bit too (a split along K
        # that reduces in bfloat16 would round more than once and depend on the number of rows)
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self._buffers: Dict[str, torch.Tensor] = {}
        self._views: Dict[tuple, tuple] = {}
        # bumped whenever a scratch buffer moves: captured CUDA graphs hold the old addresses
        self.generation = 0
        # rows every per-token buffer is first made for, so that later, larger steps do not move it
        self.reserve_rows = 0
        # rows at or below which the bfloat16 product runs the few-row kernel that streams its weights
        # by bulk copies (``skinny_mm`` off sends them to the library, as the reference's option does)
        self.skinny_enabled = True
        self.stream_max_rows = ops.stream_max_rows() if self.device.type == "cuda" else 16
        # 17 to 128 rows (a decode step of that many requests): the library's product by default, as
        # in the reference above its own kernels' 32 rows; MLXFORGE_MID_ROWS=1 (or the "tcgen05"
        # backend) takes this engine's own kernel with the weights on the M side of the tensor-core
        # instruction instead (gemm_mid_rows.cu: correct at every size, and measured slower than
        # the library on the 1B shape's matrices, so it is not the default)
        self.mid_rows_enabled = os.environ.get("MLXFORGE_MID_ROWS", "0") == "1"
        self.mid_max_rows = 128
        # many-row bfloat16 products: "library" (cuBLAS through torch.mm, as the reference uses
        # its library's matmul there), "tcgen05" (this engine's own tensor-memory kernel), or
        # "auto": the own kernel where it has SwiGLU in its epilogue (gate|up: one kernel instead
        # of the library's product and an elementwise pass over its result), the library elsewhere
        self.gemm_backend = os.environ.get("MLXFORGE_GEMM", "auto")
        if self.gemm_backend not in ("auto", "library", "tcgen05"):
            raise ValueError(f"MLXFORGE_GEMM must be 'auto', 'library' or 'tcgen05', got '{self.gemm_backend}'")
        # rows from which "auto" takes the own kernel for gate|up (below, the library's product
        # of few rows and the elementwise pass are the shorter way)
        self.fused_swiglu_min_rows = 256

    # ------------------------------------------------------------------ scratch
    def buffer(self, name: str, shape: Tuple[int, ...], dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """A contiguous scratch tensor of ``shape``; the storage behind ``name``
        only ever grows, so steady-state steps allocate nothing."""
        dtype = dtype or self.dtype
        # the same view is asked for step after step: keep it, as long as no buffer has moved
        vkey = (name, shape, dtype)
        hit = self._views.get(vkey)
        if hit is not None and hit[0] == self.generation:
            return hit[1]
        n = 1
        for s in shape:
            n *= int(s)
        key = f"{name}:{dtype}"
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            cap = n
            if len(shape) >= 2 and self.reserve_rows > shape[0]:
                cap = n // int(shape[0]) * self.reserve_rows
            buf = torch.empty(max(cap, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        view = buf[:n].view(shape)
        if len(self._views) > 8192:
            self._views.clear()
        self._views[vkey] = (self.generation, view)
        return view

    # ------------------------------------------------------------------ products
    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``out = x @ w^T`` with ``w`` [out_features, in_features].  float32
        operands use this engine's IEEE kernel; bfloat16 operands use the streamed
        few-row kernel up to 16 rows and the library product (or this engine's own
        tcgen05 kernels, see ``gemm_backend``) above, accumulating in 32-bit and
        rounding once to ``out``'s dtype."""
        if x.dtype == torch.float32 and w.dtype == torch.float32:
            ops.gemm_f32(x, w, out)
            return out
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise ops.KernelError(f"linear: operand dtypes {x.dtype} x {w.dtype} are not a supported pair")
        if self._skinny(x, w):
            ops.stream_linear(x, w, out)
            return out
        if self._mid(x, w):
            ops.mid_linear(x, w, out, self.buffer("mid.partials", (ops.mid_rows_scratch(x.shape[0]),), torch.float32))
            return out
        if self.gemm_backend == "tcgen05" and ops.gemm_ok(x, w):
            ops.gemm_bf16(x, w, out)
            return out
        if out.dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        return out

    def _skinny(self, x, w) -> bool:
        return self.skinny_enabled and x.shape[0] <= self.stream_max_rows and ops.few_rows_ok(x, w)

    def _mid(self, x, w) -> bool:
        return ((self.mid_rows_enabled or self.gemm_backend == "tcgen05") and self.gemm_backend != "library"
                and x.shape[0] <= self.mid_max_rows and ops.gemm_ok(x, w))

    def linear_swiglu(self, x: torch.Tensor, w_gu: torch.Tensor, group: int, out: torch.Tensor) -> torch.Tensor:
        """``out = silu(x Wg^T) * (x Wu^T)`` for a matrix whose rows interleave gate and
        up in groups of ``group``.  Few bfloat16 rows: one kernel with the product in
        its epilogue; otherwise the product, then the elementwise kernel."""
        if group == 8 and w_gu.shape[0] % 16 == 0 and self._skinny(x, w_gu):
            ops.stream_linear(x, w_gu, out, swiglu=True)
            return out
        if group == 8 and w_gu.shape[0] % 16 == 0 and self._mid(x, w_gu):
            ops.mid_linear(x, w_gu, out, self.buffer("mid.partials", (ops.mid_rows_scratch(x.shape[0]),), torch.float32),
                           swiglu=True)
            return out
        own = self.gemm_backend == "tcgen05" or (self.gemm_backend == "auto"
                                                 and x.shape[0] >= self.fused_swiglu_min_rows)
        if own and group == 8 and w_gu.shape[0] % 16 == 0 and ops.gemm_ok(x, w_gu):
            ops.gemm_bf16(x, w_gu, out, swiglu=True)
            return out
        gu = self.linear(x, w_gu, self.buffer("ffn.gu", (x.shape[0], w_gu.shape[0])))
        ops.swiglu(gu, out, group)
        return out
