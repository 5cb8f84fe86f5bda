// out[M, N] = x[M, K] * W[N, K]^T for a few rows of x (decoding): bfloat16 operands,
// float32 accumulation, weights streamed from HBM exactly once.
//
// The reference writes this case by hand too ("skinny" products for 2..32 rows,
// src/model/skinny_matmul.cpp:17-140: one simdgroup per output column, or 8x8
// simdgroup MMA tiles for the vocabulary head).  Here the weight rows are the
// M side of mma.sync.m16n8k16 ("swap A and B": out^T = W x^T), so 16 (or 8)
// weight rows meet up to 8*NB rows of x per instruction, and a block's 8 warps
// split K between them.  A thread loads 16 contiguous bytes of a weight row and
// the 16 bytes of x at the same k: the permutation of k inside the instruction is
// the same on both sides, so no shuffle and no shared-memory staging is needed.
//
// The order of every sum is fixed by (K, the block shape), never by M or by what
// else is in the batch.  Epilogues: plain store (bfloat16 or float32) or the
// SiLU-gated product of the feed-forward for weights whose rows interleave gate and
// up in groups of 8 (src/model/decoder_model.cpp:277-282).
#include "common.cuh"

namespace {

constexpr int WARPS = 8;

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NB: blocks of 8 rows of x (M <= 8 * NB).  ROWS: weight rows per block, 16 or 8.
// mode 0: out[m, n] = acc (OutT).  mode 1 (ROWS == 16): out[m, n/2] = silu(gate) * up.
template <int NB, int ROWS, typename OutT>
__global__ void __launch_bounds__(WARPS * 32)
skinny_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W, OutT* __restrict__ out,
              int M, int N, int K, int mode) {
  constexpr int UNROLL = NB >= 4 ? 2 : 4;
  __shared__ float red[WARPS][ROWS][NB * 8 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * ROWS;
  const int row_a = n0 + g, row_b = n0 + g + 8;
  const bool va = row_a < N, vb = (ROWS == 16) && row_b < N;
  const __nv_bfloat16* wa = W + (long long)(va ? row_a : 0) * K;
  const __nv_bfloat16* wb = W + (long long)(vb ? row_b : 0) * K;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; nb++) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;

  // Two stages of UNROLL loads each are kept in flight: while one stage is multiplied the
  // next is on its way.  The loop bound is the same for every lane of a warp (mma.sync
  // needs all 32 of them); a piece beyond K is not read and counts as zero.
  constexpr int STEP = WARPS * 32 * UNROLL;
  uint4 a0[UNROLL], b0[UNROLL], x0[UNROLL][NB], a1[UNROLL], b1[UNROLL], x1[UNROLL][NB];
  auto load_w = [&](uint4 (&a)[UNROLL], uint4 (&b)[UNROLL], int kb) {
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
      const int k = kb + u * WARPS * 32 + t * 8;
      const bool in = k < K;
      a[u] = (in && va) ? ldg_stream(wa + k) : zero;
      b[u] = (in && vb) ? ldg_stream(wb + k) : zero;
    }
  };
  auto load_x = [&](uint4 (&xv)[UNROLL][NB], int kb) {
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
      const int k = kb + u * WARPS * 32 + t * 8;
#pragma unroll
      for (int nb = 0; nb < NB; nb++) {
        const int m = nb * 8 + g;
        xv[u][nb] = (k < K && m < M) ? __ldg(reinterpret_cast<const uint4*>(x + (long long)m * K + k)) : zero;
      }
    }
  };
  auto multiply = [&](const uint4 (&a)[UNROLL], const uint4 (&b)[UNROLL], const uint4 (&xv)[UNROLL][NB]) {
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
#pragma unroll
      for (int nb = 0; nb < NB; nb++) {
        mma_bf16(acc[nb], a[u].x, b[u].x, a[u].y, b[u].y, xv[u][nb].x, xv[u][nb].y);
        mma_bf16(acc[nb], a[u].z, b[u].z, a[u].w, b[u].w, xv[u][nb].z, xv[u][nb].w);
      }
    }
  };
  // weights never change: the first two stages of them are fetched while the kernel that
  // produces x may still be running; x is read only after it has finished
  load_w(a0, b0, warp * 32);
  load_w(a1, b1, warp * 32 + STEP);
  pdl_wait();
  pdl_launch();      // only now: a kernel that let its dependents go before waiting would let the
                     // whole chain of kernels pile up on the SMs, all waiting
  load_x(x0, warp * 32);
  for (int kb = warp * 32; kb < K; kb += 2 * STEP) {
    load_x(x1, kb + STEP);
    multiply(a0, b0, x0);
    load_w(a0, b0, kb + 2 * STEP);
    load_x(x0, kb + 2 * STEP);
    multiply(a1, b1, x1);
    load_w(a1, b1, kb + 3 * STEP);
  }
  // ---- sum the 8 warps' partial results in a fixed order
#pragma unroll
  for (int nb = 0; nb < NB; nb++) {
    red[warp][g][nb * 8 + 2 * t] = acc[nb][0];
    red[warp][g][nb * 8 + 2 * t + 1] = acc[nb][1];
    if (ROWS == 16) {
      red[warp][g + 8][nb * 8 + 2 * t] = acc[nb][2];
      red[warp][g + 8][nb * 8 + 2 * t + 1] = acc[nb][3];
    }
  }
  __syncthreads();
  if (mode == 0) {
    for (int i = threadIdx.x; i < ROWS * NB * 8; i += WARPS * 32) {
      const int m = i / ROWS, r = i - m * ROWS;      // r fastest: neighbouring threads write neighbouring columns
      if (m >= M || n0 + r >= N) continue;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; w++) s += red[w][r][m];
      out[(long long)m * N + n0 + r] = from_f32<OutT>(s);
    }
  } else {
    // rows 0..7 of the tile are gate rows, 8..15 the matching up rows
    const int half = ROWS / 2;
    for (int i = threadIdx.x; i < half * NB * 8; i += WARPS * 32) {
      const int m = i / half, r = i - m * half;
      if (m >= M || n0 + r + half >= N) continue;
      float gs = 0.f, us = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; w++) {
        gs += red[w][r][m];
        us += red[w][r + half][m];
      }
      out[(long long)m * (N / 2) + blockIdx.x * half + r] = from_f32<OutT>(gs / (1.0f + expf(-gs)) * us);
    }
  }
}

template <int NB, typename OutT>
int launch(const __nv_bfloat16* x, const __nv_bfloat16* W, OutT* out, int M, int N, int K, int mode,
           cudaStream_t stream) {
  // few output rows: halve the tile so that there are enough blocks for every SM
  const bool small = mode == 0 && (N + 15) / 16 < 296;
  mf_count(MF_K_SKINNY);
  if (small)
    return (int)launch_dep(skinny_kernel<NB, 8, OutT>, dim3((N + 7) / 8), dim3(WARPS * 32), 0, stream, x, W, out, M, N,
                           K, mode);
  return (int)launch_dep(skinny_kernel<NB, 16, OutT>, dim3((N + 15) / 16), dim3(WARPS * 32), 0, stream, x, W, out, M,
                         N, K, mode);
}

template <typename OutT>
int dispatch(const __nv_bfloat16* x, const __nv_bfloat16* W, OutT* out, int M, int N, int K, int mode,
             cudaStream_t stream) {
  if (M <= 8) return launch<1, OutT>(x, W, out, M, N, K, mode, stream);
  if (M <= 16) return launch<2, OutT>(x, W, out, M, N, K, mode, stream);
  if (M <= 32) return launch<4, OutT>(x, W, out, M, N, K, mode, stream);
  return MF_ERR_BAD_ARG;
}

}  // namespace

// Most rows of x this kernel takes.
MF_API int mf_skinny_max_rows() { return 32; }

// mode 0: out [M, N] in out_dtype.  mode 1: W rows interleave gate and up in groups of 8
// (N even, a multiple of 16) and out is [M, N / 2] = silu(gate) * up.
// K must be a multiple of 8 and x, W 16-byte aligned (rows are read in 16-byte pieces).
MF_API int mf_skinny_linear(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K, int mode,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || M > 32 || (mode != 0 && mode != 1)) return MF_ERR_BAD_ARG;
  if (mode == 1 && N % 16) return MF_ERR_BAD_ARG;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return MF_ERR_BAD_ARG;
  const __nv_bfloat16 *xx = (const __nv_bfloat16*)x, *ww = (const __nv_bfloat16*)W;
  if (out_dtype == MF_BF16) return dispatch<__nv_bfloat16>(xx, ww, (__nv_bfloat16*)out, M, N, K, mode, stream);
  if (out_dtype == MF_F32) return dispatch<float>(xx, ww, (float*)out, M, N, K, mode, stream);
  return MF_ERR_BAD_DTYPE;
}
