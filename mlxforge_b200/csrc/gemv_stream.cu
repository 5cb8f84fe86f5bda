// out[M, N] = x[M, K] * W[N, K]^T for a few rows of x, with the weights streamed through
// shared memory by the bulk-copy engine (TMA): the decode-time product of every
// projection and of the vocabulary head.
//
// Weight rows are the M side of mma.sync.m16n8k16, up to 8*NB rows of x the N side, bfloat16
// in, float32 accumulation; the epilogue stores the product or, for a W whose rows interleave
// gate and up in groups of 8, silu(gate) * up.  How the weights arrive:
//   * a block is persistent: it walks tiles of ROWS weight rows (tile, tile + grid, ...);
//   * one producer thread issues cp.async.bulk copies of row segments (KT elements of each
//     of the tile's rows) into a ring of STAGES shared-memory buffers and signals an
//     mbarrier per buffer with the byte count; it runs ahead across tile boundaries, so
//     HBM requests never drain while a tile's epilogue runs;
//   * eight consumer warps wait for a buffer, read their 64-element slice of every row
//     straight from it (rows are padded so that the 16-byte reads hit distinct banks),
//     multiply, and hand the buffer back through a second mbarrier.
// Two blocks run per SM.  Widths that are whole spans of 64 columns take the second kernel of
// this file, which brings a stage with one tensor copy instead of sixteen row-segment copies.
//
// The producer starts before the kernel that makes x has finished (weights never change);
// consumers wait for it before they read x.  Every mbarrier wait is bounded: after
// WAIT_LIMIT polls a thread records an error code in `status` and goes on, so the kernel
// always ends and the host sees the code.
//
// Reference: the hand-written few-row products of hvasconcelos/mlxforge,
// src/model/skinny_matmul.cpp:17-140 (weights streamed once, fp32 accumulation).
#include "common.cuh"
#include "tma_host.cuh"

namespace {

int g_stream_tensor_copies = 1;     // 0: row-segment copies for every width (mf_set_stream_tensor_copies)

constexpr int CW = 8;                 // consumer warps
constexpr int KT = 512;               // elements of K per stage
constexpr int ROW_BYTES = KT * 2 + 64;   // +64: row r starts 16 banks after row r-1
constexpr unsigned WAIT_LIMIT = 1u << 24;

template <int ROWS> struct Ring { static constexpr int STAGES = ROWS == 16 ? 5 : 10; };

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// true when the phase with this parity has completed; bounded
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int* status, int code) {
  for (unsigned i = 0; i < WAIT_LIMIT; i++) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  if (status) atomicExch(status, code);
  return false;
}
__device__ __forceinline__ void bulk_copy(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint4 lds128(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Before the producer copies into a stage that the consumers have read.  Their reads are ordinary loads
// (generic proxy), the copy comes from the copy engine (async proxy), and an mbarrier orders accesses
// within one proxy only: the thread that issues the copy puts a proxy fence between its wait for the
// stage and the copy.  Without it a lane now and then multiplied with the NEXT copy's bytes (weights
// coded by tile and stage showed it: 16 rows of x, 2048 x 8192, wrong in 595 of 600 launches, 17 of
// 600 at 16384 x 2048; with the fence 0 of 600, whether the readers fence before they hand the stage
// back or the producer fences once it has it: the latter is one thread's fence, off the readers' path).
__device__ __forceinline__ void stage_is_mine() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CW * 32) : "memory"); }

template <int NB, int ROWS, typename OutT>
__global__ void __launch_bounds__((CW + 1) * 32)
stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W, OutT* __restrict__ out,
              int M, int N, int K, int mode, int* __restrict__ status) {
  constexpr int STAGES = Ring<ROWS>::STAGES;
  constexpr int STAGE_BYTES = ROWS * ROW_BYTES;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* ring = smem;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + STAGES * STAGE_BYTES);   // full[S], empty[S]
  float* red = reinterpret_cast<float*>(bars + 2 * STAGES);                                        // [CW][ROWS][NB*8+1]
  constexpr int RED_M = NB * 8 + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (N + ROWS - 1) / ROWS, n_ks = (K + KT - 1) / KT;
  const unsigned ring_u = smem_u32(ring), bars_u = smem_u32(bars);

  if (threadIdx.x == 0) {
    pdl_launch();            // the kernels after this one take an SM's room as blocks of this one leave
    for (int s = 0; s < STAGES; s++) {
      mbar_init(bars_u + 8 * s, 1);                  // full: the producer's arrive + the bytes
      mbar_init(bars_u + 8 * (STAGES + s), CW);      // empty: one arrive per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  if (warp == CW) {
    // ------------------------------------------------------------ producer (one warp)
    // lane 0 waits for the buffer and announces the byte count; lane r then copies row r, so the
    // rows of a stage are issued side by side and not one after the other by a single thread
    unsigned it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      const int n0 = tile * ROWS, nvalid = min(ROWS, N - n0);
      for (int ks = 0; ks < n_ks; ks++, it++) {
        const unsigned s = it % STAGES, round = it / STAGES;
        const unsigned kbytes = (unsigned)min(KT, K - ks * KT) * 2u;
        const unsigned full = bars_u + 8 * s;
        if (lane == 0) {
          if (round > 0) mbar_wait(bars_u + 8 * (STAGES + s), (round - 1) & 1, status, 1);
          mbar_expect_tx(full, kbytes * (unsigned)nvalid);
        }
        __syncwarp();
        stage_is_mine();       // every lane that copies: after lane 0's wait, before its own copy
        if (lane < nvalid)
          bulk_copy(ring_u + s * STAGE_BYTES + lane * ROW_BYTES,
                    W + (long long)(n0 + lane) * K + (long long)ks * KT, kbytes, full);
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumers (8 warps)
  const int g = lane >> 2, t = lane & 3;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  pdl_wait();                // x comes from the kernel before this one
  unsigned it = 0;
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int n0 = tile * ROWS;
    const bool va = n0 + g < N, vb = (ROWS == 16) && n0 + g + 8 < N;
    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; nb++) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;

    for (int ks = 0; ks < n_ks; ks++, it++) {
      const unsigned s = it % STAGES, round = it / STAGES;
      // this warp's 64 elements of the stage, as two pieces of 32: x first (it does not wait for the weights)
      uint4 xv[2][NB];
      const int kl = warp * 64 + t * 8;
#pragma unroll
      for (int c = 0; c < 2; c++) {
        const int k = ks * KT + kl + c * 32;
#pragma unroll
        for (int nb = 0; nb < NB; nb++) {
          const int m = nb * 8 + g;
          xv[c][nb] = (k < K && m < M) ? __ldg(reinterpret_cast<const uint4*>(x + (long long)m * K + k)) : zero;
        }
      }
      mbar_wait(bars_u + 8 * s, round & 1, status, 2);
      const unsigned base = ring_u + s * STAGE_BYTES + kl * 2;
#pragma unroll
      for (int c = 0; c < 2; c++) {
        const bool in = ks * KT + kl + c * 32 < K;
        const uint4 a = (in && va) ? lds128(base + g * ROW_BYTES + c * 64) : zero;
        const uint4 b = (in && vb) ? lds128(base + (g + 8) * ROW_BYTES + c * 64) : zero;
#pragma unroll
        for (int nb = 0; nb < NB; nb++) {
          mma_bf16(acc[nb], a.x, b.x, a.y, b.y, xv[c][nb].x, xv[c][nb].y);
          mma_bf16(acc[nb], a.z, b.z, a.w, b.w, xv[c][nb].z, xv[c][nb].w);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars_u + 8 * (STAGES + s));
    }

    // ---- sum the 8 warps' partial results in a fixed order
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {
      red[(warp * ROWS + g) * RED_M + nb * 8 + 2 * t] = acc[nb][0];
      red[(warp * ROWS + g) * RED_M + nb * 8 + 2 * t + 1] = acc[nb][1];
      if (ROWS == 16) {
        red[(warp * ROWS + g + 8) * RED_M + nb * 8 + 2 * t] = acc[nb][2];
        red[(warp * ROWS + g + 8) * RED_M + nb * 8 + 2 * t + 1] = acc[nb][3];
      }
    }
    consumer_sync();
    if (mode == 0) {
      for (int i = threadIdx.x; i < ROWS * NB * 8; i += CW * 32) {
        const int m = i / ROWS, r = i - m * ROWS;
        if (m >= M || n0 + r >= N) continue;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < CW; w++) sum += red[(w * ROWS + r) * RED_M + m];
        out[(long long)m * N + n0 + r] = from_f32<OutT>(sum);
      }
    } else {
      constexpr int HALF = ROWS / 2;       // rows 0..7 of a tile are gate rows, 8..15 the matching up rows
      for (int i = threadIdx.x; i < HALF * NB * 8; i += CW * 32) {
        const int m = i / HALF, r = i - m * HALF;
        if (m >= M || n0 + r + HALF >= N) continue;
        float gs = 0.f, us = 0.f;
#pragma unroll
        for (int w = 0; w < CW; w++) {
          gs += red[(w * ROWS + r) * RED_M + m];
          us += red[(w * ROWS + r + HALF) * RED_M + m];
        }
        out[(long long)m * (N / 2) + tile * HALF + r] = from_f32<OutT>(gs / (1.0f + expf(-gs)) * us);
      }
    }
    consumer_sync();       // `red` is free for the next tile
  }
}


// ---------------------------------------------------------------------------------------------
// The same product with ONE tensor copy per stage.  Row segments of 1 KB cost the copy engine an
// instruction each, and at sixteen per stage it is the rate of those, not HBM, that bounds the
// stream (about 6.0 TB/s here against 7.0 with one 16 KB copy).  The matrix is described to the
// engine as [K/64 chunks][N rows][64 elements]; a box of (8 chunks x 16 rows) or (16 chunks x 8
// rows) is one stage, stored [chunk][row][128 bytes] with the 128-byte swizzle, which also keeps
// the fragment reads off each other's banks: a thread takes the 16-byte pieces 2t and 2t+1 of
// its warp's chunk, so the eight threads of a quarter-warp (rows g, g+1) touch eight different
// pieces.  Needs K to be whole spans of 64 columns; other widths take the kernel above.
// Stages of the ring: six (see dispatch()).
constexpr int T_STAGE_BYTES = 16384;

__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

template <int NB, int ROWS, int T_STAGES, typename OutT>
__global__ void __launch_bounds__((CW + 1) * 32)
stream_tmap_kernel(const __nv_bfloat16* __restrict__ x, const __grid_constant__ CUtensorMap map,
                   OutT* __restrict__ out, int M, int N, int K, int mode, int* __restrict__ status) {
  constexpr int SUB = 16 / ROWS;                 // chunks of 64 per warp and stage (1 or 2)
  constexpr int KSTAGE = 512 * SUB;              // elements of K per stage
  constexpr int CHUNK_BYTES = ROWS * 128;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + T_STAGES * T_STAGE_BYTES);
  float* red = reinterpret_cast<float*>(bars + 2 * T_STAGES);                                      // [CW][ROWS][NB*8+1]
  constexpr int RED_M = NB * 8 + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (N + ROWS - 1) / ROWS, n_ks = (K + KSTAGE - 1) / KSTAGE;
  const unsigned ring_u = smem_u32(smem), bars_u = smem_u32(bars);

  if (threadIdx.x == 0) {
    pdl_launch();            // the kernels after this one take an SM's room as blocks of this one leave
    for (int s = 0; s < T_STAGES; s++) {
      mbar_init(bars_u + 8 * s, 1);
      mbar_init(bars_u + 8 * (T_STAGES + s), CW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  if (warp == CW) {
    if (lane == 0) {
      unsigned it = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        for (int ks = 0; ks < n_ks; ks++, it++) {
          const unsigned s = it % T_STAGES, round = it / T_STAGES;
          if (round > 0) {
            mbar_wait(bars_u + 8 * (T_STAGES + s), (round - 1) & 1, status, 1);
            stage_is_mine();
          }
          mbar_expect_tx(bars_u + 8 * s, T_STAGE_BYTES);       // rows outside the matrix arrive as zeros
          tma_load_3d(ring_u + s * T_STAGE_BYTES, &map, 0, tile * ROWS, ks * (KSTAGE / 64), bars_u + 8 * s);
        }
      }
    }
    return;
  }

  const int g = lane >> 2, t = lane & 3;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  pdl_wait();                // x comes from the kernel before this one
  unsigned it = 0;
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int n0 = tile * ROWS;
    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; nb++) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;

    for (int ks = 0; ks < n_ks; ks++, it++) {
      const unsigned s = it % T_STAGES, round = it / T_STAGES;
      // x first (it does not wait for the weights): pieces 2t and 2t+1 of this warp's chunk(s)
      uint4 xv[SUB][2][NB];
#pragma unroll
      for (int h = 0; h < SUB; h++)
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const int k = ks * KSTAGE + (warp + CW * h) * 64 + (2 * t + c) * 8;
#pragma unroll
          for (int nb = 0; nb < NB; nb++) {
            const int m = nb * 8 + g;
            xv[h][c][nb] = (k < K && m < M) ? __ldg(reinterpret_cast<const uint4*>(x + (long long)m * K + k)) : zero;
          }
        }
      mbar_wait(bars_u + 8 * s, round & 1, status, 2);
#pragma unroll
      for (int h = 0; h < SUB; h++) {
        const unsigned base = ring_u + s * T_STAGE_BYTES + (warp + CW * h) * CHUNK_BYTES + g * 128;
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const unsigned piece = (unsigned)((2 * t + c) ^ g) << 4;
          const uint4 a = lds128(base + piece);
          const uint4 b = ROWS == 16 ? lds128(base + 1024 + piece) : zero;
#pragma unroll
          for (int nb = 0; nb < NB; nb++) {
            mma_bf16(acc[nb], a.x, b.x, a.y, b.y, xv[h][c][nb].x, xv[h][c][nb].y);
            mma_bf16(acc[nb], a.z, b.z, a.w, b.w, xv[h][c][nb].z, xv[h][c][nb].w);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars_u + 8 * (T_STAGES + s));
    }

    // ---- sum the 8 warps' partial results in a fixed order
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {
      red[(warp * ROWS + g) * RED_M + nb * 8 + 2 * t] = acc[nb][0];
      red[(warp * ROWS + g) * RED_M + nb * 8 + 2 * t + 1] = acc[nb][1];
      if (ROWS == 16) {
        red[(warp * ROWS + g + 8) * RED_M + nb * 8 + 2 * t] = acc[nb][2];
        red[(warp * ROWS + g + 8) * RED_M + nb * 8 + 2 * t + 1] = acc[nb][3];
      }
    }
    consumer_sync();
    if (mode == 0) {
      for (int i = threadIdx.x; i < ROWS * NB * 8; i += CW * 32) {
        const int m = i / ROWS, r = i - m * ROWS;
        if (m >= M || n0 + r >= N) continue;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < CW; w++) sum += red[(w * ROWS + r) * RED_M + m];
        out[(long long)m * N + n0 + r] = from_f32<OutT>(sum);
      }
    } else {
      constexpr int HALF = ROWS / 2;       // rows 0..7 of a tile are gate rows, 8..15 the matching up rows
      for (int i = threadIdx.x; i < HALF * NB * 8; i += CW * 32) {
        const int m = i / HALF, r = i - m * HALF;
        if (m >= M || n0 + r + HALF >= N) continue;
        float gs = 0.f, us = 0.f;
#pragma unroll
        for (int w = 0; w < CW; w++) {
          gs += red[(w * ROWS + r) * RED_M + m];
          us += red[(w * ROWS + r + HALF) * RED_M + m];
        }
        out[(long long)m * (N / 2) + tile * HALF + r] = from_f32<OutT>(gs / (1.0f + expf(-gs)) * us);
      }
    }
    consumer_sync();       // `red` is free for the next tile
  }
}

template <int NB, int ROWS, int T_STAGES, typename OutT>
int launch_tmap(const __nv_bfloat16* x, const __nv_bfloat16* W, OutT* out, int M, int N, int K, int mode, int* status,
                int n_sms, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)T_STAGES * T_STAGE_BYTES + 2 * T_STAGES * 8 + (size_t)CW * ROWS * (NB * 8 + 1) * 4;
  static DeviceOnce once;
  const int dev_ = mf_current_device();
  if (dev_ < 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev_]) {
    cudaError_t e = cudaFuncSetAttribute(stream_tmap_kernel<NB, ROWS, T_STAGES, OutT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    once.done[dev_] = true;
  }
  CUtensorMap map;
  const int rc = tma_host::bf16_map_chunked(W, N, K, ROWS, 128 / ROWS, &map);
  if (rc != 0) return rc;
  const int n_tiles = (N + ROWS - 1) / ROWS;
  // as many blocks as give every block the same number of tiles (to within one): 1024 tiles on
  // 296 block slots are four rounds either way, and 256 blocks of four tiles end together
  const int rounds = (n_tiles + 2 * n_sms - 1) / (2 * n_sms);
  const int grid = (n_tiles + rounds - 1) / rounds;
  mf_count(MF_K_STREAM_TMAP);
  return (int)launch_dep(stream_tmap_kernel<NB, ROWS, T_STAGES, OutT>, dim3(grid), dim3((CW + 1) * 32), smem, stream, x, map,
                         out, M, N, K, mode, status);
}

template <int NB, int ROWS, typename OutT>
int launch_one(const __nv_bfloat16* x, const __nv_bfloat16* W, OutT* out, int M, int N, int K, int mode, int* status,
               int n_sms, cudaStream_t stream) {
  constexpr int STAGES = Ring<ROWS>::STAGES;
  const size_t smem = (size_t)STAGES * ROWS * ROW_BYTES + 2 * STAGES * 8 + (size_t)CW * ROWS * (NB * 8 + 1) * 4;
  static DeviceOnce once;
  const int dev_ = mf_current_device();
  if (dev_ < 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev_]) {
    cudaError_t e = cudaFuncSetAttribute(stream_kernel<NB, ROWS, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);   // smem depends on the template arguments only
    if (e != cudaSuccess) return (int)e;
    once.done[dev_] = true;
  }
  const int n_tiles = (N + ROWS - 1) / ROWS;
  // two blocks per SM
  const int grid = n_tiles < 2 * n_sms ? n_tiles : 2 * n_sms;
  mf_count(MF_K_STREAM_ROWS);
  return (int)launch_dep(stream_kernel<NB, ROWS, OutT>, dim3(grid), dim3((CW + 1) * 32), smem, stream, x, W, out, M,
                         N, K, mode, status);
}

template <typename OutT>
int dispatch(const __nv_bfloat16* x, const __nv_bfloat16* W, OutT* out, int M, int N, int K, int mode, int* status,
             cudaStream_t stream) {
  const int n_sms = mf_sm_count();
  if (n_sms <= 0) return MF_ERR_BAD_ARG;
  // few output rows: tiles of 8 rows, so that there are blocks for every SM
  const bool small = mode == 0 && (N + 15) / 16 < 2 * n_sms;
  // Tensor copies for every width of whole 64-column spans; a box that hangs over the end of the
  // matrix along K arrives with zeros there and counts its full size.  (Widths that are not whole
  // stages were once kept off this path because 3 x 128256 x 64 gave wrong rows: that was the
  // missing fence of stage_is_mine(), which shows most where a block has many one-stage tiles.)
  if (K % 64 == 0 && g_stream_tensor_copies) {
    // Six stages of 16 KB, two blocks per SM: under load a copy takes 3 to 4 us to arrive, so an SM
    // has to keep nearly all of its shared memory on the way (four stages: 1.141 ms for a decode step
    // of batch 8, six: 1.133, and 1.102 against 1.117 once the kernels before let this one start early).
    if (M <= 8)
      return small ? launch_tmap<1, 8, 6, OutT>(x, W, out, M, N, K, mode, status, n_sms, stream)
                   : launch_tmap<1, 16, 6, OutT>(x, W, out, M, N, K, mode, status, n_sms, stream);
    if (M <= 16)
      return small ? launch_tmap<2, 8, 6, OutT>(x, W, out, M, N, K, mode, status, n_sms, stream)
                   : launch_tmap<2, 16, 6, OutT>(x, W, out, M, N, K, mode, status, n_sms, stream);
    return MF_ERR_BAD_ARG;
  }
  if (M <= 8) {
    return small ? launch_one<1, 8, OutT>(x, W, out, M, N, K, mode, status, n_sms, stream)
                 : launch_one<1, 16, OutT>(x, W, out, M, N, K, mode, status, n_sms, stream);
  }
  if (M <= 16) {
    return small ? launch_one<2, 8, OutT>(x, W, out, M, N, K, mode, status, n_sms, stream)
                 : launch_one<2, 16, OutT>(x, W, out, M, N, K, mode, status, n_sms, stream);
  }
  return MF_ERR_BAD_ARG;
}

}  // namespace

MF_API int mf_stream_max_rows() { return 16; }

// 1 (the default): widths that are a multiple of 64 stream with one tensor copy per stage;
// 0: every width streams with row-segment copies.  For tests and measurements.
MF_API int mf_set_stream_tensor_copies(int on) {
  g_stream_tensor_copies = on ? 1 : 0;
  return 0;
}

// mode 0: out [M, N] in out_dtype.  mode 1: W rows interleave gate and up in groups of 8 (N a
// multiple of 16) and out is [M, N / 2] = silu(gate) * up.  K must be a multiple of 8 and x, W
// 16-byte aligned.  `status`: a device int (may be null) that receives a non-zero code if a wait
// inside the kernel ran out (1: producer, 2: consumer).
MF_API int mf_stream_linear(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K, int mode,
                            int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || M > 16 || (mode != 0 && mode != 1)) return MF_ERR_BAD_ARG;
  if (mode == 1 && N % 16) return MF_ERR_BAD_ARG;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return MF_ERR_BAD_ARG;
  const __nv_bfloat16 *xx = (const __nv_bfloat16*)x, *ww = (const __nv_bfloat16*)W;
  if (out_dtype == MF_BF16) return dispatch<__nv_bfloat16>(xx, ww, (__nv_bfloat16*)out, M, N, K, mode, status, stream);
  if (out_dtype == MF_F32) return dispatch<float>(xx, ww, (float*)out, M, N, K, mode, status, stream);
  return MF_ERR_BAD_DTYPE;
}
