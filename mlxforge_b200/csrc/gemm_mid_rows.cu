// out[M, N] = x[M, K] * W[N, K]^T for 17 to 128 rows of x (a decode step of that many requests):
// bfloat16 operands, float32 accumulation in tensor memory, weights streamed once.
//
// With so few rows the product is bound by reading W, so the weights go on the M side of the
// tensor-core instruction: D[128 weight rows, NT tokens] += W_tile[128, 16] * x_tile[NT, 16]^T
// (tcgen05.mma cta_group::1 kind::f16, M = 128, N = NT = M rounded up to 16), and the work is cut
// so that every SM streams the same number of weight bytes whatever the matrix's shape:
//   * a unit is one 128-row x 64-column piece of W (16 KB) with the matching 64 columns of x;
//     units are numbered tile after tile, along K inside a tile;
//   * the grid is one persistent block per SM; block g takes units [g U / G, (g + 1) U / G), so a
//     block's share may begin in the middle of one tile and end in the middle of another;
//   * warp 0 brings a unit's two boxes in by TMA (128-byte swizzle) into a ring of stages, warp 1
//     issues the four products of a unit and hands the stage back with tcgen05.commit, warps 2-5
//     read the accumulator (tcgen05.ld; a thread holds one weight row = one output column) and
//     store; two accumulators alternate so that an epilogue runs under the next part's products;
//   * a tile that one block computes whole is stored straight away.  A tile shared by several
//     blocks: each writes its partial sums to scratch and takes a ticket; whoever takes the last
//     ticket adds the partial sums in the order of their K ranges (so the result does not depend
//     on who was last) and stores.  Nobody waits for anybody.
// The weights' boxes are requested before the kernel waits for its predecessor (they never
// change); x, the scratch and the output are touched after it.  Every mbarrier wait is bounded and
// reports through `status`; tensor memory is freed in every case.
//
// Reference: the few-row products that hvasconcelos/mlxforge writes by hand for 2 to 32 rows
// (src/model/skinny_matmul.cpp:95-140, gate :161-173); above that it uses its library's matmul.
#include "common.cuh"
#include "tma_host.cuh"

namespace {

constexpr int TILE = 128;              // weight rows per tile
constexpr int BK = 64;                 // columns of K per operand tile (one 128-byte swizzle span)
constexpr int W_BYTES = TILE * BK * 2;
constexpr int RING_BYTES = 200 * 1024;
constexpr unsigned WAIT_LIMIT = 1u << 26;
constexpr int MAX_TILES = 1 << 16;

// One ticket per tile: how many of its parts are in scratch.  Zero between launches (the block that
// takes a tile's last ticket puts it back).  Launches of this kernel on one device must follow one
// another on a stream, as the engine's do.
__device__ int g_mid_tickets[MAX_TILES];

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
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
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* map, int c0, int c1, int c2, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// One unit's piece of a matrix: CHUNKS spans of 64 columns starting at span k * CHUNKS, `rows` rows from row0.
// CHUNKS == 1: a 2-D box; else one 3-D box of the matrix seen as [K/64][rows][64] (tma_host::bf16_map_chunked),
// which lands as CHUNKS operand tiles one after the other.
template <int CHUNKS>
__device__ __forceinline__ void load_piece(unsigned dst, const CUtensorMap* map, int k, int row0, unsigned bar) {
  if (CHUNKS == 1) tma_load_2d(dst, map, k * BK, row0, bar);
  else tma_load_3d(dst, map, 0, row0, k * CHUNKS, bar);
}
// K-major operand tile, rows of 64 bfloat16 (128 bytes), 128-byte swizzle: groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr >> 4) & 0x3FFF);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
__device__ __forceinline__ void umma(unsigned tmem_c, unsigned long long da, unsigned long long db, unsigned idesc,
                                     unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]);
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

// Which block's share holds unit u, for shares [g U / G, (g + 1) U / G).
__device__ __forceinline__ int share_of(long long u, long long U, int G) {
  int g = (int)(u * G / U);
  while (g + 1 < G && (long long)(g + 1) * U / G <= u) g++;
  while (g > 0 && (long long)g * U / G > u) g--;
  return g;
}

// Stores 16 tokens (m0 .. m0 + 15) of this thread's weight row `n`.  MODE 0: out[m, n] in OutT.
// MODE 1: the rows of W interleave gate and up in groups of 8, so lanes l and l + 8 (l % 16 < 8)
// hold a pair; out[m, n / 16 * 8 + n % 8] = silu(gate) * up, bfloat16.
template <int MODE, typename OutT>
__device__ __forceinline__ void store16(OutT* __restrict__ out, const float (&v)[16], int m0, int M, int n, int N) {
  if (MODE == 0) {
    if (n >= N) return;
#pragma unroll
    for (int j = 0; j < 16; j++)
      if (m0 + j < M) out[(long long)(m0 + j) * N + n] = from_f32<OutT>(v[j]);
  } else {
    const bool gate = (n & 8) == 0;
    const int col = (n >> 4) * 8 + (n & 7);
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const float up = __shfl_down_sync(0xffffffffu, v[j], 8);
      if (gate && n + 8 < N && m0 + j < M)
        out[(long long)(m0 + j) * (N / 2) + col] = from_f32<OutT>(v[j] / (1.0f + expf(-v[j])) * up);
    }
  }
}

template <int MODE, int CHUNKS, typename OutT>
__global__ void __launch_bounds__(192, 1)
mid_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                OutT* __restrict__ out, float* __restrict__ scratch, int M, int N, int K, int NT, int stages,
                int* __restrict__ status) {
  extern __shared__ unsigned char raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  const int stage_bytes = CHUNKS * (W_BYTES + NT * BK * 2);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + stages * stage_bytes);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * stages + 4);
  int* flag = reinterpret_cast<int*>(tmem_slot + 1);
  const unsigned smem_u = smem_u32(smem), bars_u = smem_u32(bars);
  const unsigned full0 = bars_u, empty0 = bars_u + 8 * stages;
  const unsigned acc_full0 = bars_u + 16 * stages, acc_empty0 = acc_full0 + 16;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, g = blockIdx.x;
  const int kb = (K + BK * CHUNKS - 1) / (BK * CHUNKS);
  const long long U = (long long)((N + TILE - 1) / TILE) * kb;
  const long long u0 = (long long)g * U / G, u1 = (long long)(g + 1) * U / G;
  const unsigned tmem_cols = NT <= 16 ? 32u : NT <= 32 ? 64u : NT <= 64 ? 128u : 256u;   // two accumulators

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; s++) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(acc_full0 + 8 * a, 1);
      mbar_init(acc_empty0 + 8 * a, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // the weights of the first ring-full of units do not wait for the kernel before this one
      const long long ahead = u1 - u0 < stages ? u1 - u0 : stages;
      for (long long i = 0; i < ahead; i++) {
        const long long u = u0 + i;
        const int tile = (int)(u / kb), k = (int)(u % kb);
        mbar_expect_tx(full0 + 8 * (unsigned)i, (unsigned)stage_bytes);
        load_piece<CHUNKS>(smem_u + (unsigned)i * stage_bytes, &map_w, k, tile * TILE, full0 + 8 * (unsigned)i);
      }
      pdl_wait();
      pdl_launch();
      for (long long i = 0; i < ahead; i++) {
        const int k = (int)((u0 + i) % kb);
        load_piece<CHUNKS>(smem_u + (unsigned)i * stage_bytes + CHUNKS * W_BYTES, &map_x, k, 0, full0 + 8 * (unsigned)i);
      }
      for (long long i = ahead; i < u1 - u0; i++) {
        const long long u = u0 + i;
        const int tile = (int)(u / kb), k = (int)(u % kb);
        const unsigned s = (unsigned)(i % stages), round = (unsigned)(i / stages);
        mbar_wait(empty0 + 8 * s, (round - 1) & 1, status, 21);
        mbar_expect_tx(full0 + 8 * s, (unsigned)stage_bytes);
        load_piece<CHUNKS>(smem_u + s * stage_bytes, &map_w, k, tile * TILE, full0 + 8 * s);
        load_piece<CHUNKS>(smem_u + s * stage_bytes + CHUNKS * W_BYTES, &map_x, k, 0, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(NT >> 3) << 17) | ((unsigned)(TILE >> 4) << 24);
      unsigned part = 0;
      long long i = 0;
      for (long long u = u0; u < u1; part++) {
        const long long tile_end = (u / kb + 1) * kb;
        const long long pe = tile_end < u1 ? tile_end : u1;       // this part: units [u, pe) of one tile
        const unsigned acc = part & 1, use = part >> 1;
        if (use > 0) {
          mbar_wait(acc_empty0 + 8 * acc, (use - 1) & 1, status, 24);
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        }
        const unsigned tmem_c = tmem_base + acc * (unsigned)NT;
        for (bool first = true; u < pe; u++, i++) {
          const unsigned s = (unsigned)(i % stages), round = (unsigned)(i / stages);
          mbar_wait(full0 + 8 * s, round & 1, status, 22);
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned a_addr = smem_u + s * stage_bytes, b_addr = a_addr + CHUNKS * W_BYTES;
#pragma unroll
          for (int c = 0; c < CHUNKS; c++)
#pragma unroll
            for (int k4 = 0; k4 < BK / 16; k4++) {
              umma(tmem_c, smem_desc(a_addr + c * W_BYTES + k4 * 32), smem_desc(b_addr + c * NT * BK * 2 + k4 * 32), idesc,
                   first ? 0u : 1u);
              first = false;
            }
          umma_commit(empty0 + 8 * s);
        }
        umma_commit(acc_full0 + 8 * acc);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, 32 weight rows each)
    const int lg = warp & 3;
    const int r = lg * 32 + lane;                 // this thread's row of the tile
    const int et = threadIdx.x - 64;              // 0..127 among the epilogue threads
    pdl_wait();
    unsigned part = 0;
    for (long long u = u0; u < u1; part++) {
      const int tile = (int)(u / kb);
      const long long tile_begin = (long long)tile * kb, tile_end = tile_begin + kb;
      const long long pe = tile_end < u1 ? tile_end : u1;
      const bool whole = u == tile_begin && pe == tile_end;
      const unsigned acc = part & 1, use = part >> 1;
      const int n = tile * TILE + r;
      mbar_wait(acc_full0 + 8 * acc, use & 1, status, 23);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const unsigned taddr = tmem_base + ((unsigned)(lg * 32) << 16) + acc * (unsigned)NT;
      if (whole) {
        for (int c = 0; c < NT; c += 16) {
          float v[16];
          tmem_ld16(taddr + (unsigned)c, v);
          if (c < M) store16<MODE, OutT>(out, v, c, M, n, N);
        }
      } else {
        // this block's partial sums of the tile: slot 0 for the tile its share begins in, 1 otherwise
        const int slot = 2 * g + (tile == (int)(u0 / kb) ? 0 : 1);
        float* mine = scratch + (long long)slot * NT * TILE;
        for (int c = 0; c < NT; c += 16) {
          float v[16];
          tmem_ld16(taddr + (unsigned)c, v);
#pragma unroll
          for (int j = 0; j < 16; j++) __stcg(mine + (c + j) * TILE + r, v[j]);
        }
      }
      // the accumulator is free for the part after next
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(acc_empty0 + 8 * acc) : "memory");
      if (!whole) {
        const int g_first = share_of(tile_begin, U, G), g_last = share_of(tile_end - 1, U, G);
        __threadfence();
        epilogue_sync();
        if (et == 0) {
          const int last = atomicAdd(g_mid_tickets + tile, 1) == g_last - g_first;
          if (last) g_mid_tickets[tile] = 0;
          *flag = last;
        }
        epilogue_sync();
        const bool last = *flag != 0;
        epilogue_sync();          // everyone has read the flag before the next part writes it
        if (last) {
          __threadfence();
          for (int c = 0; c < NT && c < M; c += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] = 0.f;
            for (int p = g_first; p <= g_last; p++) {
              const int pslot = 2 * p + (tile == (int)(((long long)p * U / G) / kb) ? 0 : 1);
              const float* theirs = scratch + (long long)pslot * NT * TILE;
#pragma unroll
              for (int j = 0; j < 16; j++) v[j] += __ldcg(theirs + (c + j) * TILE + r);
            }
            store16<MODE, OutT>(out, v, c, M, n, N);
          }
        }
      }
      u = pe;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(tmem_cols));
  }
}

int g_mid_chunks = 2;     // spans of 64 columns per unit where K allows it (mf_set_mid_rows_chunks)

template <int MODE, int CHUNKS, typename OutT>
int launch(const void* x, const void* W, OutT* out, float* scratch, int M, int N, int K, int* status,
           cudaStream_t stream) {
  const int NT = (M + 15) / 16 * 16;
  const int stage_bytes = CHUNKS * (W_BYTES + NT * BK * 2);
  const int stages = RING_BYTES / stage_bytes;
  CUtensorMap mw, mx;
  int rc = CHUNKS == 1 ? tma_host::bf16_map(W, N, K, TILE, BK, &mw) : tma_host::bf16_map_chunked(W, N, K, TILE, CHUNKS, &mw);
  if (rc) return rc;
  rc = CHUNKS == 1 ? tma_host::bf16_map(x, M, K, NT, BK, &mx) : tma_host::bf16_map_chunked(x, M, K, NT, CHUNKS, &mx);
  if (rc) return rc;
  const size_t smem = (size_t)stages * stage_bytes + (2 * stages + 4) * 8 + 16 + 1024;
  static DeviceOnce once;
  const int dev_ = mf_current_device();
  const int n_sms = mf_sm_count();
  if (dev_ < 0 || n_sms <= 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev_]) {
    cudaError_t e = cudaFuncSetAttribute(mid_rows_kernel<MODE, CHUNKS, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         RING_BYTES + 2048);
    if (e != cudaSuccess) return (int)e;
    once.done[dev_] = true;
  }
  const long long U = (long long)((N + TILE - 1) / TILE) * ((K + BK * CHUNKS - 1) / (BK * CHUNKS));
  // every block at least two units, so that a share is never empty and rarely a sliver
  long long G = U / 2 < n_sms ? U / 2 : n_sms;
  if (G < 1) G = 1;
  mf_count(MF_K_MID_ROWS);
  return (int)launch_dep(mid_rows_kernel<MODE, CHUNKS, OutT>, dim3((unsigned)G), dim3(192), smem, stream, mw, mx, out, scratch, M,
                         N, K, NT, stages, status);
}

// Units of several spans where K is whole units (the unit's k-steps are counted from K, so a unit that
// hangs over would multiply zero-filled spans for nothing); other widths take one span per unit
// through 2-D boxes.
template <int MODE, typename OutT>
int launch_for_width(const void* x, const void* W, OutT* out, float* scratch, int M, int N, int K, int* status,
                     cudaStream_t stream) {
  if (g_mid_chunks >= 4 && K % (4 * BK) == 0) return launch<MODE, 4, OutT>(x, W, out, scratch, M, N, K, status, stream);
  if (g_mid_chunks >= 2 && K % (2 * BK) == 0) return launch<MODE, 2, OutT>(x, W, out, scratch, M, N, K, status, stream);
  return launch<MODE, 1, OutT>(x, W, out, scratch, M, N, K, status, stream);
}

}  // namespace

// 1, 2 or 4 spans of 64 columns per unit (for measurements; widths that are no multiple fall back to 1).
MF_API int mf_set_mid_rows_chunks(int chunks) {
  const int old = g_mid_chunks;
  g_mid_chunks = chunks >= 4 ? 4 : chunks >= 2 ? 2 : 1;
  return old;
}

// Rows of x this kernel takes: more than the streamed few-row product, up to one instruction's width.
MF_API int mf_mid_rows_min() { return 17; }
MF_API int mf_mid_rows_max() { return 128; }

// float32 elements of scratch a call needs (the partial sums of tiles shared between blocks).
MF_API long long mf_mid_rows_scratch(int M) {
  const int n_sms = mf_sm_count();
  const long long NT = (M + 15) / 16 * 16;
  return 2ll * (n_sms > 0 ? n_sms : 256) * NT * TILE;
}

// Puts the tickets back to zero after a kernel of this file gave up a bounded wait.
MF_API int mf_reset_mid_rows_tickets(cudaStream_t stream) {
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_mid_tickets);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemsetAsync(p, 0, sizeof(int) * MAX_TILES, stream);
}

// mode 0: out [M, N] in out_dtype.  mode 1: the rows of W interleave gate and up in groups of 8 (N a
// multiple of 16) and out is bfloat16 or float32 [M, N / 2] = silu(gate) * up.  17 <= M <= 128, K a
// multiple of 8, x and W 16-byte aligned.  `scratch`: mf_mid_rows_scratch(M) floats.  `status` as in
// mf_stream_linear (codes 21: producer, 22 and 24: MMA issuer, 23: epilogue).
MF_API int mf_mid_rows_linear(const void* x, const void* W, void* out, int out_dtype, float* scratch, int M, int N,
                              int K, int mode, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || K <= 0 || K % 8 || (mode != 0 && mode != 1)) return MF_ERR_BAD_ARG;
  if (mode == 1 && N % 16) return MF_ERR_BAD_ARG;
  if ((((uintptr_t)x | (uintptr_t)W) & 15) || scratch == nullptr) return MF_ERR_BAD_ARG;
  if ((N + TILE - 1) / TILE > MAX_TILES) return MF_ERR_BAD_ARG;
  if (out_dtype == MF_BF16) {
    __nv_bfloat16* o = (__nv_bfloat16*)out;
    return mode ? launch_for_width<1, __nv_bfloat16>(x, W, o, scratch, M, N, K, status, stream)
                : launch_for_width<0, __nv_bfloat16>(x, W, o, scratch, M, N, K, status, stream);
  }
  if (out_dtype == MF_F32) {
    float* o = (float*)out;
    return mode ? launch_for_width<1, float>(x, W, o, scratch, M, N, K, status, stream)
                : launch_for_width<0, float>(x, W, o, scratch, M, N, K, status, stream);
  }
  return MF_ERR_BAD_DTYPE;
}
