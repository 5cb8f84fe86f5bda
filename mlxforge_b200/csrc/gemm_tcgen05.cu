// C[M, N] = A[M, K] * W[N, K]^T for many rows (prompt portions): bfloat16 operands, float32
// accumulation in tensor memory, on the 5th-generation tensor cores.
//
// A block computes 128 x BN tiles of C (BN = 256 or 128), one after the other:
//   warp 0     one thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of a
//              128 x 64 tile of A and a BN x 64 tile of W into a ring of STAGES buffers, each
//              signalled by an mbarrier with the byte count;
//   warp 1     allocates BN columns of tensor memory; one thread issues tcgen05.mma
//              (cta_group::1, kind::f16, M = 128, N = BN, K = 16: four per 64-wide stage) from
//              shared-memory descriptors and commits each stage back to the producer, then
//              commits the accumulator to the epilogue;
//   warps 2-5  read the accumulator with tcgen05.ld (32 lanes x 32 columns at a time), convert
//              and store: bfloat16, float32 (logits), or the SiLU-gated product for a W whose
//              rows interleave gate and up in groups of 8 (src/model/decoder_model.cpp:277-282).
// Rows and columns beyond M, N and K are zero-filled by the TMA unit and masked at the store.
// Every mbarrier wait is bounded: after WAIT_LIMIT polls a thread records a code in `status`
// and goes on, the tensor memory is freed in every case, and the kernel ends.
//
// The reference runs these products through its tensor library (`mx::matmul`,
// src/model/decoder_model.cpp:191).
#include "common.cuh"
#include "tma_host.cuh"

namespace {

constexpr int BM = 128, BK = 64, STAGES = 4;
constexpr unsigned WAIT_LIMIT = 1u << 26;
constexpr int A_BYTES = BM * BK * 2;

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
// K-major operand tile in shared memory, rows of 64 bfloat16 (128 bytes), 128-byte swizzle:
// groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr >> 4) & 0x3FFF);          // start address
  d |= (unsigned long long)1 << 16;                          // leading byte offset (unused for this layout)
  d |= (unsigned long long)(1024 >> 4) << 32;                // stride byte offset: 8 rows x 128 B
  d |= (unsigned long long)1 << 46;                          // descriptor version of this architecture
  d |= (unsigned long long)2 << 61;                          // 128-byte swizzle
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
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// Stores 32 consecutive columns of one row of the accumulator.
template <int EPI>
__device__ __forceinline__ void store_chunk(void* __restrict__ C, const unsigned (&r)[32], int row, int col, int N) {
  if (EPI == 0) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(C) + (long long)row * N + col;
    if (col + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
      for (int v = 0; v < 4; v++) {
        uint4 pk;
        pk.x = pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
        pk.y = pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
        pk.z = pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
        pk.w = pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
        reinterpret_cast<uint4*>(dst)[v] = pk;
      }
    } else {
      for (int j = 0; j < 32 && col + j < N; j++) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
  } else if (EPI == 1) {
    float* dst = reinterpret_cast<float*>(C) + (long long)row * N + col;
    if (col + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
      for (int v = 0; v < 8; v++)
        reinterpret_cast<float4*>(dst)[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                        __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
    } else {
      for (int j = 0; j < 32 && col + j < N; j++) dst[j] = __uint_as_float(r[j]);
    }
  } else {
    // 32 columns = two groups of [8 gate | 8 up] -> 16 outputs at column col / 2
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(C) + (long long)row * (N / 2) + col / 2;
#pragma unroll
    for (int grp = 0; grp < 2; grp++) {
      if (col + grp * 16 + 16 > N) break;
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; j++)
        o[j] = silu_mul(__uint_as_float(r[grp * 16 + j]), __uint_as_float(r[grp * 16 + 8 + j]));
      if ((((uintptr_t)(dst + grp * 8)) & 15) == 0) {
        uint4 pk;
        pk.x = pack_bf16(o[0], o[1]); pk.y = pack_bf16(o[2], o[3]);
        pk.z = pack_bf16(o[4], o[5]); pk.w = pack_bf16(o[6], o[7]);
        *reinterpret_cast<uint4*>(dst + grp * 8) = pk;
      } else {
        for (int j = 0; j < 8; j++) dst[grp * 8 + j] = __float2bfloat16_rn(o[j]);
      }
    }
  }
}

// EPI 0: C bfloat16 [M, N].  EPI 1: C float32 [M, N].  EPI 2: C bfloat16 [M, N/2] = silu(gate) * up.
// Persistent: a block walks tiles (tile, tile + grid, ...; the M index runs fastest, so blocks
// that run together share tiles of W).  Two accumulators in tensor memory alternate, so the
// epilogue of one tile runs while the products of the next are issued.
template <int BN, int EPI>
__global__ void __launch_bounds__(192)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* __restrict__ C,
            int M, int N, int K, int* __restrict__ status) {
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;
  extern __shared__ unsigned char raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + STAGES * STAGE_BYTES);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 4);
  const unsigned smem_u = smem_u32(smem), bars_u = smem_u32(bars);
  const unsigned full0 = bars_u, empty0 = bars_u + 8 * STAGES;
  const unsigned acc_full0 = bars_u + 16 * STAGES, acc_empty0 = acc_full0 + 16;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_mt = (M + BM - 1) / BM, n_nt = (N + BN - 1) / BN, n_tiles = n_mt * n_nt;
  const int n_kt = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(acc_full0 + 8 * a, 1);       // the issuer's commit
      mbar_init(acc_empty0 + 8 * a, 4);      // one arrive per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      unsigned it = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int m0 = (tile % n_mt) * BM, n0 = (tile / n_mt) * BN;
        for (int kt = 0; kt < n_kt; kt++, it++) {
          const unsigned s = it % STAGES, round = it / STAGES;
          if (round > 0) mbar_wait(empty0 + 8 * s, (round - 1) & 1, status, 11);
          const unsigned full = full0 + 8 * s;
          mbar_expect_tx(full, STAGE_BYTES);
          tma_load_2d(smem_u + s * STAGE_BYTES, &map_a, kt * BK, m0, full);
          tma_load_2d(smem_u + s * STAGE_BYTES + A_BYTES, &map_w, kt * BK, n0, full);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: D float32, A and B bfloat16, both K-major, N, M
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
      unsigned it = 0, i = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, i++) {
        const unsigned acc = i & 1, use = i >> 1;
        if (use > 0) {
          mbar_wait(acc_empty0 + 8 * acc, (use - 1) & 1, status, 14);     // the epilogue has drained it
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        }
        const unsigned tmem_c = tmem_base + acc * BN;
        for (int kt = 0; kt < n_kt; kt++, it++) {
          const unsigned s = it % STAGES, round = it / STAGES;
          mbar_wait(full0 + 8 * s, round & 1, status, 12);
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned a_addr = smem_u + s * STAGE_BYTES, b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; k4++)
            umma(tmem_c, smem_desc(a_addr + k4 * 32), smem_desc(b_addr + k4 * 32), idesc, (kt > 0 || k4 > 0) ? 1u : 0u);
          umma_commit(empty0 + 8 * s);          // the stage is free once these products have read it
        }
        umma_commit(acc_full0 + 8 * acc);        // this tile's accumulator is complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, 32 rows each)
    const int lg = warp & 3;                   // the 32 lanes of tensor memory this warp may read
    unsigned i = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, i++) {
      const int m0 = (tile % n_mt) * BM, n0 = (tile / n_mt) * BN;
      const unsigned acc = i & 1, use = i >> 1;
      const int row = m0 + lg * 32 + lane;
      mbar_wait(acc_full0 + 8 * acc, use & 1, status, 13);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        unsigned r[32];
        tmem_ld32(tmem_base + ((unsigned)(lg * 32) << 16) + acc * BN + (unsigned)(c * 32), r);
        const int col = n0 + c * 32;
        if (row < M && col < N) store_chunk<EPI>(C, r, row, col, N);
      }
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(acc_empty0 + 8 * acc) : "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

// ------------------------------------------------------------------ host side
template <int BN, int EPI>
int launch(const void* A, const void* W, void* C, int M, int N, int K, int* status, cudaStream_t stream) {
  CUtensorMap ma, mw;
  int rc = tma_host::bf16_map(A, M, K, BM, BK, &ma);
  if (rc) return rc;
  rc = tma_host::bf16_map(W, N, K, BN, BK, &mw);
  if (rc) return rc;
  const size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
  static DeviceOnce once;
  const int dev_ = mf_current_device();
  if (dev_ < 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev_]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    once.done[dev_] = true;
  }
  const int n_sms = mf_sm_count();
  if (n_sms <= 0) return MF_ERR_BAD_ARG;
  const int n_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  mf_count(EPI == 2 ? MF_K_GEMM_TC_SWIGLU : MF_K_GEMM_TC);
  gemm_kernel<BN, EPI><<<n_tiles < n_sms ? n_tiles : n_sms, 192, smem, stream>>>(ma, mw, C, M, N, K, status);
  return (int)cudaGetLastError();
}

}  // namespace

// epilogue 0: C bfloat16 [M, N]; 1: C float32 [M, N]; 2: C bfloat16 [M, N/2] = silu(gate) * up for a W
// whose rows interleave gate and up in groups of 8 (N a multiple of 16).
// K must be a multiple of 8 and A, W 16-byte aligned (TMA strides).  `status` as in mf_stream_linear
// (codes 11: producer, 12: MMA issuer, 13: epilogue).
MF_API int mf_gemm_bf16(const void* A, const void* W, void* C, int M, int N, int K, int epilogue, int* status,
                        cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || epilogue < 0 || epilogue > 2) return MF_ERR_BAD_ARG;
  if (epilogue == 2 && N % 16) return MF_ERR_BAD_ARG;
  if (((uintptr_t)A | (uintptr_t)W) & 15) return MF_ERR_BAD_ARG;
  const bool wide = N > 128;
  switch (epilogue) {
    case 0: return wide ? launch<256, 0>(A, W, C, M, N, K, status, stream) : launch<128, 0>(A, W, C, M, N, K, status, stream);
    case 1: return wide ? launch<256, 1>(A, W, C, M, N, K, status, stream) : launch<128, 1>(A, W, C, M, N, K, status, stream);
    default: return wide ? launch<256, 2>(A, W, C, M, N, K, status, stream) : launch<128, 2>(A, W, C, M, N, K, status, stream);
  }
}
