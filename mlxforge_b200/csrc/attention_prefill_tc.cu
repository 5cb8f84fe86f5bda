// Paged causal attention of prompt portions for head sizes 64 and 128 on the 5th-generation
// tensor cores: both products of a 128-query x 128-key tile (x 64 keys for head size 128) are tcgen05.mma instructions with their
// results in tensor memory, the keys and values come in by TMA, and four warps do nothing
// but the softmax.
//
// A block takes 128 consecutive queries of one head of one sequence and walks the key tiles
// its queries can see, lowest first:
//   warp 4   (producer) one tensor copy per granule of 16 keys (a page holds whole granules):
//            8 key boxes and 8 value boxes per tile, 128-byte swizzled, into a ring of two
//            stages; the queries' own tile once at the start;
//   warp 5   (issuer) one thread: S = Q K^T (M 128, N 128, four steps of K 16 over the head)
//            into tensor memory, then, when the softmax warps have left P in shared memory,
//            O += P V (M 128, N 64, eight steps of 16 keys; V is the N-major operand: its rows
//            are keys, its 128-byte lines run along the head);
//   warps 0-3 a query row per thread (a lane of tensor memory): read the row of S, mask where
//            the tile touches the diagonal or a window's end, running maximum and sum in
//            float32, rescale the row of O in tensor memory when the maximum moved, write the
//            row of P as bfloat16 in the operand layout, at the end divide and store.
// Two blocks share an SM (112 KB of shared memory and 256 columns of tensor memory each), so
// one block's softmax runs under the other's products.  Keys outside every query's range in
// a tile may be stale memory: their scores are masked by selection, and their value rows are
// cleared in shared memory before the second product (0 x NaN would poison it).
//
// Every wait is bounded (codes 41-47 in `status`), and the tensor memory is freed in every
// case.  Formula: src/model/sdpa.cpp:71-95; the reference calls its library's fused kernel.
#include "common.cuh"
#include "tma_host.cuh"

namespace {

// Head size 64: key tiles of 128; head size 128: key tiles of 64.  Either way a stage of keys
// and values is 32 KB, the block's shared memory 112 KB and its tensor memory 256 columns
// (S: BN columns, O: HD columns), so that two blocks share an SM.
constexpr int BM = 128;
constexpr int STAGES = 2;
constexpr int BOX_BYTES = 16 * 64 * 2;             // one tensor copy: 16 keys x 64 values
constexpr int TMEM_COLS = 256;
template <int HD, int BN> struct Shape {
  static constexpr int SPANS = HD / 64;            // 64-wide spans of the head (a swizzled line holds one)
  static constexpr int GRANS = BN / 16;            // granules of 16 keys per tile
  static constexpr int Q_BYTES = BM * HD * 2;
  static constexpr int K_BYTES = BN * HD * 2;
  static constexpr int K_SPAN_BYTES = BN * 128;    // [BN keys][128 bytes] per span
  static constexpr int STAGE_BYTES = 2 * K_BYTES;  // keys then values
  static constexpr int P_BYTES = BM * BN * 2;      // BN / 64 operand tiles of 128 x 64
  static_assert(SPANS * GRANS == 8, "eight key boxes and eight value boxes per stage");
  static_assert(BN + HD <= TMEM_COLS, "S and O share the block's tensor memory");
};
constexpr unsigned WAIT_LIMIT = 1u << 26;
constexpr float LOG2E = 1.4426950408889634f;

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
// Operand tiles in shared memory are lines of 128 bytes with the 128-byte swizzle, eight lines
// (1024 bytes) to a group.  K-major (Q, K, P): a line is 64 values along the contraction.
// N-major (V): a line is 64 values along N, successive lines are successive contraction
// indices.  Either way groups of eight lines are 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr >> 4) & 0x3FFF);          // start address
  d |= (unsigned long long)1 << 16;                          // leading byte offset (one 64-wide span: unused)
  d |= (unsigned long long)(1024 >> 4) << 32;                // stride byte offset: 8 lines x 128 B
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
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&r)[32]) {
  unsigned u[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
        "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]),
        "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]),
        "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; i++) r[i] = __uint_as_float(u[i]);
}
// The same load in two halves, so that a row's next 32 columns are on their way while the
// current 32 are worked on: `issue` starts it, `landed` waits for every load issued so far.
// `landed` names the registers as operands so that no use of them moves above the wait.
__device__ __forceinline__ void tmem_ld32_issue(unsigned taddr, unsigned (&u)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
        "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]),
        "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]),
        "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld32_landed(unsigned (&u)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;\n"
      : "+r"(u[0]), "+r"(u[1]), "+r"(u[2]), "+r"(u[3]), "+r"(u[4]), "+r"(u[5]), "+r"(u[6]), "+r"(u[7]),
        "+r"(u[8]), "+r"(u[9]), "+r"(u[10]), "+r"(u[11]), "+r"(u[12]), "+r"(u[13]), "+r"(u[14]), "+r"(u[15]),
        "+r"(u[16]), "+r"(u[17]), "+r"(u[18]), "+r"(u[19]), "+r"(u[20]), "+r"(u[21]), "+r"(u[22]), "+r"(u[23]),
        "+r"(u[24]), "+r"(u[25]), "+r"(u[26]), "+r"(u[27]), "+r"(u[28]), "+r"(u[29]), "+r"(u[30]), "+r"(u[31])
      :: "memory");
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const float (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      ::"r"(taddr),
        "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])), "r"(__float_as_uint(r[3])),
        "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])), "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])),
        "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])), "r"(__float_as_uint(r[11])),
        "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])), "r"(__float_as_uint(r[14])), "r"(__float_as_uint(r[15])),
        "r"(__float_as_uint(r[16])), "r"(__float_as_uint(r[17])), "r"(__float_as_uint(r[18])), "r"(__float_as_uint(r[19])),
        "r"(__float_as_uint(r[20])), "r"(__float_as_uint(r[21])), "r"(__float_as_uint(r[22])), "r"(__float_as_uint(r[23])),
        "r"(__float_as_uint(r[24])), "r"(__float_as_uint(r[25])), "r"(__float_as_uint(r[26])), "r"(__float_as_uint(r[27])),
        "r"(__float_as_uint(r[28])), "r"(__float_as_uint(r[29])), "r"(__float_as_uint(r[30])), "r"(__float_as_uint(r[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void sts128(unsigned addr, unsigned a, unsigned b, unsigned c, unsigned d) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// The two passes over a thread's row of S, in a form with the mask and one without: the mask
// costs four integer instructions per score and pass, and all but the tiles on the diagonal
// (or at a window's end) need none.  With AHEAD the row's next 32 columns are on their way
// from tensor memory while the current 32 are worked on (the loop is then unrolled, with two
// sets of registers); without it each load is waited for before anything else.
template <bool EDGE, int BN, bool AHEAD>
__device__ __forceinline__ float row_max(unsigned taddr, int key0, int my_pos, int my_lo) {
  float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains instead of one
  unsigned u[AHEAD ? 2 : 1][32];
  if (AHEAD) tmem_ld32_issue(taddr, u[0]);
#pragma unroll(AHEAD ? BN / 32 : 1)
  for (int c = 0; c < BN / 32; c++) {
    unsigned (&cur)[32] = u[AHEAD ? (c & 1) : 0];
    if (!AHEAD) tmem_ld32_issue(taddr + (unsigned)(c * 32), cur);
    tmem_ld32_landed(cur);
    if (AHEAD && c + 1 < BN / 32) tmem_ld32_issue(taddr + (unsigned)((c + 1) * 32), u[AHEAD ? ((c + 1) & 1) : 0]);
#pragma unroll
    for (int j = 0; j < 32; j++) {
      float x = __uint_as_float(cur[j]);
      if (EDGE) {
        const int key = key0 + c * 32 + j;
        if (key > my_pos || key < my_lo) x = -INFINITY;
      }
      mx4[j & 3] = fmaxf(mx4[j & 3], x);
    }
  }
  return fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
}

template <bool EDGE, int BN, bool AHEAD>
__device__ __forceinline__ float row_probabilities(unsigned taddr, unsigned p_row, int r, int key0, int my_pos,
                                                   int my_lo, float scale_log2, float m_off) {
  float sum4[4] = {0.f, 0.f, 0.f, 0.f};
  unsigned u[AHEAD ? 2 : 1][32];
  if (AHEAD) tmem_ld32_issue(taddr, u[0]);
#pragma unroll(AHEAD ? BN / 32 : 1)
  for (int c = 0; c < BN / 32; c++) {
    unsigned (&cur)[32] = u[AHEAD ? (c & 1) : 0];
    if (!AHEAD) tmem_ld32_issue(taddr + (unsigned)(c * 32), cur);
    tmem_ld32_landed(cur);
    if (AHEAD && c + 1 < BN / 32) tmem_ld32_issue(taddr + (unsigned)((c + 1) * 32), u[AHEAD ? ((c + 1) & 1) : 0]);
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) {
      float x = __uint_as_float(cur[j]);
      if (EDGE) {
        const int key = key0 + c * 32 + j;
        if (key > my_pos || key < my_lo) x = -INFINITY;
      }
      const float p = ex2(fmaf(x, scale_log2, -m_off));
      v[j] = p;
      sum4[j & 3] += p;
    }
    // 32 keys = four 16-byte pieces of the row's 128-byte line in half (c >> 1) of P
    const unsigned half_u = p_row + (c >> 1) * (BM * 128);
#pragma unroll
    for (int q4 = 0; q4 < 4; q4++) {
      const int piece = (c & 1) * 4 + q4;
      sts128(half_u + ((piece ^ (r & 7)) << 4), pack_bf16(v[q4 * 8 + 0], v[q4 * 8 + 1]),
             pack_bf16(v[q4 * 8 + 2], v[q4 * 8 + 3]), pack_bf16(v[q4 * 8 + 4], v[q4 * 8 + 5]),
             pack_bf16(v[q4 * 8 + 6], v[q4 * 8 + 7]));
    }
  }
  return (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
}

int g_prefill_tc = 1;       // 0: the mma.sync kernel for every shape (mf_set_prefill_tcgen05)

template <int HD, int BN, bool AHEAD>
__global__ void __launch_bounds__(192, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                       const int* __restrict__ seq_ctx_len, int table_row0, PagedView pv, int n_heads,
                       float scale_log2, int window, int* __restrict__ status) {
  using SH = Shape<HD, BN>;
  constexpr int Q_BYTES = SH::Q_BYTES, K_BYTES = SH::K_BYTES, STAGE_BYTES = SH::STAGE_BYTES, P_BYTES = SH::P_BYTES;
  constexpr int SPANS = SH::SPANS, GRANS = SH::GRANS, K_SPAN_BYTES = SH::K_SPAN_BYTES;
  extern __shared__ __align__(1024) unsigned char smem[];      // the swizzled tiles need 1024-byte alignment
  const unsigned q_u = smem_u32(smem), kv_u = q_u + Q_BYTES, p_u = kv_u + STAGES * STAGE_BYTES;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + Q_BYTES + STAGES * STAGE_BYTES + P_BYTES);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 16);
  const unsigned bars_u = smem_u32(bars);
  const unsigned q_full = bars_u, kv_full0 = bars_u + 8, kv_empty0 = bars_u + 24, s_full = bars_u + 40,
                 p_full = bars_u + 48, o_done = bars_u + 56;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the heaviest tiles (the last queries of a portion see the most keys) are launched first, for
  // all heads before any lighter tile
  const int tile = (int)gridDim.y - 1 - (int)blockIdx.y, head = blockIdx.x, s = blockIdx.z;
  const int q_len = seq_q_len[s];
  if (tile * BM >= q_len) return;
  if (q_u & 1023u) {                                       // never seen; refused rather than computed wrongly
    if (threadIdx.x == 0 && status) atomicExch(status, 40);
    return;
  }
  const int q_start = seq_q_start[s], ctx = seq_ctx_len[s];
  const int seq_row = table_row0 + s;
  const int p0 = ctx - q_len;                              // position of the portion's first token
  const int kvh = head / (n_heads / pv.n_kv_heads);
  const int rows = min(BM, q_len - tile * BM);             // valid queries in this tile
  const int pos_first = p0 + tile * BM, pos_last = pos_first + rows - 1;
  const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
  const int kt0 = lo_first / BN, kt1 = pos_last / BN;      // key tiles [kt0, kt1]
  const int n_kt = kt1 - kt0 + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int st = 0; st < STAGES; st++) {
      mbar_init(kv_full0 + 8 * st, 1);
      mbar_init(kv_empty0 + 8 * st, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);                 // one arrive per softmax warp
    mbar_init(o_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  const unsigned tmem_s = tmem_base, tmem_o = tmem_base + BN;     // S: columns [0, BN), O: [BN, BN + HD)

  if (warp == 4) {
    // ------------------------------------------------------------ producer
    if (lane == 0) mbar_expect_tx(q_full, Q_BYTES);      // rows past the end of q arrive as zeros
    __syncwarp();
    if (lane < SPANS) tma_load_2d(q_u + lane * (BM * 128), &map_q, head * HD + lane * 64, q_start + tile * BM, q_full);
    for (int i = 0; i < n_kt; i++) {
      const int kt = kt0 + i;
      const unsigned st = i % STAGES, round = i / STAGES;
      // lanes 0..7: the key boxes (granule x span of the head); lanes 8..15: the value boxes.
      // A granule with no visible key is not fetched.
      const int gran = lane & (GRANS - 1), span = (lane & 7) / GRANS;
      const int key16 = kt * BN + gran * 16;
      const bool valid = lane < 16 && key16 <= pos_last && key16 + 16 > lo_first;
      int box_row = 0;
      if (valid) {
        const int blk = key16 / pv.page_size;
        const int page = pv.block_table[(long long)seq_row * pv.bt_stride + blk];
        box_row = (page * pv.n_kv_heads + kvh) * pv.page_size + (key16 - blk * pv.page_size);
      }
      const unsigned n_valid = __popc(__ballot_sync(0xffffffffu, valid));
      if (lane == 0) {
        if (round > 0) mbar_wait(kv_empty0 + 8 * st, (round - 1) & 1, status, 41);
        mbar_expect_tx(kv_full0 + 8 * st, n_valid * BOX_BYTES);
      }
      __syncwarp();
      if (valid)
        tma_load_2d(kv_u + st * STAGE_BYTES + (lane >> 3) * K_BYTES + span * K_SPAN_BYTES + gran * BOX_BYTES,
                    lane < 8 ? &map_k : &map_v, span * 64, box_row, kv_full0 + 8 * st);
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ issuer
    if (lane == 0) {
      // instruction descriptors: D float32, A and B bfloat16; N >> 3 at bit 17, M >> 4 at bit 24;
      // bit 16: B is N-major (the values)
      const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
      const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(64 >> 3) << 17) |
                                ((unsigned)(BM >> 4) << 24);
      mbar_wait(q_full, 0, status, 42);
      for (int i = 0; i < n_kt; i++) {
        const unsigned st = i % STAGES, round = i / STAGES;
        mbar_wait(kv_full0 + 8 * st, round & 1, status, 43);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned k_addr = kv_u + st * STAGE_BYTES, v_addr = k_addr + K_BYTES;
        // S = Q K^T: steps of 16 along the head, span after span
#pragma unroll
        for (int k = 0; k < HD / 16; k++)
          umma(tmem_s, smem_desc(q_u + (k >> 2) * (BM * 128) + (k & 3) * 32),
               smem_desc(k_addr + (k >> 2) * K_SPAN_BYTES + (k & 3) * 32), idesc_qk, k > 0 ? 1u : 0u);
        umma_commit(s_full);
        mbar_wait(p_full, i & 1, status, 44);           // P is in shared memory, S has been read
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        // O += P V: steps of 16 keys; a product of N = 64 for each span of the head
#pragma unroll
        for (int k = 0; k < BN / 16; k++)
#pragma unroll
          for (int sp = 0; sp < SPANS; sp++)
            umma(tmem_o + (unsigned)(sp * 64), smem_desc(p_u + (k >> 2) * (BM * 128) + (k & 3) * 32),
                 smem_desc(v_addr + sp * K_SPAN_BYTES + k * 16 * 128), idesc_pv, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(kv_empty0 + 8 * st);                 // the stage is free once both products have read it
        umma_commit(o_done);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax: a query row per thread
    const int r = warp * 32 + lane;
    const unsigned lane_field = (unsigned)(warp * 32) << 16;
    const int my_pos = pos_first + r;
    const int my_lo = (window > 0 && my_pos - window + 1 > 0) ? my_pos - window + 1 : 0;
    const int w_pos_first = pos_first + warp * 32;          // this warp's first query
    const int w_lo_last = (window > 0 && w_pos_first + 31 - window + 1 > 0) ? w_pos_first + 31 - window + 1 : 0;
    float m_row = -INFINITY, l_row = 0.f;
    for (int i = 0; i < n_kt; i++) {
      const int kt = kt0 + i, key0 = kt * BN;
      const unsigned st = i % STAGES;
      mbar_wait(s_full, i & 1, status, 45);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      // mask only where the tile touches this warp's diagonal or an end of its windows
      const bool edge = key0 + BN - 1 > w_pos_first || key0 < w_lo_last;
      // ---- first pass over the row of S: its maximum
      float mx = edge ? row_max<true, BN, AHEAD>(tmem_s + lane_field, key0, my_pos, my_lo)
                      : row_max<false, BN, AHEAD>(tmem_s + lane_field, key0, my_pos, my_lo);
      mx *= scale_log2;                                      // scale > 0: the max commutes with it
      const float m_new = fmaxf(m_row, mx);
      const float m_off = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m_row == -INFINITY) ? 0.f : ex2(m_row - m_off);
      // ---- the product before this one has read P and left O: rescale O if a maximum moved
      if (i > 0) {
        mbar_wait(o_done, (i - 1) & 1, status, 46);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (__any_sync(0xffffffffu, m_new != m_row)) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; c++) {
            float v[32];
            tmem_ld32(tmem_o + lane_field + (unsigned)(c * 32), v);
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] *= alpha;
            tmem_st32(tmem_o + lane_field + (unsigned)(c * 32), v);
          }
        }
      }
      // ---- value rows of keys that no query of the tile may see: clear them (thread = key)
      if (key0 + BN - 1 > pos_last || key0 < lo_first) {
        const int key = key0 + r;
        if (r < BN && (key > pos_last || key < lo_first)) {
#pragma unroll
          for (int sp = 0; sp < SPANS; sp++) {
            const unsigned row_u = kv_u + st * STAGE_BYTES + K_BYTES + sp * K_SPAN_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < 8; c++) sts128(row_u + c * 16, 0u, 0u, 0u, 0u);
          }
        }
      }
      // ---- second pass: probabilities, their sum, and the row of P in the operand layout
      const unsigned p_row = p_u + (r >> 3) * 1024 + (r & 7) * 128;
      const float sum =
          edge ? row_probabilities<true, BN, AHEAD>(tmem_s + lane_field, p_row, r, key0, my_pos, my_lo, scale_log2, m_off)
               : row_probabilities<false, BN, AHEAD>(tmem_s + lane_field, p_row, r, key0, my_pos, my_lo, scale_log2, m_off);
      l_row = l_row * alpha + sum;
      m_row = m_new;
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");     // P and the cleared rows, before the product reads them
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- normalise and store (rows of the portion only)
    mbar_wait(o_done, (n_kt - 1) & 1, status, 47);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const float inv = 1.0f / l_row;
    __nv_bfloat16* orow = out + ((long long)(q_start + tile * BM + r) * n_heads + head) * HD;
#pragma unroll 1
    for (int c = 0; c < HD / 32; c++) {
      float v[32];
      tmem_ld32(tmem_o + lane_field + (unsigned)(c * 32), v);
      if (r < rows) {
#pragma unroll
        for (int q4 = 0; q4 < 4; q4++) {
          uint4 pk;
          pk.x = pack_bf16(v[q4 * 8 + 0] * inv, v[q4 * 8 + 1] * inv);
          pk.y = pack_bf16(v[q4 * 8 + 2] * inv, v[q4 * 8 + 3] * inv);
          pk.z = pack_bf16(v[q4 * 8 + 4] * inv, v[q4 * 8 + 5] * inv);
          pk.w = pack_bf16(v[q4 * 8 + 6] * inv, v[q4 * 8 + 7] * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = pk;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

template <int HD, int BN>
int launch_tc(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool, __nv_bfloat16* out,
              const int* seq_q_start, const int* seq_q_len, const int* seq_ctx_len, int table_row0, int n_seqs,
              int max_q_len, int n_tokens, int n_heads, PagedView pv, float scale, int window, int* status,
              cudaStream_t stream) {
  using SH = Shape<HD, BN>;
  CUtensorMap mq, mk, mv;
  int rc = tma_host::bf16_map(q, n_tokens, (long long)n_heads * HD, BM, 64, &mq);
  if (rc) return rc;
  // the maps' row count only bounds the unit's own range check; rows beyond the pool are never asked for
  rc = tma_host::bf16_map(k_pool, 1ll << 28, HD, 16, 64, &mk);
  if (rc) return rc;
  rc = tma_host::bf16_map(v_pool, 1ll << 28, HD, 16, 64, &mv);
  if (rc) return rc;
  const size_t smem = SH::Q_BYTES + STAGES * SH::STAGE_BYTES + SH::P_BYTES + 16 * 8 + 16;
  // Head size 128 (key tiles of 64: two loads per pass) gains 4 to 6 % from loads that run ahead;
  // head size 64 (four loads per pass, 168 registers) loses 15 % on a prompt of 2048 and gains 4 % on
  // one of 8192, so it keeps the serial passes.
  constexpr bool AHEAD = HD == 128;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, BN, AHEAD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(n_heads, (max_q_len + BM - 1) / BM, n_seqs);
  attn_prefill_tc_kernel<HD, BN, AHEAD><<<grid, 192, smem, stream>>>(mq, mk, mv, out, seq_q_start, seq_q_len, seq_ctx_len,
                                                                    table_row0, pv, n_heads, scale * LOG2E, window, status);
  return (int)cudaGetLastError();
}

}  // namespace

// 1 (the default): portions of at least 128 tokens with head size 64 or 128 take the tcgen05
// kernel; 0: every shape takes the mma.sync kernel.  For tests and measurements.
MF_API int mf_set_prefill_tcgen05(int on) {
  g_prefill_tc = on ? 1 : 0;
  return 0;
}

// Arguments as launch_prefill of attention_prefill.cu plus the number of rows of q.  Returns
// MF_ERR_BAD_ARG when this kernel does not take the shape (the caller then uses the other one).
int launch_prefill_tc(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool,
                      __nv_bfloat16* out, const int* seq_q_start, const int* seq_q_len, const int* seq_ctx_len,
                      int table_row0, int n_seqs, int max_q_len, int n_tokens, int n_heads, PagedView pv,
                      float scale, int window, int* status, cudaStream_t stream) {
  if (!g_prefill_tc || pv.page_size % 16 || max_q_len < BM || n_tokens <= 0) return MF_ERR_BAD_ARG;
  if ((((uintptr_t)q | (uintptr_t)out) & 15) != 0) return MF_ERR_BAD_ARG;
  if (pv.head_dim == 64)
    return launch_tc<64, 128>(q, k_pool, v_pool, out, seq_q_start, seq_q_len, seq_ctx_len, table_row0, n_seqs,
                              max_q_len, n_tokens, n_heads, pv, scale, window, status, stream);
  if (pv.head_dim == 128)
    return launch_tc<128, 64>(q, k_pool, v_pool, out, seq_q_start, seq_q_len, seq_ctx_len, table_row0, n_seqs,
                              max_q_len, n_tokens, n_heads, pv, scale, window, status, stream);
  return MF_ERR_BAD_ARG;
}
