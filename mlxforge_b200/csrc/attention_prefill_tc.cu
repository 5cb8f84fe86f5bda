// Paged causal attention of prompt portions for head sizes 64 and 128 on the 5th-generation
// tensor cores: both products of a tile of 128 queries x 64 keys are tcgen05.mma instructions
// with their results in tensor memory, the keys and values come in by TMA, and four warps do
// nothing but the softmax.
//
// A block takes 128 consecutive queries of one head of one sequence and walks the tiles of 64
// keys its queries can see, lowest first:
//   warp 4   (producer) one tensor copy per granule of 16 keys (a page holds whole granules)
//            and 64-wide span of the head, 128-byte swizzled, into a ring of stages; the
//            queries' own tile once at the start;
//   warp 5   (issuer) one thread: S = Q K^T (M 128, N 64, steps of K 16 over the head) into
//            tensor memory, then, when the softmax warps have left P in shared memory,
//            O += P V (M 128, N 64 per span of the head, four steps of 16 keys; V is the
//            N-major operand: its rows are keys, its 128-byte lines run along the head);
//   warps 0-3 a query row per thread (a lane of tensor memory): read the row of S once into
//            registers, mask it where the tile touches the diagonal or a window's end, running
//            maximum and sum in float32, rescale the row of O in tensor memory when the
//            exponent's reference moves (rarely: see MAX_SLACK_LOG2), write the row of P as
//            bfloat16 in the operand layout, at the end divide and store.
// Two blocks share an SM (112 KB of shared memory and 256 columns of tensor memory each).
// Head size 128 has one S per block, so one block's softmax runs under the other block's
// products; head size 64 has room for two S per block and issues its products two tiles
// ahead of the softmax (the second kernel below).  Keys outside every query's range in a tile
// may be stale memory: their scores are masked by selection, and their value rows are cleared
// in shared memory before the second product (0 x NaN would poison it).
//
// Every wait is bounded (codes 41-47 in `status`), and the tensor memory is freed in every
// case.  Formula: src/model/sdpa.cpp:71-95; the reference calls its library's fused kernel.
#include "common.cuh"
#include "tma_host.cuh"

namespace {

// The kernel with one S (head size 128): key tiles of 64, a stage of keys and values is 32 KB,
// the block's shared memory 112 KB and its tensor memory 256 columns (S: BN columns, O: HD
// columns), so that two blocks share an SM.
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
  static_assert(BN == 64, "a row of S is read into registers as two loads of 32 columns");
  static_assert(BN + HD <= TMEM_COLS, "S and O share the block's tensor memory");
};
constexpr unsigned WAIT_LIMIT = 1u << 26;
constexpr float LOG2E = 1.4426950408889634f;
// The exponent's reference for a row is its running maximum, but it need not be THE maximum:
// any reference cancels in O / l.  A warp moves its rows' references (and rescales its rows of
// O in tensor memory, a load, 64 multiplications and a store per row) only when some row's
// maximum has grown by more than 2^8 since the last move; until then probabilities may reach
// 256, which float32 sums and bfloat16's eight exponent bits hold as well as values below one.
constexpr float MAX_SLACK_LOG2 = 8.0f;

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

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// A thread's row of S for 64 keys: read from tensor memory ONCE into `u` (both loads on their
// way before the first is waited for), masked in place where the tile touches the diagonal or a
// window's end (all other tiles take the form without the mask: four integer instructions per
// score less), and its maximum returned.  The second pass works on the registers.
template <bool EDGE>
__device__ __forceinline__ float row_scores_max(unsigned taddr, unsigned (&u)[2][32], int key0, int my_pos, int my_lo) {
  tmem_ld32_issue(taddr, u[0]);
  tmem_ld32_issue(taddr + 32u, u[1]);
  float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains instead of one
#pragma unroll
  for (int c = 0; c < 2; c++) {
    tmem_ld32_landed(u[c]);                      // waits for both; the second call finds them there
    if (EDGE) {
#pragma unroll
      for (int j = 0; j < 32; j++) {
        const int key = key0 + c * 32 + j;
        if (key > my_pos || key < my_lo) u[c][j] = __float_as_uint(-INFINITY);
      }
    }
#pragma unroll
    for (int j = 0; j < 32; j += 2)
      mx4[(j >> 1) & 3] = fmax3(mx4[(j >> 1) & 3], __uint_as_float(u[c][j]), __uint_as_float(u[c][j + 1]));
  }
  return fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
}

// Second pass: probabilities (in place), their sum, and the row of P as bfloat16 in the operand
// layout: 64 keys = the eight 16-byte pieces of the row's 128-byte line.
__device__ __forceinline__ float row_probabilities(unsigned (&u)[2][32], unsigned p_row, int r, float scale_log2,
                                                   float m_off) {
  float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c = 0; c < 2; c++) {
    float (&v)[32] = reinterpret_cast<float (&)[32]>(u[c]);
#pragma unroll
    for (int j = 0; j < 32; j++) {
      const float p = ex2(fmaf(v[j], scale_log2, -m_off));
      v[j] = p;
      sum4[j & 3] += p;
    }
#pragma unroll
    for (int q4 = 0; q4 < 4; q4++) {
      const int piece = c * 4 + q4;
      sts128(p_row + ((piece ^ (r & 7)) << 4), pack_bf16(v[q4 * 8 + 0], v[q4 * 8 + 1]),
             pack_bf16(v[q4 * 8 + 2], v[q4 * 8 + 3]), pack_bf16(v[q4 * 8 + 4], v[q4 * 8 + 5]),
             pack_bf16(v[q4 * 8 + 6], v[q4 * 8 + 7]));
    }
  }
  return (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
}

int g_prefill_tc = 1;       // 0: the mma.sync kernel for every shape (mf_set_prefill_tcgen05)

template <int HD, int BN>
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
      unsigned sc[2][32];
      float mx = edge ? row_scores_max<true>(tmem_s + lane_field, sc, key0, my_pos, my_lo)
                      : row_scores_max<false>(tmem_s + lane_field, sc, key0, my_pos, my_lo);
      mx *= scale_log2;                                      // scale > 0: the max commutes with it
      const float m_cand = fmaxf(m_row, mx);
      const bool moved = __any_sync(0xffffffffu, m_cand - m_row > MAX_SLACK_LOG2);      // also from -inf
      const float m_new = moved ? m_cand : m_row;
      const float m_off = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = !moved ? 1.f : ((m_row == -INFINITY) ? 0.f : ex2(m_row - m_off));
      // ---- the product before this one has read P and left O: rescale O if a maximum moved
      if (i > 0) {
        mbar_wait(o_done, (i - 1) & 1, status, 46);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (moved) {
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
      const float sum = row_probabilities(sc, p_row, r, scale_log2, m_off);
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

// ---------------------------------------------------------------------------------------------
// Head size 64 with the products running AHEAD of the softmax.  The kernel above has one S in
// tensor memory, so within a block S = Q K^T, the softmax and O += P V take turns and only the
// SM's other block fills the gaps.  Here a block works on sub-tiles of 64 keys and has two
// S buffers (tensor memory: S0 64 columns, S1 64, O 64): while the softmax warps work on
// sub-tile j, S of sub-tile j + 1 is already there and that of j + 2 is issued as soon as P of
// j has been handed over, right behind O += P_j V_j.  The softmax warps never wait for a
// product in the steady state.  Keys and values come in stages of 64 keys (8 KB each, four
// tensor copies of 16 keys) through a ring of five, so that the keys two sub-tiles ahead are
// there when their product is issued.  P stays single: a softmax pass writes it only after
// it has waited for the previous O += P V (which it needs anyway before it rescales O).
namespace ahead {
constexpr int HD = 64, SUB = 64, RING = 5;
constexpr int Q_BYTES = BM * HD * 2, K_BYTES = SUB * HD * 2, STAGE_BYTES = 2 * K_BYTES, P_BYTES = BM * SUB * 2;
constexpr size_t SMEM = Q_BYTES + RING * STAGE_BYTES + P_BYTES + 16 * 8 + 16;
}  // namespace ahead

__global__ void __launch_bounds__(192, 2)
attn_prefill_tc_ahead_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                             const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                             const int* __restrict__ seq_ctx_len, int table_row0, PagedView pv, int n_heads,
                             float scale_log2, int window, int* __restrict__ status) {
  using namespace ahead;
  extern __shared__ __align__(1024) unsigned char smem[];
  const unsigned q_u = smem_u32(smem), kv_u = q_u + Q_BYTES, p_u = kv_u + RING * STAGE_BYTES;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + Q_BYTES + RING * STAGE_BYTES + P_BYTES);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 16);
  const unsigned bars_u = smem_u32(bars);
  const unsigned q_full = bars_u, kv_full0 = bars_u + 8, kv_empty0 = kv_full0 + 8 * RING, s_full0 = kv_empty0 + 8 * RING,
                 p_full = s_full0 + 16, o_done = p_full + 8;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = (int)gridDim.y - 1 - (int)blockIdx.y, head = blockIdx.x, s = blockIdx.z;
  const int q_len = seq_q_len[s];
  if (tile * BM >= q_len) return;
  if (q_u & 1023u) {
    if (threadIdx.x == 0 && status) atomicExch(status, 40);
    return;
  }
  const int q_start = seq_q_start[s], ctx = seq_ctx_len[s];
  const int seq_row = table_row0 + s;
  const int p0 = ctx - q_len;
  const int kvh = head / (n_heads / pv.n_kv_heads);
  const int rows = min(BM, q_len - tile * BM);
  const int pos_first = p0 + tile * BM, pos_last = pos_first + rows - 1;
  const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
  const int sub0 = lo_first / SUB, n_sub = pos_last / SUB - sub0 + 1;        // sub-tiles of 64 keys

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int st = 0; st < RING; st++) {
      mbar_init(kv_full0 + 8 * st, 1);
      mbar_init(kv_empty0 + 8 * st, 1);
    }
    mbar_init(s_full0, 1);
    mbar_init(s_full0 + 8, 1);
    mbar_init(p_full, 4);
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
  const unsigned tmem_s = tmem_base, tmem_o = tmem_base + 2 * SUB;      // S0, S1: 64 columns each; then O

  if (warp == 4) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
      tma_load_2d(q_u, &map_q, head * HD, q_start + tile * BM, q_full);
    }
    for (int j = 0; j < n_sub; j++) {
      const unsigned st = j % RING, round = j / RING;
      // lanes 0..3: the key boxes of the sub-tile's four granules; lanes 4..7: the value boxes
      const int key16 = (sub0 + j) * SUB + (lane & 3) * 16;
      const bool valid = lane < 8 && key16 <= pos_last && key16 + 16 > lo_first;
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
        tma_load_2d(kv_u + st * STAGE_BYTES + (lane >> 2) * K_BYTES + (lane & 3) * BOX_BYTES, lane < 4 ? &map_k : &map_v,
                    0, box_row, kv_full0 + 8 * st);
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ issuer
    if (lane == 0) {
      const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(SUB >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
      const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) |
                                ((unsigned)(BM >> 4) << 24);
      auto scores = [&](int j) {                   // S[j & 1] = Q K_j^T
        const unsigned st = j % RING;
        mbar_wait(kv_full0 + 8 * st, (j / RING) & 1, status, 43);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned k_addr = kv_u + st * STAGE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; k++)
          umma(tmem_s + (unsigned)((j & 1) * SUB), smem_desc(q_u + k * 32), smem_desc(k_addr + k * 32), idesc_qk,
               k > 0 ? 1u : 0u);
        umma_commit(s_full0 + 8 * (j & 1));
      };
      mbar_wait(q_full, 0, status, 42);
      scores(0);
      if (n_sub > 1) scores(1);
      for (int j = 0; j < n_sub; j++) {
        const unsigned st = j % RING;
        mbar_wait(p_full, j & 1, status, 44);          // P_j is in shared memory, S[j & 1] has been read
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned v_addr = kv_u + st * STAGE_BYTES + K_BYTES;
#pragma unroll
        for (int k = 0; k < SUB / 16; k++)
          umma(tmem_o, smem_desc(p_u + k * 32), smem_desc(v_addr + k * 16 * 128), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(kv_empty0 + 8 * st);               // both products of this stage are behind this
        umma_commit(o_done);
        if (j + 2 < n_sub) scores(j + 2);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax: a query row per thread
    const int r = warp * 32 + lane;
    const unsigned lane_field = (unsigned)(warp * 32) << 16;
    const int my_pos = pos_first + r;
    const int my_lo = (window > 0 && my_pos - window + 1 > 0) ? my_pos - window + 1 : 0;
    const int w_pos_first = pos_first + warp * 32;
    const int w_lo_last = (window > 0 && w_pos_first + 31 - window + 1 > 0) ? w_pos_first + 31 - window + 1 : 0;
    const unsigned p_row = p_u + (r >> 3) * 1024 + (r & 7) * 128;
    float m_row = -INFINITY, l_row = 0.f;
    for (int j = 0; j < n_sub; j++) {
      const int key0 = (sub0 + j) * SUB;
      const unsigned st = j % RING;
      const unsigned s_addr = tmem_s + lane_field + (unsigned)((j & 1) * SUB);
      mbar_wait(s_full0 + 8 * (j & 1), (j >> 1) & 1, status, 45);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const bool edge = key0 + SUB - 1 > w_pos_first || key0 < w_lo_last;
      unsigned sc[2][32];
      float mx = edge ? row_scores_max<true>(s_addr, sc, key0, my_pos, my_lo)
                      : row_scores_max<false>(s_addr, sc, key0, my_pos, my_lo);
      mx *= scale_log2;
      const float m_cand = fmaxf(m_row, mx);
      const bool moved = __any_sync(0xffffffffu, m_cand - m_row > MAX_SLACK_LOG2);      // also from -inf
      const float m_new = moved ? m_cand : m_row;
      const float m_off = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = !moved ? 1.f : ((m_row == -INFINITY) ? 0.f : ex2(m_row - m_off));
      if (j > 0) {                                   // O += P V of the sub-tile before: P is free, O is whole
        mbar_wait(o_done, (j - 1) & 1, status, 46);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (moved) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; c++) {
            float v[32];
            tmem_ld32(tmem_o + lane_field + (unsigned)(c * 32), v);
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] *= alpha;
            tmem_st32(tmem_o + lane_field + (unsigned)(c * 32), v);
          }
        }
      }
      if (key0 + SUB - 1 > pos_last || key0 < lo_first) {      // value rows of keys no query may see (thread = key)
        const int key = key0 + r;
        if (r < SUB && (key > pos_last || key < lo_first)) {
          const unsigned row_u = kv_u + st * STAGE_BYTES + K_BYTES + r * 128;
#pragma unroll
          for (int c = 0; c < 8; c++) sts128(row_u + c * 16, 0u, 0u, 0u, 0u);
        }
      }
      const float sum = row_probabilities(sc, p_row, r, scale_log2, m_off);
      l_row = l_row * alpha + sum;
      m_row = m_new;
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    mbar_wait(o_done, (n_sub - 1) & 1, status, 47);
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

int launch_tc_ahead(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool, __nv_bfloat16* out,
                    const int* seq_q_start, const int* seq_q_len, const int* seq_ctx_len, int table_row0, int n_seqs,
                    int max_q_len, int n_tokens, int n_heads, PagedView pv, float scale, int window, int* status,
                    cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  int rc = tma_host::bf16_map(q, n_tokens, (long long)n_heads * ahead::HD, BM, 64, &mq);
  if (rc) return rc;
  rc = tma_host::bf16_map(k_pool, 1ll << 28, ahead::HD, 16, 64, &mk);
  if (rc) return rc;
  rc = tma_host::bf16_map(v_pool, 1ll << 28, ahead::HD, 16, 64, &mv);
  if (rc) return rc;
  static DeviceOnce once;
  const int dev_ = mf_current_device();
  if (dev_ < 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev_]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_ahead_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)ahead::SMEM);
    if (e != cudaSuccess) return (int)e;
    once.done[dev_] = true;
  }
  dim3 grid(n_heads, (max_q_len + BM - 1) / BM, n_seqs);
  mf_count(MF_K_ATTN_PREFILL_TC);
  attn_prefill_tc_ahead_kernel<<<grid, 192, ahead::SMEM, stream>>>(mq, mk, mv, out, seq_q_start, seq_q_len, seq_ctx_len,
                                                                   table_row0, pv, n_heads, scale * LOG2E, window, status);
  return (int)cudaGetLastError();
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
  static DeviceOnce once;
  const int dev_ = mf_current_device();
  if (dev_ < 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev_]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    once.done[dev_] = true;
  }
  dim3 grid(n_heads, (max_q_len + BM - 1) / BM, n_seqs);
  mf_count(MF_K_ATTN_PREFILL_TC);
  attn_prefill_tc_kernel<HD, BN><<<grid, 192, smem, stream>>>(mq, mk, mv, out, seq_q_start, seq_q_len, seq_ctx_len,
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
    return launch_tc_ahead(q, k_pool, v_pool, out, seq_q_start, seq_q_len, seq_ctx_len, table_row0, n_seqs, max_q_len,
                           n_tokens, n_heads, pv, scale, window, status, stream);
  if (pv.head_dim == 128)
    return launch_tc<128, 64>(q, k_pool, v_pool, out, seq_q_start, seq_q_len, seq_ctx_len, table_row0, n_seqs,
                              max_q_len, n_tokens, n_heads, pv, scale, window, status, stream);
  return MF_ERR_BAD_ARG;
}
