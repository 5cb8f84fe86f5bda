// Decode attention for head sizes 64 and 128 with the keys and values brought in by the TMA unit.
//
// It computes exactly what attn_decode_kernel (attention_decode.cu) computes and writes the
// same per-split partial results, but is built around the memory system instead of around the
// warps, and it merges its splits itself: the block that finishes the last split of a (token,
// head group) adds the splits' results in their order and writes the output (see g_tickets).
// Launches with more groups than there are tickets leave the merge to attn_decode_merge_kernel.
//   * persistent blocks (two per SM for head size 64, one for 128: a stage of 128 keys and values
//     is 32 or 64 KB) walk work items (token, KV head x head group, split of 512 keys or more),
//     item = block, block + grid, ...;
//   * a producer warp issues 2-D tensor copies per granule of 16 keys (a page holds whole
//     granules, so a granule is 16 contiguous rows of the pool; a box is 16 rows of 64 columns,
//     one 128-byte swizzle span, so head size 128 takes two boxes per granule): 8 key granules and
//     8 value granules per stage of 128 keys into a ring of STAGES stages, each signalled by
//     an mbarrier; it runs ahead across item boundaries, so the ring(s) of an SM keep about
//     130-190 KB on their way, and no thread computes an address per 16 bytes;
//   * eight consumer warps take 16 keys of a stage each (scores and the second product on
//     mma.sync as in the other kernel, softmax statistics in fp32, running over the item's
//     stages), hand the stage back, and at the end of an item combine into one partial result.
// Query rows of an item are one contiguous run of G * head_dim values: one bulk copy.
//
// All waits are bounded (see gemv_stream.cu).  Formula: src/model/sdpa.cpp:71-95.
#include "common.cuh"
#include "tma_host.cuh"

namespace {

constexpr int CW = 8;                   // consumer warps
constexpr int TILE = 128;               // keys per stage: 8 granules of 16
constexpr int BOX_BYTES = 16 * 64 * 2;  // 2 KB: 16 rows of one 128-byte span
constexpr int MIN_SPLIT_KEYS = 512, MAX_SPLIT_KEYS = 2048;   // keys per work item: chosen per launch
constexpr float LOG2E = 1.4426950408889634f;
constexpr unsigned WAIT_LIMIT = 1u << 24;

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
__device__ __forceinline__ void bulk_copy(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
// Before a thread copies into a buffer that the consumers have read: their reads are generic-proxy
// accesses, the copy an async-proxy write, and the mbarrier alone does not order the one before the
// other (see gemv_stream.cu, where it was measured).  Every lane that issues a copy fences after the
// wait for the buffer (lane 0's, passed on by __syncwarp) and before its copy.
__device__ __forceinline__ void stage_is_mine() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CW * 32) : "memory"); }

// One counter per (token, group of heads): every split of that group that saw keys takes a
// ticket when its partial result is written; the block that draws the last one merges the
// splits into the output, in the order of the splits, and puts the counter back to zero.
// Nobody waits for another block.  Launches with more groups than this merge in a kernel of
// their own (attn_decode_merge_kernel).  The counters belong to the device, not to a launch:
// launches of this kernel on one device must follow one another (one stream, as the engine
// has it), not run side by side.
constexpr int MAX_TICKETS = 1 << 16;
__device__ int g_tickets[MAX_TICKETS];

// What an item is, computed the same way by the producer and the consumers.
struct Item {
  int t, kvh, head0, n_rows, split, pos, lo, seq, tile0, tile1;
  bool live;
};
__device__ __forceinline__ Item make_item(int item, int max_splits, int groups, int hgroups, int G,
                                          const int* positions, const int* seq_of_token, int window,
                                          int SPLIT_KEYS) {
  Item it;
  it.split = item % max_splits;
  const int rest = item / max_splits;
  const int grp = rest % groups;
  it.t = rest / groups;
  it.kvh = grp / hgroups;
  const int hg = grp - it.kvh * hgroups;
  it.head0 = it.kvh * G + hg * 16;
  it.n_rows = min(16, G - hg * 16);
  it.pos = positions[it.t];
  it.seq = seq_of_token[it.t];
  it.lo = (window > 0 && it.pos - window + 1 > 0) ? it.pos - window + 1 : 0;
  const int k_begin = it.split * SPLIT_KEYS;
  it.live = !(k_begin > it.pos || k_begin + SPLIT_KEYS <= it.lo);
  it.tile0 = max(k_begin, it.lo) / TILE;
  it.tile1 = min(k_begin + SPLIT_KEYS - 1, it.pos) / TILE;
  return it;
}

template <int HD, int STAGES>
__global__ void __launch_bounds__((CW + 1) * 32)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const __nv_bfloat16* __restrict__ q, float* __restrict__ part_o, float* __restrict__ part_ml,
                       __nv_bfloat16* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ seq_of_token, PagedView pv,
                       int n_heads, int n_tokens, float scale_log2, int window, int max_splits, int comb_rows,
                       int split_keys, int* __restrict__ status) {
  constexpr int HALVES = HD / 64;                   // spans of 64 columns per row of the cache
  constexpr int GRAN_BYTES = HALVES * BOX_BYTES;    // a granule: [span][16 rows][128 bytes]
  constexpr int STAGE_BYTES = 2 * 8 * GRAN_BYTES;   // 8 key granules, then 8 value granules
  constexpr int Q_BYTES = 16 * HD * 2;
  extern __shared__ unsigned char raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  unsigned char* ring = smem;                                             // [STAGES][K 8 granules | V 8 granules]
  unsigned char* q_s = smem + STAGES * STAGE_BYTES;                       // [2][16][HD] bf16
  float* comb = reinterpret_cast<float*>(q_s + 2 * Q_BYTES);              // [CW][comb_rows][HD + 2]: m, l, o[HD]
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(comb + CW * comb_rows * (HD + 2));
  int* last_flag = reinterpret_cast<int*>(bars + 2 * STAGES + 4);
  const int CR = comb_rows;              // rows of the combine buffer per warp: the heads of a group
  const unsigned ring_u = smem_u32(ring), q_u = smem_u32(q_s), bars_u = smem_u32(bars);
  const unsigned full0 = bars_u, empty0 = bars_u + 8 * STAGES;
  const unsigned qfull0 = bars_u + 16 * STAGES, qempty0 = qfull0 + 16;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = n_heads / pv.n_kv_heads, hgroups = (G + 15) / 16, groups = pv.n_kv_heads * hgroups;
  const int n_items = n_tokens * groups * max_splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, CW);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(qfull0 + 8 * b, 1);
      mbar_init(qempty0 + 8 * b, CW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // rows of q beyond the group stay zero for the whole kernel
  for (int i = threadIdx.x; i < 2 * Q_BYTES / 16; i += blockDim.x) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");    // before the copy unit writes there
  __syncthreads();
  // q and each token's newest key and value come from the kernel before this one; everything
  // older in the cache does not, so the producer starts filling its ring before it waits
  if (warp != CW) {
    pdl_wait();
    if (threadIdx.x == 0) pdl_launch();
  }

  if (warp == CW) {
    // ------------------------------------------------------------ producer warp
    // What the copies of an item need from memory (the token's position and sequence, and the
    // page of each of the split's 32 granules: lane l looks up granule l) is fetched one item
    // ahead, so that the ring never waits for a table lookup.
    // a split has up to MAX_SPLIT_KEYS / 16 = 128 granules: four per lane
    auto fetch = [&](int item, Item& w, int (&row)[4]) {
      w = make_item(item, max_splits, groups, hgroups, G, positions, seq_of_token, window, split_keys);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int key16 = w.split * split_keys + (j * 32 + lane) * 16;
        row[j] = -1;
        if (w.live && (j * 32 + lane) * 16 < split_keys && key16 <= w.pos && key16 + 16 > w.lo) {
          const int blk = key16 / pv.page_size;
          const int page = pv.block_table[(long long)w.seq * pv.bt_stride + blk];
          row[j] = (page * pv.n_kv_heads + w.kvh) * pv.page_size + (key16 - blk * pv.page_size);
        }
      }
    };
    unsigned it = 0, live_items = 0;
    bool waited = false;
    int item = blockIdx.x;
    Item w, w_next;
    int row[4] = {-1, -1, -1, -1}, row_next[4] = {-1, -1, -1, -1};
    w_next.live = false;
    if (item < n_items) fetch(item, w, row);
    while (item < n_items) {
      const int next = item + gridDim.x;
      if (next < n_items) fetch(next, w_next, row_next);
      if (w.live) {
        // the item's queries: G contiguous rows (only after the wait: the kernel before wrote them)
        const unsigned qb = live_items & 1, quse = live_items >> 1;
        auto issue_q = [&]() {
          if (lane == 0) {
            if (quse > 0) {
              mbar_wait(qempty0 + 8 * qb, (quse - 1) & 1, status, 21);
              stage_is_mine();
            }
            mbar_expect_tx(qfull0 + 8 * qb, (unsigned)w.n_rows * HD * 2);
            bulk_copy(q_u + qb * Q_BYTES, q + ((long long)w.t * n_heads + w.head0) * HD,
                      (unsigned)w.n_rows * HD * 2, qfull0 + 8 * qb);
          }
        };
        bool q_done = false;
        live_items++;
        for (int tile = w.tile0; tile <= w.tile1; tile++, it++) {
          const unsigned s = it % STAGES, round = it / STAGES;
          // Before the wait only tiles of older keys may be fetched, and only while the ring has
          // room (the consumers cannot free a stage before they have their queries).
          if (!waited && ((tile + 1) * TILE > w.pos || round > 0)) {
            pdl_wait();
            waited = true;
          }
          if (waited && !q_done) {
            issue_q();
            q_done = true;
          }
          // lanes 0 .. 8 HALVES - 1: the key boxes (span lane / 8 of granule lane % 8); the next
          // 8 HALVES lanes: the value boxes
          const int gran = lane & 7, half = (lane >> 3) % HALVES, is_v = lane / (8 * HALVES);
          const int gi = (tile * TILE - w.split * split_keys) / 16 + gran;           // granule of the split
          const int j = gi >> 5;                                                       // the same for the tile's 8
          const int mine = j == 0 ? row[0] : (j == 1 ? row[1] : (j == 2 ? row[2] : row[3]));
          const int box_row = __shfl_sync(0xffffffffu, mine, gi & 31);                 // from who looked it up
          const bool valid = lane < 16 * HALVES && box_row >= 0;
          const unsigned n_valid = __popc(__ballot_sync(0xffffffffu, valid));
          if (lane == 0) {
            if (round > 0) mbar_wait(empty0 + 8 * s, (round - 1) & 1, status, 22);
            mbar_expect_tx(full0 + 8 * s, n_valid * BOX_BYTES);
          }
          __syncwarp();
          stage_is_mine();
          if (valid) {
            const unsigned dst = ring_u + s * STAGE_BYTES + is_v * 8 * GRAN_BYTES + gran * GRAN_BYTES + half * BOX_BYTES;
            tma_load_2d(dst, is_v ? &map_v : &map_k, half * 64, box_row, full0 + 8 * s);
          }
        }
        if (!q_done) {
          if (!waited) {
            pdl_wait();
            waited = true;
          }
          issue_q();
        }
      }
      w = w_next;
#pragma unroll
      for (int j = 0; j < 4; j++) row[j] = row_next[j];
      item = next;
    }
    if (!waited) pdl_wait();
    return;
  }

  // -------------------------------------------------------------- consumers
  const int g = lane >> 2, tq = lane & 3;
  // one split per group (every context of the launch fits into one): an item's result is the
  // output, so it is stored at once and neither partial results nor tickets are needed
  const bool direct = max_splits == 1 && out != nullptr;
  unsigned it = 0, live_items = 0;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const Item w = make_item(item, max_splits, groups, hgroups, G, positions, seq_of_token, window, split_keys);
    if (!w.live) continue;
    // ---- the query tile as A fragments (read once per item)
    unsigned qa[HD / 16][4];
    {
      const unsigned b = live_items & 1, use = live_items >> 1;
      mbar_wait(qfull0 + 8 * b, use & 1, status, 23);
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++)
        ldmatrix_x4(qa[kk], q_u + b * Q_BYTES + (lane & 15) * (HD * 2) + (kk * 16 + (lane >> 4) * 8) * 2);
      __syncwarp();
      if (lane == 0) mbar_arrive(qempty0 + 8 * b);
    }
    live_items++;
    float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; d++) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    for (int tile = w.tile0; tile <= w.tile1; tile++, it++) {
      const unsigned s = it % STAGES, round = it / STAGES;
      mbar_wait(full0 + 8 * s, round & 1, status, 24);
      const int w_begin = tile * TILE + warp * 16;                 // this warp's granule
      if (w_begin <= w.pos && w_begin + 16 > w.lo) {
        const unsigned k_box = ring_u + s * STAGE_BYTES + warp * GRAN_BYTES;
        const unsigned v_box = k_box + 8 * GRAN_BYTES;
        // ---- scores S[16 heads x 16 keys]; rows of a box are 128 bytes, 16-byte pieces swizzled by row & 7
        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; j++) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
        const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) {
          unsigned b[4];
          const int key = (mi >> 1) * 8 + r8, piece = (kk & 3) * 2 + (mi & 1);
          ldmatrix_x4(b, k_box + (kk >> 2) * BOX_BYTES + key * 128 + ((piece ^ (key & 7)) << 4));
          mma_bf16(sc[0], qa[kk], b[0], b[1]);
          mma_bf16(sc[1], qa[kk], b[2], b[3]);
        }
        const bool edge = w_begin < w.lo || w_begin + 15 > w.pos;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; j++) {
#pragma unroll
          for (int e = 0; e < 4; e++) {
            float v = sc[j][e] * scale_log2;
            if (edge) {
              const int key = w_begin + j * 8 + tq * 2 + (e & 1);
              if (key < w.lo || key > w.pos) v = -INFINITY;
            }
            sc[j][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
          }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
          const float m_new = fmaxf(m_row[h], mx[h]);
          m_use[h] = (m_new == -INFINITY) ? 0.f : m_new;
          alpha[h] = (m_row[h] == -INFINITY) ? 0.f : exp2f(m_row[h] - m_use[h]);
          m_row[h] = m_new;
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 2; j++) {
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const float p = exp2f(sc[j][e] - m_use[e >> 1]);
            sc[j][e] = p;
            sum[e >> 1] += p;
          }
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
          sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
          sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
          l_row[h] = l_row[h] * alpha[h] + sum[h];
        }
#pragma unroll
        for (int d = 0; d < HD / 8; d++) {
          o[d][0] *= alpha[0]; o[d][1] *= alpha[0];
          o[d][2] *= alpha[1]; o[d][3] *= alpha[1];
        }
        if (edge) {
          // rows of the box beyond the visible range hold whatever the page held before: their
          // probability is exactly 0, but 0 x NaN would still poison the product, so clear them
          for (int r = 0; r < 16; r++) {
            const int key = w_begin + r;
            if ((key < w.lo || key > w.pos) && lane < 8 * HALVES)
              asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n"
                           ::"r"(v_box + (lane >> 3) * BOX_BYTES + r * 128 + (lane & 7) * 16), "r"(0u) : "memory");
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
          __syncwarp();
        }
        // ---- O[16 x 64] += P V
        unsigned a[4];
        a[0] = pack_bf16(sc[0][0], sc[0][1]);
        a[1] = pack_bf16(sc[0][2], sc[0][3]);
        a[2] = pack_bf16(sc[1][0], sc[1][1]);
        a[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
        for (int d = 0; d < HD / 8; d += 2) {
          unsigned b[4];
          const int key = (mi & 1) * 8 + r8, piece = (d & 7) + (mi >> 1);
          ldmatrix_x4_trans(b, v_box + (d >> 3) * BOX_BYTES + key * 128 + ((piece ^ (key & 7)) << 4));
          mma_bf16(o[d], a, b[0], b[1]);
          mma_bf16(o[d + 1], a, b[2], b[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }

    // ---- combine the 8 warps into the item's partial result (rows of the group only)
    constexpr int CS = HD + 2;
    if (tq == 0) {
      if (g < w.n_rows) { comb[(warp * CR + g) * CS] = m_row[0]; comb[(warp * CR + g) * CS + 1] = l_row[0]; }
      if (g + 8 < w.n_rows) { comb[(warp * CR + g + 8) * CS] = m_row[1]; comb[(warp * CR + g + 8) * CS + 1] = l_row[1]; }
    }
#pragma unroll
    for (int d = 0; d < HD / 8; d++) {
      if (g < w.n_rows) *reinterpret_cast<float2*>(comb + (warp * CR + g) * CS + 2 + d * 8 + tq * 2) = make_float2(o[d][0], o[d][1]);
      if (g + 8 < w.n_rows)
        *reinterpret_cast<float2*>(comb + (warp * CR + g + 8) * CS + 2 + d * 8 + tq * 2) = make_float2(o[d][2], o[d][3]);
    }
    consumer_sync();
    for (int i = threadIdx.x; i < w.n_rows * HD; i += CW * 32) {
      const int r = i / HD, d = i - r * HD;
      float M = -INFINITY;
#pragma unroll
      for (int cw = 0; cw < CW; cw++) M = fmaxf(M, comb[(cw * CR + r) * CS]);
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int cw = 0; cw < CW; cw++) {
        const float mw = comb[(cw * CR + r) * CS];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        L += comb[(cw * CR + r) * CS + 1] * f;
        acc += comb[(cw * CR + r) * CS + 2 + d] * f;
      }
      if (direct) {
        // the only split of its group: what a merge of one split would compute, acc * 2^0 / (L * 2^0)
        out[((long long)w.t * n_heads + w.head0 + r) * HD + d] = __float2bfloat16_rn(acc / L);
        continue;
      }
      const long long row = ((long long)w.t * n_heads + w.head0 + r) * max_splits + w.split;
      part_o[row * HD + d] = acc;
      if (d == 0) {
        part_ml[row * 2 + 0] = M;
        part_ml[row * 2 + 1] = L;
      }
    }
    if (out == nullptr || direct) {
      consumer_sync();     // `comb` is free for the next item
      continue;
    }
    // ---- the ticket; whoever draws the group's last one merges its splits (out != nullptr)
    __threadfence();       // this thread's part of the partial result, before the ticket
    consumer_sync();       // also: `comb` is free for the next item
    const int s0 = w.lo / split_keys, n_live = w.pos / split_keys - s0 + 1;
    if (threadIdx.x == 0) {
      const int slot = item / max_splits;
      const int last = atomicAdd(g_tickets + slot, 1) == n_live - 1;
      if (last) g_tickets[slot] = 0;
      *last_flag = last;
    }
    consumer_sync();
    const bool last = *last_flag != 0;
    consumer_sync();       // everyone has read the flag before the next item writes it
    if (last) {
      __threadfence();
      for (int i = threadIdx.x; i < w.n_rows * HD; i += CW * 32) {
        const int r = i / HD, d = i - r * HD;
        const long long row = ((long long)w.t * n_heads + w.head0 + r) * max_splits + s0;
        // eight splits' statistics and values are fetched at once (their addresses do not depend on
        // one another: one round trip through L2 instead of one per split), then added in order
        float M = -INFINITY, L = 0.f, acc = 0.f;
        for (int s8 = 0; s8 < n_live; s8 += 8) {
          float pm[8], pl[8], po[8];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const bool in = s8 + j < n_live;
            pm[j] = in ? __ldcg(part_ml + (row + s8 + j) * 2) : -INFINITY;
            pl[j] = in ? __ldcg(part_ml + (row + s8 + j) * 2 + 1) : 0.f;
            po[j] = in ? __ldcg(part_o + (row + s8 + j) * HD + d) : 0.f;
          }
          float M8 = M;
#pragma unroll
          for (int j = 0; j < 8; j++) M8 = fmaxf(M8, pm[j]);
          const float keep = (M == -INFINITY) ? 0.f : exp2f(M - M8);     // what was summed so far, on the new scale
          L *= keep;
          acc *= keep;
          M = M8;
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const float f = (pm[j] == -INFINITY) ? 0.f : exp2f(pm[j] - M);
            L += pl[j] * f;
            acc += po[j] * f;
          }
        }
        out[((long long)w.t * n_heads + w.head0 + r) * HD + d] = __float2bfloat16_rn(acc / L);
      }
    }
  }
}

}  // namespace

int g_merge_inside = 1;

namespace {

template <int HD, int STAGES, int BLOCKS_PER_SM>
int launch_for(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool, __nv_bfloat16* out,
               float* part_o, float* part_ml, int n_tokens, int n_heads, PagedView pv, long long pool_rows,
               const int* positions, const int* seq_of_token, float scale, int window, int max_ctx, int unequal,
               int* status, int* split_out, int* merged_out, cudaStream_t stream) {
  constexpr int STAGE_BYTES = 2 * 8 * (HD / 64) * BOX_BYTES, Q_BYTES = 16 * HD * 2;
  CUtensorMap mk, mv;
  int rc = tma_host::bf16_map(k_pool, pool_rows, HD, 16, 64, &mk);
  if (rc) return rc;
  rc = tma_host::bf16_map(v_pool, pool_rows, HD, 16, 64, &mv);
  if (rc) return rc;
  const int G0 = n_heads / pv.n_kv_heads;
  const int comb_rows = G0 < 16 ? G0 : 16;
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 2 * Q_BYTES + (size_t)CW * comb_rows * (HD + 2) * 4 + (2 * STAGES + 4) * 8 + 8 + 1024;
  if (smem > 227 * 1024) return MF_ERR_BAD_ARG;       // the caller takes another kernel
  static DeviceOnce once;
  const int dev_ = mf_current_device();
  const int n_sms = mf_sm_count();
  if (dev_ < 0 || n_sms <= 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev_]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<HD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
    once.done[dev_] = true;
  }
  const int slots = BLOCKS_PER_SM * n_sms;
  // Longer splits cost less per key (an item ends with a combine of the eight warps), shorter
  // ones give more items: take the longest split that still gives most blocks an item.
  const int G = n_heads / pv.n_kv_heads, hgroups = (G + 15) / 16;
  int split_keys = MAX_SPLIT_KEYS;
  long long n_items = 0;
  for (;; split_keys /= 2) {
    n_items = (long long)n_tokens * pv.n_kv_heads * hgroups * ((max_ctx + split_keys - 1) / split_keys);
    if (split_keys == MIN_SPLIT_KEYS || n_items * 20 >= (long long)slots * 17) break;
  }
  *split_out = split_keys;
  const int max_splits = (max_ctx + split_keys - 1) / split_keys;
  if (n_items > 0x7fffffff) return MF_ERR_BAD_ARG;
  // One block per SM has nobody beside it to stream while it combines, writes and hands in an item's
  // result, and items are dealt out in turn, not by size: with many items of unequal contexts to a
  // block (64 requests of 128 to 4352 tokens: a serving run's decode steps took 11.7 ms instead of
  // 6.6) the kernel without tensor copies, whose many small blocks the hardware deals out, is the
  // faster one.  Up to two items a block this one is (62 against 68 us at 8 x 8192, 15 against 21 us
  // at 1 x 8192 on the 3B shape).
  if (BLOCKS_PER_SM == 1 && n_items > 2ll * slots) return MF_ERR_BAD_ARG;
  // The same with two blocks per SM once the caller says that the contexts are of very unequal
  // length (64 requests of 128 to 4352 tokens on the 1B shape: a serving run took 1.46 s with this
  // kernel and 1.12 to 1.31 s with the other; with equal contexts this one wins at every batch size).
  if (unequal && n_items > 2ll * slots) return MF_ERR_BAD_ARG;
  const int grid = n_items < slots ? (int)n_items : slots;
  // the merge inside this kernel, where the tickets reach (g_merge_inside: for measurements)
  // Every item pays for its ticket (a fence and two barriers of the consumer warps), the merge kernel
  // costs one launch: with more than two items to a block the kernel of its own is the cheaper way
  // (batch 64 at context 8192, seven items a block: 3.96 ms a step inside, 3.77 ms with the kernel).
  const bool inside = g_merge_inside && (long long)n_tokens * pv.n_kv_heads * hgroups <= MAX_TICKETS &&
                      n_items <= 2ll * grid;
  *merged_out = inside ? 1 : 0;
  return (int)launch_dep(attn_decode_tma_kernel<HD, STAGES>, dim3(grid), dim3((CW + 1) * 32), smem, stream, mk, mv, q, part_o,
                         part_ml, inside ? out : (__nv_bfloat16*)nullptr, positions, seq_of_token, pv, n_heads, n_tokens, scale * LOG2E, window, max_splits,
                         comb_rows, split_keys, status);
}

}  // namespace

// Launches the first kernel of the decode attention for head sizes 64 and 128 (the merge kernel of
// attention_decode.cu follows it unless *merged_out says that it merged its splits itself).
// Returns MF_ERR_BAD_ARG when this path does not apply.
int launch_decode_tma(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool,
                      __nv_bfloat16* out, float* part_o, float* part_ml, int n_tokens, int n_heads, PagedView pv,
                      long long pool_rows, const int* positions, const int* seq_of_token, float scale, int window,
                      int max_ctx, int unequal, int* status, int* split_out, int* merged_out, cudaStream_t stream) {
  if (pv.page_size % 16) return MF_ERR_BAD_ARG;
  if (pv.head_dim == 64)
    return launch_for<64, 3, 2>(q, k_pool, v_pool, out, part_o, part_ml, n_tokens, n_heads, pv, pool_rows, positions,
                                seq_of_token, scale, window, max_ctx, unequal, status, split_out, merged_out, stream);
  if (pv.head_dim == 128) {
    // one block per SM with three stages of 64 KB; groups of many heads need a combine buffer that
    // leaves room for two stages only
    const int rc = launch_for<128, 3, 1>(q, k_pool, v_pool, out, part_o, part_ml, n_tokens, n_heads, pv, pool_rows,
                                         positions, seq_of_token, scale, window, max_ctx, unequal, status, split_out, merged_out, stream);
    if (rc != MF_ERR_BAD_ARG) return rc;
    return launch_for<128, 2, 1>(q, k_pool, v_pool, out, part_o, part_ml, n_tokens, n_heads, pv, pool_rows, positions,
                                 seq_of_token, scale, window, max_ctx, unequal, status, split_out, merged_out, stream);
  }
  return MF_ERR_BAD_ARG;
}

// After a kernel of this file gave up a bounded wait its tickets may be left counting: the next
// launch's merges would then fire at the wrong split or never.  This puts every ticket back to
// zero (on `stream`, ordered like any launch).
MF_API int mf_reset_decode_tickets(cudaStream_t stream) {
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_tickets);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemsetAsync(p, 0, sizeof(int) * MAX_TICKETS, stream);
}
