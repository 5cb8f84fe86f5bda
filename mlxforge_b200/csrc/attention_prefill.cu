// Causal GQA attention of prompt portions (two or more new tokens per sequence)
// over the paged bfloat16 cache: one block per (128 or 64 queries, query head, sequence),
// key tiles of 64 double-buffered through shared memory with cp.async, both
// products on the tensor cores (mma.sync m16n8k16, bf16 in, fp32 out), online
// softmax in fp32.  The new tokens' own keys are already in the cache (the rotary
// kernel wrote them), so a portion attends to everything before it and to itself
// through the same pages.
//
// Formula: src/model/sdpa.cpp:71-95, src/model/decoder_model.cpp:260-275 of
// hvasconcelos/mlxforge: scores * scale, causal mask aligned to the end of the keys
// (query j of a portion sits at absolute position ctx - q_len + j), softmax over
// keys, p * v; query head h reads KV head h / (n_heads / n_kv_heads).
//
// Key tiles start at multiples of 64 of the absolute position, so the order of
// every sum depends only on the query's position, not on where a prompt was cut.
#include "common.cuh"

namespace {

constexpr int BN = 64;      // keys per tile
constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
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

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// MT: 16-row query tiles per warp (2 for head sizes up to 128: the fragments of a key tile are
// then read from shared memory once for 32 queries; 1 above, where registers run out).
template <int HD_MAX> struct Shape { static constexpr int MT = 1; };

template <int HD_MAX>
__global__ void __launch_bounds__(WARPS * 32)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                    const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out,
                    const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                    const int* __restrict__ seq_ctx_len, int table_row0, PagedView pv, int n_heads,
                    float scale_log2, int window) {
  constexpr int DT = HD_MAX / 8;
  constexpr int MT = Shape<HD_MAX>::MT;
  constexpr int BM = WARPS * 16 * MT;                          // queries per block
  const int hd = pv.head_dim, ld = hd + 8, chunks = hd >> 3;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [BM][ld]
  __nv_bfloat16* kv_s = q_s + BM * ld;                                    // [2 stages][K, V][BN][ld]

  // the heaviest tiles (the last queries of a portion see the most keys) are launched first, for
  // all heads before any lighter tile
  const int tile = (int)gridDim.y - 1 - (int)blockIdx.y, head = blockIdx.x, s = blockIdx.z;
  const int q_len = seq_q_len[s];
  if (tile * BM >= q_len) return;
  const int q_start = seq_q_start[s], ctx = seq_ctx_len[s];
  const int seq_row = table_row0 + s;
  const int p0 = ctx - q_len;                              // position of the portion's first token
  const int kvh = head / (n_heads / pv.n_kv_heads);
  const int rows = min(BM, q_len - tile * BM);             // valid queries in this tile
  const int pos_first = p0 + tile * BM, pos_last = pos_first + rows - 1;
  const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
  const int kt0 = lo_first / BN, kt1 = pos_last / BN;      // key tiles [kt0, kt1]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;

  auto load_kv = [&](int kt, int stage) {
    __nv_bfloat16* k_s = kv_s + (stage * 2 + 0) * BN * ld;
    __nv_bfloat16* v_s = kv_s + (stage * 2 + 1) * BN * ld;
    // one block-table lookup per granule of 16 keys (lanes 0..3 of every warp), then shared
    long long gran_off = 0;
    {
      const int key16 = kt * BN + lane * 16;
      if (lane < BN / 16 && key16 <= pos_last && key16 + 16 > lo_first) gran_off = granule_offset(pv, seq_row, key16, kvh);
    }
    for (int i = threadIdx.x; i < BN * chunks; i += WARPS * 32) {
      const int r = i / chunks, c = i - r * chunks;
      const int key = kt * BN + r;
      const bool valid = key >= lo_first && key <= pos_last;
      const long long off = __shfl_sync(0xffffffffu, gran_off, r >> 4) + (r & 15) * hd + c * 8;
      cp_async_16(k_s + r * ld + c * 8, k_pool + (valid ? off : 0), valid);
      cp_async_16(v_s + r * ld + c * 8, v_pool + (valid ? off : 0), valid);
    }
  };

  // ---- queries of this tile (rows beyond the portion are zero), first key tile
  for (int i = threadIdx.x; i < BM * chunks; i += WARPS * 32) {
    const int r = i / chunks, c = i - r * chunks;
    const int rr = min(r, rows - 1);
    cp_async_16(q_s + r * ld + c * 8, q + ((long long)(q_start + tile * BM + rr) * n_heads + head) * hd + c * 8,
                r < rows);
  }
  load_kv(kt0, 0);
  cp_async_commit();

  // this warp's queries: MT tiles of 16 rows; thread rows g and g + 8 of each
  const int wrow0 = warp * 16 * MT;
  float m_row[MT][2], l_row[MT][2];
  float o[MT][DT][4];
  int my_pos[MT][2], my_lo[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; mt++) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
      m_row[mt][h] = -INFINITY;
      l_row[mt][h] = 0.f;
      my_pos[mt][h] = pos_first + wrow0 + mt * 16 + g + h * 8;
      my_lo[mt][h] = (window > 0 && my_pos[mt][h] - window + 1 > 0) ? my_pos[mt][h] - window + 1 : 0;
    }
#pragma unroll
    for (int d = 0; d < DT; d++) o[mt][d][0] = o[mt][d][1] = o[mt][d][2] = o[mt][d][3] = 0.f;
  }
  const int w_pos_first = pos_first + wrow0, w_pos_last = w_pos_first + 16 * MT - 1;
  const int w_lo_last = (window > 0 && w_pos_last - window + 1 > 0) ? w_pos_last - window + 1 : 0;

  for (int kt = kt0; kt <= kt1; kt++) {
    const int stage = (kt - kt0) & 1;
    if (kt < kt1) load_kv(kt + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();           // everything but the tile just requested has landed
    __syncthreads();
    const __nv_bfloat16* k_s = kv_s + (stage * 2 + 0) * BN * ld;
    const __nv_bfloat16* v_s = kv_s + (stage * 2 + 1) * BN * ld;

    // a warp whose queries all lie before this key tile has nothing to do in it
    const bool active = kt * BN <= w_pos_last;
    if (active) {
      float sc[MT][BN / 8][4];
#pragma unroll
      for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int j = 0; j < BN / 8; j++) sc[mt][j][0] = sc[mt][j][1] = sc[mt][j][2] = sc[mt][j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD_MAX / 16; kk++) {
        if (kk * 16 < hd) {
          unsigned a[MT][4];
#pragma unroll
          for (int mt = 0; mt < MT; mt++)
            ldmatrix_x4(a[mt], q_s + (wrow0 + mt * 16 + (lane & 15)) * ld + kk * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int j = 0; j < BN / 8; j += 2) {
            unsigned b[4];
            const int mi = lane >> 3, r = lane & 7;
            ldmatrix_x4(b, k_s + (j * 8 + (mi >> 1) * 8 + r) * ld + kk * 16 + (mi & 1) * 8);
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
              mma_bf16(sc[mt][j], a[mt], b[0], b[1]);
              mma_bf16(sc[mt][j + 1], a[mt], b[2], b[3]);
            }
          }
        }
      }
      // ---- mask only where the tile touches the diagonal or an end of a window; online softmax
      const bool edge = kt * BN + BN - 1 > w_pos_first || kt * BN < w_lo_last;
      if (edge) {            // a loop of its own under one branch: tiles off the diagonal pay nothing for the mask
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
          for (int j = 0; j < BN / 8; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const int key = kt * BN + j * 8 + tq * 2 + (e & 1);
              if (key > my_pos[mt][e >> 1] || key < my_lo[mt][e >> 1]) sc[mt][j][e] = -INFINITY;
            }
      }
#pragma unroll
      for (int mt = 0; mt < MT; mt++) {
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < BN / 8; j++) {
#pragma unroll
          for (int e = 0; e < 4; e++) mx[e >> 1] = fmaxf(mx[e >> 1], sc[mt][j][e]);
        }
        float alpha[2], m_off[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
          mx[h] *= scale_log2;                                        // scale > 0: the max commutes with it
          const float m_new = fmaxf(m_row[mt][h], mx[h]);
          m_off[h] = (m_new == -INFINITY) ? 0.f : m_new;
          alpha[h] = (m_row[mt][h] == -INFINITY) ? 0.f : ex2(m_row[mt][h] - m_off[h]);
          m_row[mt][h] = m_new;
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < BN / 8; j++) {
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const float p = ex2(fmaf(sc[mt][j][e], scale_log2, -m_off[e >> 1]));   // one multiply-add, one ex2
            sc[mt][j][e] = p;
            sum[e >> 1] += p;
          }
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
          sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
          sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
          l_row[mt][h] = l_row[mt][h] * alpha[h] + sum[h];
        }
#pragma unroll
        for (int d = 0; d < DT; d++) {
          o[mt][d][0] *= alpha[0]; o[mt][d][1] *= alpha[0];
          o[mt][d][2] *= alpha[1]; o[mt][d][3] *= alpha[1];
        }
      }
      // ---- O += P V
#pragma unroll
      for (int kk = 0; kk < BN / 16; kk++) {
        unsigned a[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
          a[mt][0] = pack_bf16(sc[mt][2 * kk][0], sc[mt][2 * kk][1]);
          a[mt][1] = pack_bf16(sc[mt][2 * kk][2], sc[mt][2 * kk][3]);
          a[mt][2] = pack_bf16(sc[mt][2 * kk + 1][0], sc[mt][2 * kk + 1][1]);
          a[mt][3] = pack_bf16(sc[mt][2 * kk + 1][2], sc[mt][2 * kk + 1][3]);
        }
#pragma unroll
        for (int d = 0; d < DT; d += 2) {
          if (d * 8 < hd) {
            unsigned b[4];
            const int mi = lane >> 3, r = lane & 7;
            ldmatrix_x4_trans(b, v_s + (kk * 16 + (mi & 1) * 8 + r) * ld + d * 8 + (mi >> 1) * 8);
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
              mma_bf16(o[mt][d], a[mt], b[0], b[1]);
              mma_bf16(o[mt][d + 1], a[mt], b[2], b[3]);
            }
          }
        }
      }
    }
    __syncthreads();      // this stage is free for the tile after next
  }
  cp_async_wait<0>();

  // ---- normalise and store (rows of the portion only)
#pragma unroll
  for (int mt = 0; mt < MT; mt++) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int r = wrow0 + mt * 16 + g + h * 8;
      if (r >= rows) continue;
      const float inv = 1.0f / l_row[mt][h];
      __nv_bfloat16* orow = out + ((long long)(q_start + tile * BM + r) * n_heads + head) * hd;
#pragma unroll
      for (int d = 0; d < DT; d++) {
        if (d * 8 < hd) {
          *reinterpret_cast<unsigned*>(orow + d * 8 + tq * 2) =
              pack_bf16(o[mt][d][h * 2] * inv, o[mt][d][h * 2 + 1] * inv);
        }
      }
    }
  }
}

template <int HD_MAX>
int launch_prefill(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool,
                   __nv_bfloat16* out, const int* seq_q_start, const int* seq_q_len, const int* seq_ctx_len,
                   int table_row0, int n_seqs, int max_q_len, int n_heads, PagedView pv, float scale, int window,
                   cudaStream_t stream) {
  constexpr int BM = WARPS * 16 * Shape<HD_MAX>::MT;
  const int ld = pv.head_dim + 8;
  const size_t smem = (size_t)(BM * ld + 4 * BN * ld) * sizeof(__nv_bfloat16);
  static DeviceOnce once;
  const int dev_ = mf_current_device();
  if (dev_ < 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev_]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_prefill_kernel<HD_MAX>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return (int)e;
    once.done[dev_] = true;
  }
  dim3 grid(n_heads, (max_q_len + BM - 1) / BM, n_seqs);
  mf_count(MF_K_ATTN_PREFILL_MMA);
  attn_prefill_kernel<HD_MAX><<<grid, WARPS * 32, smem, stream>>>(q, k_pool, v_pool, out, seq_q_start, seq_q_len,
                                                                 seq_ctx_len, table_row0, pv, n_heads,
                                                                 scale * LOG2E, window);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_prefill_tc(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool,
                      __nv_bfloat16* out, const int* seq_q_start, const int* seq_q_len, const int* seq_ctx_len,
                      int table_row0, int n_seqs, int max_q_len, int n_tokens, int n_heads, PagedView pv,
                      float scale, int window, int* status, cudaStream_t stream);

// q, out: [T, n_heads * hd] of the whole step.  The n_seqs sequences start at row
// `table_row0` of the block table; seq_q_start / seq_q_len / seq_ctx_len are their
// first token's index in q, their number of new tokens and their length after the
// step.  `max_q_len` bounds seq_q_len (it sizes the grid); `n_tokens` is T.  `status`: a device int
// (may be null) for the bounded waits of the tcgen05 kernel (attention_prefill_tc.cu), which
// takes head size 64 when a portion has at least 128 tokens.
MF_API int mf_attention_prefill(const void* q, const void* k_pool, const void* v_pool, void* out,
                                const int* seq_q_start, const int* seq_q_len, const int* seq_ctx_len,
                                int table_row0, int n_seqs, int max_q_len, int n_tokens, int n_heads, int n_kv,
                                int hd, const int* block_table, int bt_stride, int page_size, float scale,
                                int window, int* status, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  if (hd < 16 || hd > 256 || hd % 16 || n_kv <= 0 || n_heads % n_kv) return MF_ERR_BAD_ARG;
  if (n_heads > 65535 || n_seqs > 65535) return MF_ERR_BAD_ARG;
  PagedView pv{block_table, bt_stride, page_size, n_kv, hd};
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)k_pool,
                      *vv = (const __nv_bfloat16*)v_pool;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
  {
    const int rc = launch_prefill_tc(qq, kk, vv, oo, seq_q_start, seq_q_len, seq_ctx_len, table_row0, n_seqs,
                                     max_q_len, n_tokens, n_heads, pv, scale, window, status, stream);
    if (rc != MF_ERR_BAD_ARG) return rc;
  }
  if (hd <= 64)
    return launch_prefill<64>(qq, kk, vv, oo, seq_q_start, seq_q_len, seq_ctx_len, table_row0, n_seqs, max_q_len,
                              n_heads, pv, scale, window, stream);
  if (hd <= 128)
    return launch_prefill<128>(qq, kk, vv, oo, seq_q_start, seq_q_len, seq_ctx_len, table_row0, n_seqs, max_q_len,
                               n_heads, pv, scale, window, stream);
  return launch_prefill<256>(qq, kk, vv, oo, seq_q_start, seq_q_len, seq_ctx_len, table_row0, n_seqs, max_q_len,
                             n_heads, pv, scale, window, stream);
}
