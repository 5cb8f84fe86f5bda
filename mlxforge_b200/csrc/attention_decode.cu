// Attention of single new tokens (decoding) over the paged bfloat16 cache, split
// over the keys so that a few sequences fill the machine.
//
// Kernel 1, one block per (split of the keys, KV head x group of <= 16 query heads,
// token): the query heads that share a KV head are the 16 rows of one tensor-core
// tile, so each key and value is read from memory once for all of them (the
// reference's fused kernel does GQA natively too, src/model/decoder_model.cpp:268;
// its unfused path shows the grouping, src/model/sdpa.cpp:27).  Each of the 4 warps
// takes KEYS_PER_WARP keys: scores by mma.sync (bf16 in, fp32 out), softmax
// statistics in fp32, probabilities rounded to bf16 for the second product.  The
// block writes an unnormalised partial result (max, sum, output) per query head.
// Kernel 2 merges the partials of a token's splits.
//
// The split size is fixed (it depends on the head size only), so a token's result
// does not depend on what else is in the batch.  Formula: src/model/sdpa.cpp:71-95.
#include "common.cuh"

namespace {

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
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

// Keys per warp and tile by head size: a tile is WARPS * KPW keys, staged twice (double
// buffer) as [WARPS][K, V][KPW][hd + 8] bfloat16.  A block walks SPLIT_KEYS keys.
template <int HD_MAX> struct Tile {
  static constexpr int KPW = HD_MAX <= 64 ? 32 : 16;
  static constexpr int W = 4;                        // warps per block
};
constexpr int SPLIT_KEYS = 512;
constexpr int NSTAGE = 2;               // tiles in flight per warp: NSTAGE - 1 while one is multiplied

template <int HD_MAX>
__global__ void __launch_bounds__(Tile<HD_MAX>::W * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                   const __nv_bfloat16* __restrict__ v_pool, float* __restrict__ part_o,
                   float* __restrict__ part_ml, const int* __restrict__ positions,
                   const int* __restrict__ seq_of_token, PagedView pv, int n_heads, float scale_log2,
                   int window, int max_splits) {
  constexpr int KPW = Tile<HD_MAX>::KPW;
  constexpr int WARPS = Tile<HD_MAX>::W;
  constexpr int TILE = KPW * WARPS;
  constexpr int NT = KPW / 8;           // score n-tiles per warp and tile
  constexpr int DT = HD_MAX / 8;        // output n-tiles (channels / 8)
  constexpr int KS = HD_MAX / 16;       // k-steps of the score product
  const int hd = pv.head_dim;
  const int ld = hd + 8;                // padded row: conflict-free ldmatrix for every hd % 16 == 0
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [16][ld]
  __nv_bfloat16* kv_s = q_s + 16 * ld;                                              // [NSTAGE][WARPS][2][KPW][ld]

  pdl_wait();
  pdl_launch();
  const int split = blockIdx.x, t = blockIdx.z;
  const int G = n_heads / pv.n_kv_heads;
  const int hgroups = (G + 15) / 16;
  const int kvh = blockIdx.y / hgroups, hg = blockIdx.y - kvh * hgroups;
  const int head0 = kvh * G + hg * 16;
  const int n_rows = min(16, G - hg * 16);
  const int pos = positions[t], seq = seq_of_token[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int k_begin = split * SPLIT_KEYS;
  if (k_begin > pos || k_begin + SPLIT_KEYS <= lo) return;       // nothing visible in this split
  // tiles of this split that hold visible keys
  const int tile0 = max(k_begin, lo) / TILE, tile1 = min(k_begin + SPLIT_KEYS - 1, pos) / TILE;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = hd >> 3;            // 16-byte pieces per row

  // a warp copies its own KPW keys and values of a tile; one table lookup per 16 keys
  auto load_tile = [&](int tile, int stage) {
    __nv_bfloat16* k_s = kv_s + ((stage * WARPS + warp) * 2 + 0) * KPW * ld;
    __nv_bfloat16* v_s = k_s + KPW * ld;
    const int w_begin = tile * TILE + warp * KPW;
    long long gran_off = 0;
    {
      const int key16 = w_begin + lane * 16;
      if (lane < KPW / 16 && key16 <= pos && key16 + 16 > lo) gran_off = granule_offset(pv, seq, key16, kvh);
    }
    for (int i = lane; i < KPW * chunks; i += 32) {
      const int r = i / chunks, c = i - r * chunks;
      const int key = w_begin + r;
      const bool valid = key >= lo && key <= pos;
      const long long off = __shfl_sync(0xffffffffu, gran_off, r >> 4) + (r & 15) * hd + c * 8;
      cp_async_16(k_s + r * ld + c * 8, k_pool + (valid ? off : 0), valid);
      cp_async_16(v_s + r * ld + c * 8, v_pool + (valid ? off : 0), valid);
    }
  };

  // ---- stage q (rows beyond the group are zero) with the first tile
  for (int i = threadIdx.x; i < 16 * chunks; i += WARPS * 32) {
    const int r = i / chunks, c = i - r * chunks;
    cp_async_16(q_s + r * ld + c * 8, q + ((long long)t * n_heads + head0 + min(r, n_rows - 1)) * hd + c * 8,
                r < n_rows);
  }
  // prologue: NSTAGE - 1 tiles on their way (an empty group where the split has fewer)
#pragma unroll
  for (int p = 0; p < NSTAGE - 1; p++) {
    if (tile0 + p <= tile1) load_tile(tile0 + p, p);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }

  const int g = lane >> 2, tq = lane & 3;
  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[DT][4];
#pragma unroll
  for (int d = 0; d < DT; d++) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  unsigned qa[KS][4];                    // the query tile as A fragments, read once

  for (int tile = tile0; tile <= tile1; tile++) {
    const int stage = (tile - tile0) % NSTAGE;
    if (tile + NSTAGE - 1 <= tile1) load_tile(tile + NSTAGE - 1, (tile - tile0 + NSTAGE - 1) % NSTAGE);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    asm volatile("cp.async.wait_group %0;\n" ::"n"(NSTAGE - 1) : "memory");
    if (tile == tile0) {
      __syncthreads();                   // q came from all warps
#pragma unroll
      for (int kk = 0; kk < KS; kk++)
        if (kk * 16 < hd) ldmatrix_x4(qa[kk], q_s + (lane & 15) * ld + kk * 16 + (lane >> 4) * 8);
    } else {
      __syncwarp();                      // keys and values of a tile are the warp's own
    }
    const __nv_bfloat16* k_s = kv_s + ((stage * WARPS + warp) * 2 + 0) * KPW * ld;
    const __nv_bfloat16* v_s = k_s + KPW * ld;
    const int w_begin = tile * TILE + warp * KPW;
    if (w_begin <= pos && w_begin + KPW > lo) {
      // ---- scores S[16 x KPW] = Q K^T
      float s[NT][4];
#pragma unroll
      for (int j = 0; j < NT; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KS; kk++) {
        if (kk * 16 < hd) {
#pragma unroll
          for (int j = 0; j < NT; j += 2) {
            unsigned b[4];
            const int mi = lane >> 3, r = lane & 7;
            ldmatrix_x4(b, k_s + (j * 8 + (mi >> 1) * 8 + r) * ld + kk * 16 + (mi & 1) * 8);
            mma_bf16(s[j], qa[kk], b[0], b[1]);
            mma_bf16(s[j + 1], qa[kk], b[2], b[3]);
          }
        }
      }
      // ---- scale, mask where the tile crosses an end of the visible range, running softmax
      const bool edge = w_begin < lo || w_begin + KPW - 1 > pos;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < NT; j++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
          float v = s[j][e] * scale_log2;
          if (edge) {
            const int key = w_begin + j * 8 + tq * 2 + (e & 1);
            if (key < lo || key > pos) v = -INFINITY;
          }
          s[j][e] = v;
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
      for (int j = 0; j < NT; j++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float p = exp2f(s[j][e] - m_use[e >> 1]);
          s[j][e] = p;
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
      for (int d = 0; d < DT; d++) {
        o[d][0] *= alpha[0]; o[d][1] *= alpha[0];
        o[d][2] *= alpha[1]; o[d][3] *= alpha[1];
      }
      // ---- O[16 x hd] += P V
#pragma unroll
      for (int kk = 0; kk < KPW / 16; kk++) {
        unsigned a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int d = 0; d < DT; d += 2) {
          if (d * 8 < hd) {
            unsigned b[4];
            const int mi = lane >> 3, r = lane & 7;
            ldmatrix_x4_trans(b, v_s + (kk * 16 + (mi & 1) * 8 + r) * ld + d * 8 + (mi >> 1) * 8);
            mma_bf16(o[d], a, b[0], b[1]);
            mma_bf16(o[d + 1], a, b[2], b[3]);
          }
        }
      }
    }
    __syncwarp();        // the warp is done with this stage before it refills it
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  __syncthreads();     // every warp is done with its keys and values: reuse the space

  // ---- combine the warps: ml_s[WARPS][16][2], o_s[WARPS][16][hd + 8] in float
  float* ml_s = reinterpret_cast<float*>(kv_s);
  float* o_s = ml_s + WARPS * 16 * 2;
  const int lo_s = hd + 8;              // row stride that spreads the 8 rows of a store over the banks
  if (tq == 0) {
    ml_s[(warp * 16 + g) * 2 + 0] = m_row[0];
    ml_s[(warp * 16 + g) * 2 + 1] = l_row[0];
    ml_s[(warp * 16 + g + 8) * 2 + 0] = m_row[1];
    ml_s[(warp * 16 + g + 8) * 2 + 1] = l_row[1];
  }
#pragma unroll
  for (int d = 0; d < DT; d++) {
    if (d * 8 < hd) {
      float* r0 = o_s + (warp * 16 + g) * lo_s + d * 8 + tq * 2;
      float* r1 = o_s + (warp * 16 + g + 8) * lo_s + d * 8 + tq * 2;
      *reinterpret_cast<float2*>(r0) = make_float2(o[d][0], o[d][1]);
      *reinterpret_cast<float2*>(r1) = make_float2(o[d][2], o[d][3]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_rows * hd; i += WARPS * 32) {
    const int r = i / hd, d = i - r * hd;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; w++) M = fmaxf(M, ml_s[(w * 16 + r) * 2]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; w++) {
      const float mw = ml_s[(w * 16 + r) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L += ml_s[(w * 16 + r) * 2 + 1] * f;
      acc += o_s[(w * 16 + r) * lo_s + d] * f;
    }
    const long long row = ((long long)t * n_heads + head0 + r) * max_splits + split;
    part_o[row * hd + d] = acc;
    if (d == 0) {
      part_ml[row * 2 + 0] = M;
      part_ml[row * 2 + 1] = L;
    }
  }
}

// One block per (token, head): merge the partials of the splits that saw keys.
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         __nv_bfloat16* __restrict__ out, const int* __restrict__ positions,
                                         int n_heads, int hd, int window, int max_splits, int split_keys) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = positions[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int s0 = lo / split_keys, s1 = pos / split_keys, n = s1 - s0 + 1;
  const long long row = ((long long)t * n_heads + h) * max_splits + s0;
  // every warp works out the same weights, a split per lane: w_s = 2^(m_s - M) / L, so that the
  // loads of the splits' statistics go out together and not one after the other
  const int lane = threadIdx.x & 31;
  float M = -INFINITY;
  for (int s = lane; s < n; s += 32) M = fmaxf(M, part_ml[(row + s) * 2]);
  M = warp_max(M);
  float L = 0.f;
  for (int s = lane; s < n; s += 32) L += part_ml[(row + s) * 2 + 1] * exp2f(part_ml[(row + s) * 2] - M);
  L = warp_sum(L);
  const float inv = 1.0f / L;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f;
    int s = 0;
    for (; s + 4 <= n; s += 4) {
      const float o0 = part_o[(row + s) * hd + d], o1 = part_o[(row + s + 1) * hd + d];
      const float o2 = part_o[(row + s + 2) * hd + d], o3 = part_o[(row + s + 3) * hd + d];
      const float m0 = part_ml[(row + s) * 2], m1 = part_ml[(row + s + 1) * 2];
      const float m2 = part_ml[(row + s + 2) * 2], m3 = part_ml[(row + s + 3) * 2];
      acc += o0 * exp2f(m0 - M);
      acc += o1 * exp2f(m1 - M);
      acc += o2 * exp2f(m2 - M);
      acc += o3 * exp2f(m3 - M);
    }
    for (; s < n; s++) acc += part_o[(row + s) * hd + d] * exp2f(part_ml[(row + s) * 2] - M);
    out[((long long)t * n_heads + h) * hd + d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int HD_MAX>
int launch_decode(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool,
                  __nv_bfloat16* out, float* part_o, float* part_ml, int n_tokens, int n_heads, PagedView pv,
                  const int* positions, const int* seq_of_token, float scale, int window, int max_ctx,
                  cudaStream_t stream) {
  constexpr int KPW = Tile<HD_MAX>::KPW;
  constexpr int WARPS = Tile<HD_MAX>::W;
  constexpr int SPLIT = SPLIT_KEYS;
  const int hd = pv.head_dim, ld = hd + 8;
  const int max_splits = (max_ctx + SPLIT - 1) / SPLIT;
  const int G = n_heads / pv.n_kv_heads;
  const int hgroups = (G + 15) / 16;
  const size_t stage = (size_t)(16 * ld + NSTAGE * WARPS * 2 * KPW * ld) * sizeof(__nv_bfloat16);
  const size_t combine = (size_t)16 * ld * sizeof(__nv_bfloat16) + (size_t)WARPS * 16 * (10 + hd) * sizeof(float);
  const size_t smem = stage > combine ? stage : combine;
  static DeviceOnce once;
  const int dev_ = mf_current_device();
  if (dev_ < 0) return MF_ERR_BAD_ARG;
  if (!once.done[dev_]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_decode_kernel<HD_MAX>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return (int)e;
    once.done[dev_] = true;
  }
  dim3 grid(max_splits, pv.n_kv_heads * hgroups, n_tokens);
  mf_count(MF_K_ATTN_DECODE);
  mf_count(MF_K_ATTN_DECODE_MERGE);
  cudaError_t e = launch_dep(attn_decode_kernel<HD_MAX>, grid, dim3(WARPS * 32), smem, stream, q, k_pool, v_pool,
                             part_o, part_ml, positions, seq_of_token, pv, n_heads, scale * LOG2E, window, max_splits);
  if (e != cudaSuccess) return (int)e;
  dim3 mgrid(n_tokens, n_heads);
  return (int)launch_dep(attn_decode_merge_kernel, mgrid, dim3(hd >= 128 ? 128 : 64), 0, stream,
                         (const float*)part_o, (const float*)part_ml, out, positions, n_heads, hd, window, max_splits,
                         SPLIT);
}

}  // namespace

// attention_decode_tma.cu: the first kernel with keys and values brought in by the TMA unit
int launch_decode_tma(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool,
                      __nv_bfloat16* out, float* part_o, float* part_ml, int n_tokens, int n_heads, PagedView pv,
                      long long pool_rows, const int* positions, const int* seq_of_token, float scale, int window,
                      int max_ctx, int unequal, int* status, int* split_out, int* merged_out, cudaStream_t stream);
extern int g_merge_inside;

static int g_decode_tma = 1;
static int g_last_decode_launches = 2;

// How many kernels the last call of mf_attention_decode launched (1: the TMA kernel merged its
// splits itself; 2: a merge kernel followed).
MF_API int mf_attention_decode_launches() { return g_last_decode_launches; }
static int* g_decode_status = nullptr;

// Whether head size 64 takes the TMA kernel (default on), and the device word its bounded
// waits report to (may be null).  Returns the previous on/off setting.
// 1 (the default): the TMA kernel merges its splits itself; 0: the merge kernel follows it.
MF_API int mf_set_decode_merge_inside(int on) {
  const int old = g_merge_inside;
  g_merge_inside = on ? 1 : 0;
  return old;
}

MF_API int mf_set_decode_tma(int on, int* status) {
  const int old = g_decode_tma;
  g_decode_tma = on ? 1 : 0;
  g_decode_status = status;
  return old;
}
// The status word alone; the on/off setting stays as it is.
MF_API int mf_set_decode_status(int* status) {
  g_decode_status = status;
  return 0;
}

// Fewest keys per split for a head size: the caller sizes the scratch with it (a launch may
// choose longer splits and then uses less).
MF_API int mf_attention_decode_split(int hd) {
  (void)hd;
  return SPLIT_KEYS;
}

// Scratch: part_o  [n_tokens * n_heads * max_splits * hd] floats,
//          part_ml [n_tokens * n_heads * max_splits * 2] floats, max_splits = ceil(max_ctx / split).
// `max_ctx` bounds position + 1 of every token; a larger value only costs idle blocks.
// `unequal_contexts` != 0: the caller knows that the tokens' contexts differ widely in length (the
// kernels read the lengths on the device, the launcher cannot); with many work items to a block
// the kernel whose blocks the hardware deals out is then taken instead of the persistent one.
MF_API int mf_attention_decode_hinted(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_o,
                                      float* part_ml, int n_tokens, int n_heads, int n_kv, int hd, const int* positions,
                                      const int* seq_of_token, const int* block_table, int bt_stride, int page_size,
                                      float scale, int window, int max_ctx, int unequal_contexts, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd < 16 || hd > 256 || hd % 16 || n_kv <= 0 || n_heads % n_kv || max_ctx <= 0) return MF_ERR_BAD_ARG;
  if (n_tokens > 65535) return MF_ERR_BAD_ARG;
  PagedView pv{block_table, bt_stride, page_size, n_kv, hd};
  g_last_decode_launches = 2;
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)k_pool,
                      *vv = (const __nv_bfloat16*)v_pool;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
  if ((hd == 64 || hd == 128) && g_decode_tma) {
    // the map's row count only bounds the unit's own range check; rows beyond the pool are never asked for
    int split = SPLIT_KEYS, merged = 0;
    const int rc = launch_decode_tma(qq, kk, vv, oo, part_o, part_ml, n_tokens, n_heads, pv, 1ll << 28, positions,
                                     seq_of_token, scale, window, max_ctx, unequal_contexts, g_decode_status, &split,
                                     &merged, stream);
    if (rc == 0 && merged) {
      mf_count(MF_K_ATTN_DECODE_TMA_MERGED);
      g_last_decode_launches = 1;
      return 0;
    }
    if (rc == 0) {
      mf_count(MF_K_ATTN_DECODE_TMA);
      mf_count(MF_K_ATTN_DECODE_MERGE);
      const int max_splits = (max_ctx + split - 1) / split;
      dim3 mgrid(n_tokens, n_heads);
      return (int)launch_dep(attn_decode_merge_kernel, mgrid, dim3(hd), 0, stream, (const float*)part_o,
                             (const float*)part_ml, oo, positions, n_heads, hd, window, max_splits, split);
    }
    if (rc != MF_ERR_BAD_ARG) return rc;
  }
  if (hd <= 64)
    return launch_decode<64>(qq, kk, vv, oo, part_o, part_ml, n_tokens, n_heads, pv, positions, seq_of_token, scale,
                             window, max_ctx, stream);
  if (hd <= 128)
    return launch_decode<128>(qq, kk, vv, oo, part_o, part_ml, n_tokens, n_heads, pv, positions, seq_of_token,
                              scale, window, max_ctx, stream);
  return launch_decode<256>(qq, kk, vv, oo, part_o, part_ml, n_tokens, n_heads, pv, positions, seq_of_token, scale,
                            window, max_ctx, stream);
}

MF_API int mf_attention_decode(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_o,
                               float* part_ml, int n_tokens, int n_heads, int n_kv, int hd, const int* positions,
                               const int* seq_of_token, const int* block_table, int bt_stride, int page_size,
                               float scale, int window, int max_ctx, cudaStream_t stream) {
  return mf_attention_decode_hinted(q, k_pool, v_pool, out, part_o, part_ml, n_tokens, n_heads, n_kv, hd, positions,
                                    seq_of_token, block_table, bt_stride, page_size, scale, window, max_ctx, 0, stream);
}

// ---------------------------------------------------------------------------------------------
// mf_attention_decode_static: the same attention, for callers that cannot give it scratch memory.
// Declared and described in attention_decode_static.h.
#include "attention_decode_static.h"

#include <cstdio>
#include <mutex>

namespace {

// The partial results of kernel 1 live here instead of in caller-provided buffers.  One copy per
// GPU that loads this library, held until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[MF_DECODE_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_static_mutex;
float* g_static_ptr[MAX_DEVICES] = {};     // device address of g_static_scratch, per device ordinal

void say(char* err, int err_len, const char* fmt, long long a = 0, long long b = 0) {
  if (err && err_len > 0) snprintf(err, (size_t)err_len, fmt, a, b);
}

}  // namespace

MF_API long long mf_attention_decode_static_bytes(int n_tokens, int n_heads, int hd, int max_ctx) {
  if (n_tokens <= 0 || n_heads <= 0 || hd <= 0 || max_ctx <= 0) return 0;
  const int split = mf_attention_decode_split(hd);
  const long long splits = (max_ctx + split - 1) / split;
  return (long long)n_tokens * n_heads * splits * (hd + 2) * (long long)sizeof(float);
}

MF_API int mf_attention_decode_static(const void* q, const void* k_pool, const void* v_pool, void* out,
                                      int n_tokens, int n_heads, int n_kv, int hd, const int* positions,
                                      const int* seq_of_token, const int* block_table, int bt_stride,
                                      int page_size, float scale, int window, int max_ctx, cudaStream_t stream,
                                      char* err, int err_len) {
  if (n_tokens <= 0) return 0;
  if (hd < 16 || hd > 256 || hd % 16 || n_kv <= 0 || n_heads <= 0 || n_heads % n_kv || max_ctx <= 0 ||
      n_tokens > 65535) {
    say(err, err_len, "mf_attention_decode_static: unsupported sizes (head size must be a multiple of 16 in "
                      "[16, 256], heads a multiple of KV heads, at most 65535 tokens)");
    return MF_ERR_BAD_ARG;
  }
  const long long need = mf_attention_decode_static_bytes(n_tokens, n_heads, hd, max_ctx);
  if (need > (long long)MF_DECODE_STATIC_SCRATCH_BYTES) {
    say(err, err_len, "mf_attention_decode_static: this call needs %lld bytes of scratch, the built-in array "
                      "holds %lld; use mf_attention_decode with buffers of your own",
        need, (long long)MF_DECODE_STATIC_SCRATCH_BYTES);
    return MF_ERR_SCRATCH_LIMIT;
  }
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= MAX_DEVICES) {
    say(err, err_len, "mf_attention_decode_static: device ordinal %lld is beyond the %lld this table holds",
        device, MAX_DEVICES);
    return MF_ERR_BAD_ARG;
  }
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_ptr[device] == nullptr) {
      // In host code `g_static_scratch` is only a handle: the address the kernels may use is this one.
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess) {
        say(err, err_len, "mf_attention_decode_static: cudaGetSymbolAddress failed with CUDA error %lld", (int)e);
        return (int)e;
      }
      g_static_ptr[device] = static_cast<float*>(p);
    }
    scratch = g_static_ptr[device];
  }
  const int split = mf_attention_decode_split(hd);
  const long long splits = (max_ctx + split - 1) / split;
  float* part_o = scratch;
  float* part_ml = scratch + (long long)n_tokens * n_heads * splits * hd;
  return mf_attention_decode(q, k_pool, v_pool, out, part_o, part_ml, n_tokens, n_heads, n_kv, hd, positions,
                             seq_of_token, block_table, bt_stride, page_size, scale, window, max_ctx, stream);
}
