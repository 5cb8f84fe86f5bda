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

constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
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

// keys per warp by head size: the tile of one warp is KPW x (hd + 8) x 2 (K and V) bf16
template <int HD_MAX> struct Tile { static constexpr int KPW = HD_MAX <= 64 ? 64 : (HD_MAX <= 128 ? 32 : 16); };

template <int HD_MAX>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                   const __nv_bfloat16* __restrict__ v_pool, float* __restrict__ part_o,
                   float* __restrict__ part_ml, const int* __restrict__ positions,
                   const int* __restrict__ seq_of_token, PagedView pv, int n_heads, float scale_log2,
                   int window, int max_splits) {
  constexpr int KPW = Tile<HD_MAX>::KPW;
  constexpr int SPLIT = KPW * WARPS;
  constexpr int NT = KPW / 8;           // score n-tiles per warp
  constexpr int DT = HD_MAX / 8;        // output n-tiles (channels / 8)
  const int hd = pv.head_dim;
  const int ld = hd + 8;                // padded row: conflict-free ldmatrix for every hd % 16 == 0
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [16][ld]
  __nv_bfloat16* kv_s = q_s + 16 * ld;                                              // [WARPS][2][KPW][ld]

  const int split = blockIdx.x, t = blockIdx.z;
  const int G = n_heads / pv.n_kv_heads;
  const int hgroups = (G + 15) / 16;
  const int kvh = blockIdx.y / hgroups, hg = blockIdx.y - kvh * hgroups;
  const int head0 = kvh * G + hg * 16;
  const int n_rows = min(16, G - hg * 16);
  const int pos = positions[t], seq = seq_of_token[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int k_begin = split * SPLIT;
  if (k_begin > pos || k_begin + SPLIT <= lo) return;       // nothing visible in this split

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = hd >> 3;            // 16-byte pieces per row

  // ---- stage q (rows beyond the group are zero) and this warp's keys and values
  for (int i = threadIdx.x; i < 16 * chunks; i += WARPS * 32) {
    const int r = i / chunks, c = i - r * chunks;
    cp_async_16(q_s + r * ld + c * 8, q + ((long long)t * n_heads + head0 + min(r, n_rows - 1)) * hd + c * 8,
                r < n_rows);
  }
  __nv_bfloat16* k_s = kv_s + (warp * 2 + 0) * KPW * ld;
  __nv_bfloat16* v_s = kv_s + (warp * 2 + 1) * KPW * ld;
  const int w_begin = k_begin + warp * KPW;
  for (int i = lane; i < KPW * chunks; i += 32) {
    const int r = i / chunks, c = i - r * chunks;
    const int key = w_begin + r;
    const bool valid = key >= lo && key <= pos;
    long long off = 0;
    if (valid) off = paged_offset(pv, seq, key, kvh) + c * 8;
    cp_async_16(k_s + r * ld + c * 8, k_pool + off, valid);
    cp_async_16(v_s + r * ld + c * 8, v_pool + off, valid);
  }
  cp_async_wait_all();
  __syncthreads();

  const int g = lane >> 2, tq = lane & 3;
  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[DT][4];
#pragma unroll
  for (int d = 0; d < DT; d++) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  if (w_begin <= pos && w_begin + KPW > lo) {
    // ---- scores S[16 x KPW] = Q K^T
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD_MAX / 16; kk++) {
      if (kk * 16 < hd) {
        unsigned a[4];
        ldmatrix_x4(a, q_s + (lane & 15) * ld + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
          unsigned b[4];
          const int mi = lane >> 3, r = lane & 7;
          ldmatrix_x4(b, k_s + (j * 8 + (mi >> 1) * 8 + r) * ld + kk * 16 + (mi & 1) * 8);
          mma_bf16(s[j], a, b[0], b[1]);
          mma_bf16(s[j + 1], a, b[2], b[3]);
        }
      }
    }
    // ---- mask, softmax statistics of this warp's keys (rows g and g + 8)
#pragma unroll
    for (int j = 0; j < NT; j++) {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int key = w_begin + j * 8 + tq * 2 + (e & 1);
        const float v = (key >= lo && key <= pos) ? s[j][e] * scale_log2 : -INFINITY;
        s[j][e] = v;
        m_row[e >> 1] = fmaxf(m_row[e >> 1], v);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
      m_row[h] = fmaxf(m_row[h], __shfl_xor_sync(0xffffffffu, m_row[h], 1));
      m_row[h] = fmaxf(m_row[h], __shfl_xor_sync(0xffffffffu, m_row[h], 2));
    }
    const float m_use[2] = {m_row[0] == -INFINITY ? 0.f : m_row[0], m_row[1] == -INFINITY ? 0.f : m_row[1]};
#pragma unroll
    for (int j = 0; j < NT; j++) {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float p = exp2f(s[j][e] - m_use[e >> 1]);
        s[j][e] = p;
        l_row[e >> 1] += p;
      }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
      l_row[h] += __shfl_xor_sync(0xffffffffu, l_row[h], 1);
      l_row[h] += __shfl_xor_sync(0xffffffffu, l_row[h], 2);
    }
    // ---- O[16 x hd] = P V
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
  __syncthreads();     // every warp is done with its keys and values: reuse the space

  // ---- combine the warps: ml_s[WARPS][16][2], o_s[WARPS][16][hd] in float
  float* ml_s = reinterpret_cast<float*>(kv_s);
  float* o_s = ml_s + WARPS * 16 * 2;
  if (tq == 0) {
    ml_s[(warp * 16 + g) * 2 + 0] = m_row[0];
    ml_s[(warp * 16 + g) * 2 + 1] = l_row[0];
    ml_s[(warp * 16 + g + 8) * 2 + 0] = m_row[1];
    ml_s[(warp * 16 + g + 8) * 2 + 1] = l_row[1];
  }
#pragma unroll
  for (int d = 0; d < DT; d++) {
    if (d * 8 < hd) {
      float* r0 = o_s + (warp * 16 + g) * hd + d * 8 + tq * 2;
      float* r1 = o_s + (warp * 16 + g + 8) * hd + d * 8 + tq * 2;
      r0[0] = o[d][0]; r0[1] = o[d][1];
      r1[0] = o[d][2]; r1[1] = o[d][3];
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
      acc += o_s[(w * 16 + r) * hd + d] * f;
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
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = positions[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int s0 = lo / split_keys, s1 = pos / split_keys;
  const long long row = ((long long)t * n_heads + h) * max_splits;
  float M = -INFINITY;
  for (int s = s0; s <= s1; s++) M = fmaxf(M, part_ml[(row + s) * 2]);
  float L = 0.f;
  for (int s = s0; s <= s1; s++) L += part_ml[(row + s) * 2 + 1] * exp2f(part_ml[(row + s) * 2] - M);
  const float inv = 1.0f / L;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f;
    for (int s = s0; s <= s1; s++) acc += part_o[(row + s) * hd + d] * exp2f(part_ml[(row + s) * 2] - M);
    out[((long long)t * n_heads + h) * hd + d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int HD_MAX>
int launch_decode(const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool,
                  __nv_bfloat16* out, float* part_o, float* part_ml, int n_tokens, int n_heads, PagedView pv,
                  const int* positions, const int* seq_of_token, float scale, int window, int max_ctx,
                  cudaStream_t stream) {
  constexpr int KPW = Tile<HD_MAX>::KPW;
  constexpr int SPLIT = KPW * WARPS;
  const int hd = pv.head_dim, ld = hd + 8;
  const int max_splits = (max_ctx + SPLIT - 1) / SPLIT;
  const int G = n_heads / pv.n_kv_heads;
  const int hgroups = (G + 15) / 16;
  const size_t stage = (size_t)(16 * ld + WARPS * 2 * KPW * ld) * sizeof(__nv_bfloat16);
  const size_t combine = (size_t)16 * ld * sizeof(__nv_bfloat16) + (size_t)WARPS * 16 * (2 + hd) * sizeof(float);
  const size_t smem = stage > combine ? stage : combine;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(max_splits, pv.n_kv_heads * hgroups, n_tokens);
  attn_decode_kernel<HD_MAX><<<grid, WARPS * 32, smem, stream>>>(q, k_pool, v_pool, part_o, part_ml, positions,
                                                                seq_of_token, pv, n_heads, scale * LOG2E, window,
                                                                max_splits);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  dim3 mgrid(n_tokens, n_heads);
  attn_decode_merge_kernel<<<mgrid, hd >= 128 ? 128 : 64, 0, stream>>>(part_o, part_ml, out, positions, n_heads, hd,
                                                                       window, max_splits, SPLIT);
  return (int)cudaGetLastError();
}

}  // namespace

// Keys per split for a head size (the caller sizes the scratch with it).
MF_API int mf_attention_decode_split(int hd) {
  if (hd <= 64) return Tile<64>::KPW * WARPS;
  if (hd <= 128) return Tile<128>::KPW * WARPS;
  return Tile<256>::KPW * WARPS;
}

// Scratch: part_o  [n_tokens * n_heads * max_splits * hd] floats,
//          part_ml [n_tokens * n_heads * max_splits * 2] floats, max_splits = ceil(max_ctx / split).
// `max_ctx` bounds position + 1 of every token; a larger value only costs idle blocks.
MF_API int mf_attention_decode(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_o,
                               float* part_ml, int n_tokens, int n_heads, int n_kv, int hd, const int* positions,
                               const int* seq_of_token, const int* block_table, int bt_stride, int page_size,
                               float scale, int window, int max_ctx, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd < 16 || hd > 256 || hd % 16 || n_kv <= 0 || n_heads % n_kv || max_ctx <= 0) return MF_ERR_BAD_ARG;
  if (n_tokens > 65535) return MF_ERR_BAD_ARG;
  PagedView pv{block_table, bt_stride, page_size, n_kv, hd};
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)k_pool,
                      *vv = (const __nv_bfloat16*)v_pool;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
  if (hd <= 64)
    return launch_decode<64>(qq, kk, vv, oo, part_o, part_ml, n_tokens, n_heads, pv, positions, seq_of_token, scale,
                             window, max_ctx, stream);
  if (hd <= 128)
    return launch_decode<128>(qq, kk, vv, oo, part_o, part_ml, n_tokens, n_heads, pv, positions, seq_of_token,
                              scale, window, max_ctx, stream);
  return launch_decode<256>(qq, kk, vv, oo, part_o, part_ml, n_tokens, n_heads, pv, positions, seq_of_token, scale,
                            window, max_ctx, stream);
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
