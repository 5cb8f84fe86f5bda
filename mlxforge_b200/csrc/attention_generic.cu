// Causal GQA attention over the paged cache, any number of new tokens per
// sequence, float32 or bfloat16 storage, every score and the softmax in 32-bit.
// One block per (token, query head).  It is the attention of the 32-bit model
// path and the plain device reference the faster bfloat16 kernels are checked
// against.  Formula: src/model/sdpa.cpp:71-95 and src/model/decoder_model.cpp:260-275
// of hvasconcelos/mlxforge (scores * scale, causal mask aligned to the end of the
// keys, softmax over keys, p * v; query head h reads KV head h / (nh/nkv)).
//
// The query at position p of its sequence sees keys [lo, p], lo = 0 or
// p - window + 1 for a windowed lane.  Keys are visited in chunks of 128 starting
// at a multiple of 128, so the order of every sum depends only on the position.
#include "common.cuh"

#define CHUNK 128

template <typename T>
__global__ void __launch_bounds__(CHUNK)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         T* __restrict__ out, const int* __restrict__ positions,
                         const int* __restrict__ seq_of_token, PagedView pv, int n_heads, float scale,
                         int window) {
  extern __shared__ float smem[];
  float* qs = smem;                 // [hd]
  float* ps = smem + pv.head_dim;   // [CHUNK]
  __shared__ float red[32];
  const int t = blockIdx.x, h = blockIdx.y;
  const int hd = pv.head_dim;
  const int kvh = h / (n_heads / pv.n_kv_heads);
  const int pos = positions[t], seq = seq_of_token[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  const T* qrow = q + ((long long)t * n_heads + h) * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = to_f32<T>(qrow[d]);
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  float acc0 = 0.f, acc1 = 0.f;     // output channels threadIdx.x and threadIdx.x + CHUNK (hd <= 256)
  for (int c0 = (lo / CHUNK) * CHUNK; c0 <= pos; c0 += CHUNK) {
    const int j = c0 + threadIdx.x;
    float s = -INFINITY;
    if (j >= lo && j <= pos) {
      const T* kr = k_pool + paged_offset(pv, seq, j, kvh);
      float dot = 0.f;
      for (int d = 0; d < hd; d++) dot = fmaf(qs[d], to_f32<T>(kr[d]), dot);
      s = dot * scale;
    }
    const float cm = block_max(s, red);
    const float m_new = fmaxf(m, cm);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    __syncthreads();
    ps[threadIdx.x] = p;
    const float psum = block_sum(p, red);   // has __syncthreads inside: ps is visible after it
    l = l * alpha + psum;
    m = m_new;
    acc0 *= alpha;
    acc1 *= alpha;
    const int jn = min(CHUNK, pos - c0 + 1);
    for (int jj = max(0, lo - c0); jj < jn; jj++) {
      const float pj = ps[jj];
      const T* vr = v_pool + paged_offset(pv, seq, c0 + jj, kvh);
      if ((int)threadIdx.x < hd) acc0 = fmaf(pj, to_f32<T>(vr[threadIdx.x]), acc0);
      if ((int)threadIdx.x + CHUNK < hd) acc1 = fmaf(pj, to_f32<T>(vr[threadIdx.x + CHUNK]), acc1);
    }
    __syncthreads();
  }
  T* orow = out + ((long long)t * n_heads + h) * hd;
  const float inv = 1.0f / l;
  if ((int)threadIdx.x < hd) orow[threadIdx.x] = from_f32<T>(acc0 * inv);
  if ((int)threadIdx.x + CHUNK < hd) orow[threadIdx.x + CHUNK] = from_f32<T>(acc1 * inv);
}

MF_API int mf_attention_generic(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                int T, int n_heads, int n_kv, int hd, const int* positions,
                                const int* seq_of_token, const int* block_table, int bt_stride,
                                int page_size, float scale, int window, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd > 2 * CHUNK || n_kv <= 0 || n_heads % n_kv) return MF_ERR_BAD_ARG;
  if (n_heads > 65535) return MF_ERR_BAD_ARG;
  PagedView pv{block_table, bt_stride, page_size, n_kv, hd};
  dim3 grid(T, n_heads);
  const size_t smem = (size_t)(hd + CHUNK) * sizeof(float);
  if (dtype == MF_F32 || dtype == MF_BF16) mf_count(MF_K_ATTN_GENERIC);
  if (dtype == MF_F32)
    attention_generic_kernel<float><<<grid, CHUNK, smem, stream>>>(
        (const float*)q, (const float*)k_pool, (const float*)v_pool, (float*)out, positions, seq_of_token, pv,
        n_heads, scale, window);
  else if (dtype == MF_BF16)
    attention_generic_kernel<__nv_bfloat16><<<grid, CHUNK, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
        (__nv_bfloat16*)out, positions, seq_of_token, pv, n_heads, scale, window);
  else
    return MF_ERR_BAD_DTYPE;
  return (int)cudaGetLastError();
}
