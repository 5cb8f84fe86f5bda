// Memory-bound kernels of the decoder step: embedding gather, residual add fused
// with RMSNorm, rotary position encoding fused with the write of keys and values
// into cache pages, and the SiLU-gated product of the feed-forward.
//
// Reference formulas (hvasconcelos/mlxforge): embedding src/model/decoder_model.cpp:194-204,
// RMSNorm :206-208, rotation :220-228, SwiGLU :277-282, residuals :288-293.
// Sums of squares, angles and the residual stream are 32-bit here.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int H) {
  const int t = blockIdx.x;
  const T* row = table + (long long)tokens[t] * H;
  float* o = out + (long long)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32<T>(row[i]);
}

MF_API int mf_embed(const void* table, int table_dtype, const int* tokens, float* out, int T, int H,
                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (table_dtype == MF_F32)
    embed_kernel<float><<<T, 256, 0, stream>>>((const float*)table, tokens, out, H);
  else if (table_dtype == MF_BF16)
    embed_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>((const __nv_bfloat16*)table, tokens, out, H);
  else
    return MF_ERR_BAD_DTYPE;
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ add + RMSNorm
// out[r] = rmsnorm(resid[src] + delta[src]) * w, src = rows ? rows[r] : r.
// Without `rows` the sum is written back to resid (the residual stream moves on);
// with `rows` only the selected rows are produced and resid is left alone.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   const float* __restrict__ w, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H) {
  __shared__ float red[32];
  const int r = blockIdx.x;
  const long long src = rows ? rows[r] : r;
  float* x = resid + src * H;
  const TD* d = delta ? delta + src * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = x[i];
    if (d) {
      v += to_f32<TD>(d[i]);
      if (!rows) x[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  TO* o = out + (long long)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = x[i];
    if (d && rows) v += to_f32<TD>(d[i]);
    o[i] = from_f32<TO>(v * inv * w[i]);
  }
}

MF_API int mf_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const float* w, float eps,
                          void* out, int out_dtype, const int* rows, int n_rows, int H,
                          cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
#define LAUNCH(TD, TO)                                                                          \
  add_rmsnorm_kernel<TD, TO><<<n_rows, threads, 0, stream>>>(resid, (const TD*)delta, w, eps,   \
                                                             (TO*)out, rows, H)
  if (delta_dtype == MF_F32 && out_dtype == MF_F32) LAUNCH(float, float);
  else if (delta_dtype == MF_BF16 && out_dtype == MF_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (delta_dtype == MF_F32 && out_dtype == MF_BF16) LAUNCH(float, __nv_bfloat16);
  else if (delta_dtype == MF_BF16 && out_dtype == MF_F32) LAUNCH(__nv_bfloat16, float);
  else return MF_ERR_BAD_DTYPE;
#undef LAUNCH
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ RoPE + KV write
// One block per token.  qkv row = [q heads | k heads | v heads], each head_dim wide.
// Half-split pairing over the first rot_dim channels: (i, i + rot_dim/2), angle =
// position / freq[i].  `precise` computes the angle and its sine/cosine in double
// (the 32-bit model path); otherwise float32 with the accurate sincosf.
// Rotated q goes to q_out [T, n_heads*hd]; rotated k and plain v go to their pages.
template <typename T>
__global__ void rope_kv_write_kernel(const T* __restrict__ qkv, int n_heads, int n_kv, int hd, int rot,
                                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                     PagedView pv, const float* __restrict__ freqs, T* __restrict__ q_out,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool, int write_kv,
                                     int precise) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int seq = seq_of_token[t];
  const int half = rot >> 1;
  const int width = (n_heads + 2 * n_kv) * hd;
  const T* row = qkv + (long long)t * width;
  const int hpairs = hd - half;           // per head: `half` rotated pairs + (hd - rot) pass-through channels
  // q and k heads
  const int n_rot_heads = n_heads + (write_kv ? n_kv : 0);
  for (int idx = threadIdx.x; idx < n_rot_heads * hpairs; idx += blockDim.x) {
    const int h = idx / hpairs, j = idx - h * hpairs;
    const T* src = row + (long long)h * hd;
    T* dst;
    if (h < n_heads) dst = q_out + ((long long)t * n_heads + h) * hd;
    else dst = k_pool + paged_offset(pv, seq, pos, h - n_heads);
    if (j < half) {
      float c, s;
      if (precise) {
        const double a = (double)pos / (double)freqs[j];
        c = (float)cos(a);
        s = (float)sin(a);
      } else {
        const float a = (float)pos / freqs[j];
        sincosf(a, &s, &c);
      }
      const float x1 = to_f32<T>(src[j]), x2 = to_f32<T>(src[j + half]);
      dst[j] = from_f32<T>(x1 * c - x2 * s);
      dst[j + half] = from_f32<T>(x1 * s + x2 * c);
    } else {
      const int ch = rot + (j - half);
      dst[ch] = src[ch];
    }
  }
  if (write_kv) {
    for (int idx = threadIdx.x; idx < n_kv * hd; idx += blockDim.x) {
      const int h = idx / hd, ch = idx - h * hd;
      v_pool[paged_offset(pv, seq, pos, h) + ch] = row[(long long)(n_heads + n_kv + h) * hd + ch];
    }
  }
}

MF_API int mf_rope_kv_write(const void* qkv, int dtype, int T, int n_heads, int n_kv, int hd, int rot_dim,
                            const int* positions, const int* seq_of_token, const int* block_table,
                            int bt_stride, int page_size, const float* freqs, void* q_out, void* k_pool,
                            void* v_pool, int write_kv, int precise, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot_dim < 0 || rot_dim > hd || (rot_dim & 1)) return MF_ERR_BAD_ARG;
  PagedView pv{block_table, bt_stride, page_size, n_kv, hd};
  if (dtype == MF_F32)
    rope_kv_write_kernel<float><<<T, 256, 0, stream>>>((const float*)qkv, n_heads, n_kv, hd, rot_dim, positions,
                                                       seq_of_token, pv, freqs, (float*)q_out, (float*)k_pool,
                                                       (float*)v_pool, write_kv, precise);
  else if (dtype == MF_BF16)
    rope_kv_write_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>(
        (const __nv_bfloat16*)qkv, n_heads, n_kv, hd, rot_dim, positions, seq_of_token, pv, freqs,
        (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, write_kv, precise);
  else
    return MF_ERR_BAD_DTYPE;
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ SwiGLU
// gu [T, 2I] holds gate and up interleaved in groups of `group` columns:
// gate i is column (i / group) * 2 * group + i % group, up i is `group` further.
// group == I is the plain [gate | up] concatenation.  out[t, i] = silu(gate) * up.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, long long n, int I, int group) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const long long t = idx / I;
  const int i = (int)(idx - t * I);
  const int col = (i / group) * 2 * group + (i % group);
  const T* row = gu + t * 2 * (long long)I;
  const float g = to_f32<T>(row[col]), u = to_f32<T>(row[col + group]);
  out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

MF_API int mf_swiglu(const void* gu, void* out, int dtype, int T, int I, int group, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (group <= 0 || I % group) return MF_ERR_BAD_ARG;
  const long long n = (long long)T * I;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  if (dtype == MF_F32)
    swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, n, I, group);
  else if (dtype == MF_BF16)
    swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                                                                 n, I, group);
  else
    return MF_ERR_BAD_DTYPE;
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ plain residual add
// resid[i] += delta[i] (the stream's last pending delta, when no norm follows).
template <typename TD>
__global__ void add_kernel(float* __restrict__ resid, const TD* __restrict__ delta, long long n) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n) resid[idx] += to_f32<TD>(delta[idx]);
}
MF_API int mf_residual_add(float* resid, const void* delta, int delta_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (delta_dtype == MF_F32) add_kernel<float><<<blocks, 256, 0, stream>>>(resid, (const float*)delta, n);
  else if (delta_dtype == MF_BF16)
    add_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(resid, (const __nv_bfloat16*)delta, n);
  else return MF_ERR_BAD_DTYPE;
  return (int)cudaGetLastError();
}
