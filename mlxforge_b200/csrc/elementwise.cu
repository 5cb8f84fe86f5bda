// Memory-bound kernels of the decoder step: embedding gather, residual add fused
// with RMSNorm, rotary position encoding fused with the write of keys and values
// into cache pages, and the SiLU-gated product of the feed-forward.
//
// Reference formulas (hvasconcelos/mlxforge): embedding src/model/decoder_model.cpp:194-204,
// RMSNorm :206-208, rotation :220-228, SwiGLU :277-282, residuals :288-293.
// Sums of squares, angles and the residual stream are 32-bit here.
#include "common.cuh"

int g_mf_pdl = 1;
MF_API int mf_set_pdl(int on) {
  const int old = g_mf_pdl;
  g_mf_pdl = on ? 1 : 0;
  return old;
}

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int H) {
  const int t = blockIdx.x;
  const T* row = table + (long long)tokens[t] * H;
  float* o = out + (long long)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32<T>(row[i]);
}

// bfloat16 rows in 16-byte pieces (H a multiple of 8)
__global__ void embed_bf16_vec_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ tokens,
                                      float* __restrict__ out, int H) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(table + (long long)tokens[t] * H);
  float4* o = reinterpret_cast<float4*>(out + (long long)t * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 v = row[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
    const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
    const float2 c = __bfloat1622float2(p[2]), d = __bfloat1622float2(p[3]);
    o[2 * i] = make_float4(a.x, a.y, b.x, b.y);
    o[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
  }
}

MF_API int mf_embed(const void* table, int table_dtype, const int* tokens, float* out, int T, int H,
                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (table_dtype == MF_BF16 && H % 8 == 0 && ((uintptr_t)table & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    return (int)launch_dep(embed_bf16_vec_kernel, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)table, tokens,
                           out, H);
  }
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

// The serving case in 16-byte pieces: bfloat16 delta and output, H a multiple of 8 and at
// most 8 * 256 * NV, every value held in registers between the two passes.
template <int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_bf16_vec_kernel(float* __restrict__ resid, const __nv_bfloat16* __restrict__ delta,
                            const float* __restrict__ w, float eps, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ rows, int H) {
  __shared__ float red[32];
  pdl_launch();              // the product after this one fetches its weights meanwhile
  pdl_wait();
  const int r = blockIdx.x;
  const long long src = rows ? rows[r] : r;
  float* x = resid + src * H;
  const __nv_bfloat16* d = delta ? delta + src * H : nullptr;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NV; j++) {
    const int i = (j * 256 + threadIdx.x) * 8;
    if (i < H) {
      const float4 a = *reinterpret_cast<const float4*>(x + i), b = *reinterpret_cast<const float4*>(x + i + 4);
      v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
      v[j][4] = b.x; v[j][5] = b.y; v[j][6] = b.z; v[j][7] = b.w;
      if (d) {
        const uint4 dv = *reinterpret_cast<const uint4*>(d + i);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float2 f = __bfloat1622float2(p[e]);
          v[j][2 * e] += f.x;
          v[j][2 * e + 1] += f.y;
        }
        if (!rows) {
          *reinterpret_cast<float4*>(x + i) = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
          *reinterpret_cast<float4*>(x + i + 4) = make_float4(v[j][4], v[j][5], v[j][6], v[j][7]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; e++) ss += v[j][e] * v[j][e];
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  __nv_bfloat16* o = out + (long long)r * H;
#pragma unroll
  for (int j = 0; j < NV; j++) {
    const int i = (j * 256 + threadIdx.x) * 8;
    if (i < H) {
      const float4 wa = *reinterpret_cast<const float4*>(w + i), wb = *reinterpret_cast<const float4*>(w + i + 4);
      uint4 pk;
      __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&pk);
      p[0] = __floats2bfloat162_rn(v[j][0] * inv * wa.x, v[j][1] * inv * wa.y);
      p[1] = __floats2bfloat162_rn(v[j][2] * inv * wa.z, v[j][3] * inv * wa.w);
      p[2] = __floats2bfloat162_rn(v[j][4] * inv * wb.x, v[j][5] * inv * wb.y);
      p[3] = __floats2bfloat162_rn(v[j][6] * inv * wb.z, v[j][7] * inv * wb.w);
      *reinterpret_cast<uint4*>(o + i) = pk;
    }
  }
}

MF_API int mf_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const float* w, float eps,
                          void* out, int out_dtype, const int* rows, int n_rows, int H,
                          cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (out_dtype == MF_BF16 && (delta == nullptr || delta_dtype == MF_BF16) && H % 8 == 0 && H <= 8 * 256 * 4 &&
      (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15) == 0) {
    const __nv_bfloat16* d = (const __nv_bfloat16*)delta;
    __nv_bfloat16* o = (__nv_bfloat16*)out;
    if (H <= 2048)
      return (int)launch_dep(add_rmsnorm_bf16_vec_kernel<1>, dim3(n_rows), dim3(256), 0, stream, resid, d, w, eps, o,
                             rows, H);
    if (H <= 4096)
      return (int)launch_dep(add_rmsnorm_bf16_vec_kernel<2>, dim3(n_rows), dim3(256), 0, stream, resid, d, w, eps, o,
                             rows, H);
    return (int)launch_dep(add_rmsnorm_bf16_vec_kernel<4>, dim3(n_rows), dim3(256), 0, stream, resid, d, w, eps, o,
                           rows, H);
  }
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

// The serving case: bfloat16, rot_dim a multiple of 16, head_dim a multiple of 8.  The
// cosines and sines of the token's position are computed once (float32, accurate sincosf)
// and shared by all heads; rows move in 16-byte pieces.
__global__ void __launch_bounds__(256)
rope_kv_write_bf16_vec_kernel(const __nv_bfloat16* __restrict__ qkv, int n_heads, int n_kv, int hd, int rot,
                              const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                              PagedView pv, const float* __restrict__ freqs, __nv_bfloat16* __restrict__ q_out,
                              __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                              int write_kv) {
  extern __shared__ float cs[];            // [half] cos, [half] sin
  pdl_launch();              // the attention after this one fetches older keys and values meanwhile
  // positions and the frequency table are in place before the step's first kernel starts and do not
  // change during it: the angles are computed before the wait, off the path between two kernels
  const int t = blockIdx.x;
  const int pos = positions[t], seq = seq_of_token[t];
  const int half = rot >> 1;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s, c;
    sincosf((float)pos / freqs[j], &s, &c);
    cs[j] = c;
    cs[half + j] = s;
  }
  __syncthreads();
  pdl_wait();
  const int width = (n_heads + 2 * n_kv) * hd;
  const __nv_bfloat16* row = qkv + (long long)t * width;
  const int rc = half >> 3;                // 16-byte pieces of rotated pairs per head
  const int pc = (hd - rot) >> 3;          // pass-through pieces per head
  const int per_head = rc + pc;
  const int n_rot_heads = n_heads + (write_kv ? n_kv : 0);
  for (int idx = threadIdx.x; idx < n_rot_heads * per_head; idx += blockDim.x) {
    const int h = idx / per_head, c = idx - h * per_head;
    const __nv_bfloat16* src = row + (long long)h * hd;
    __nv_bfloat16* dst = h < n_heads ? q_out + ((long long)t * n_heads + h) * hd
                                     : k_pool + paged_offset(pv, seq, pos, h - n_heads);
    if (c < rc) {
      const int j = c * 8;
      const uint4 a = *reinterpret_cast<const uint4*>(src + j), b = *reinterpret_cast<const uint4*>(src + j + half);
      const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
      uint4 oa, ob;
      __nv_bfloat162* oap = reinterpret_cast<__nv_bfloat162*>(&oa);
      __nv_bfloat162* obp = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float2 x1 = __bfloat1622float2(ap[e]), x2 = __bfloat1622float2(bp[e]);
        const float c0 = cs[j + 2 * e], c1 = cs[j + 2 * e + 1];
        const float s0 = cs[half + j + 2 * e], s1 = cs[half + j + 2 * e + 1];
        oap[e] = __floats2bfloat162_rn(x1.x * c0 - x2.x * s0, x1.y * c1 - x2.y * s1);
        obp[e] = __floats2bfloat162_rn(x1.x * s0 + x2.x * c0, x1.y * s1 + x2.y * c1);
      }
      *reinterpret_cast<uint4*>(dst + j) = oa;
      *reinterpret_cast<uint4*>(dst + j + half) = ob;
    } else {
      const int ch = rot + (c - rc) * 8;
      *reinterpret_cast<uint4*>(dst + ch) = *reinterpret_cast<const uint4*>(src + ch);
    }
  }
  if (write_kv) {
    const int vc = hd >> 3;
    for (int idx = threadIdx.x; idx < n_kv * vc; idx += blockDim.x) {
      const int h = idx / vc, c = idx - h * vc;
      *reinterpret_cast<uint4*>(v_pool + paged_offset(pv, seq, pos, h) + c * 8) =
          *reinterpret_cast<const uint4*>(row + (long long)(n_heads + n_kv + h) * hd + c * 8);
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
  if (dtype == MF_BF16 && !precise && rot_dim % 16 == 0 && hd % 8 == 0 &&
      (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0) {
    return (int)launch_dep(rope_kv_write_bf16_vec_kernel, dim3(T), dim3(256), (size_t)rot_dim * sizeof(float), stream,
                           (const __nv_bfloat16*)qkv, n_heads, n_kv, hd, rot_dim, positions, seq_of_token, pv, freqs,
                           (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, write_kv);
  }
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

// bfloat16 with groups of 8: 16 bytes of gate, 16 bytes of up, 16 bytes out per thread
__global__ void swiglu_bf16_g8_kernel(const uint4* __restrict__ gu, uint4* __restrict__ out, long long n_groups) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_groups) return;
  const uint4 gv = gu[2 * idx], uv = gu[2 * idx + 1];
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
  uint4 pk;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
  for (int e = 0; e < 4; e++) {
    const float2 g = __bfloat1622float2(gp[e]), u = __bfloat1622float2(up[e]);
    p[e] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
  }
  out[idx] = pk;
}

MF_API int mf_swiglu(const void* gu, void* out, int dtype, int T, int I, int group, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (group <= 0 || I % group) return MF_ERR_BAD_ARG;
  if (dtype == MF_BF16 && group == 8 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
    const long long n_groups = (long long)T * (I / 8);
    swiglu_bf16_g8_kernel<<<(unsigned)((n_groups + 255) / 256), 256, 0, stream>>>((const uint4*)gu, (uint4*)out,
                                                                                    n_groups);
    return (int)cudaGetLastError();
  }
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
