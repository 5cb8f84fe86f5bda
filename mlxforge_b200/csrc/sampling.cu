// Token selection on the device from float32 logits [n, V]: greedy argmax (ties to
// the lowest index) and temperature sampling by inverse CDF in index order with
// one uniform number per row supplied by the caller.
//
// Reference (hvasconcelos/mlxforge): greedy src/sample/sampler.cpp:59-61;
// temperature `logits / T` then a categorical draw :156-165; temperature <= 0 is
// greedy.  The reference draws with MLX's generator; here the draw is a function
// of (seed, output index) computed by the caller, so a stream of tokens can be
// reproduced on the host.
#include "common.cuh"

#define SAMPLE_THREADS 1024

// One block per row.  Row parameters: temperature[r] (<= 0 -> greedy), u[r] in [0,1).
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, long long row_stride,
              const float* __restrict__ temperature, const float* __restrict__ u, int* __restrict__ out) {
  __shared__ float red[32];
  __shared__ float sval[SAMPLE_THREADS];
  __shared__ int sidx[SAMPLE_THREADS];
  __shared__ float warp_tot[32];
  __shared__ int winner;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (long long)r * row_stride;
  const float temp = temperature ? temperature[r] : 0.f;

  // ---- max and argmax (lowest index among equals)
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < V; i += SAMPLE_THREADS) {
    const float v = x[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  sval[tid] = best;
  sidx[tid] = best_i;
  __syncthreads();
  for (int s = SAMPLE_THREADS / 2; s > 0; s >>= 1) {
    if (tid < s) {
      const float v = sval[tid + s];
      const int i = sidx[tid + s];
      if (v > sval[tid] || (v == sval[tid] && i < sidx[tid])) { sval[tid] = v; sidx[tid] = i; }
    }
    __syncthreads();
  }
  const float mx = sval[0];
  const int amax = sidx[0];
  if (!(temp > 0.f) || !isfinite(temp)) {
    if (tid == 0) out[r] = amax;
    return;
  }

  // ---- inverse CDF over contiguous per-thread segments
  const int seg = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int begin = min(V, tid * seg), end = min(V, begin + seg);
  const float inv_t = 1.0f / temp;
  float part = 0.f;
  for (int i = begin; i < end; i++) part += expf((x[i] - mx) * inv_t);
  // exclusive scan of `part` over the block: warp scan, then scan of warp totals
  const int lane = tid & 31, warp = tid >> 5;
  float incl = part;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float nb = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += nb;
  }
  if (lane == 31) warp_tot[warp] = incl;
  if (tid == 0) winner = -1;
  __syncthreads();
  if (warp == 0) {
    float w = warp_tot[lane];
    float wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float nb = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += nb;
    }
    warp_tot[lane] = wi - w;              // exclusive prefix of warp totals
    if (lane == 31) red[0] = wi;          // total
  }
  __syncthreads();
  const float total = red[0];
  const float excl = warp_tot[warp] + (incl - part);
  const float target = u[r] * total;
  // The winner is the last thread with mass whose segment starts at or before the
  // target.  (The first thread with mass starts at 0, so there always is one; a test
  // on both ends of the segment could match none or two threads after rounding.)
  if (part > 0.f && excl <= target) atomicMax(&winner, tid);
  __syncthreads();
  if (tid == winner) {
    float c = excl;
    int pick = -1, last = begin;
    for (int i = begin; i < end; i++) {
      const float e = expf((x[i] - mx) * inv_t);
      if (e > 0.f) last = i;
      c += e;
      if (c > target) { pick = i; break; }
    }
    out[r] = pick >= 0 ? pick : last;
  }
}

// Greedy rows of a large vocabulary: one block per row would read half a megabyte through one
// SM, so ARGMAX_PARTS blocks take a part of the row each and one more kernel picks among their
// results (lowest index among equals, as above).  The partial results live in an array of the
// library: launches of different streams must not overlap (the engine has one stream).
#define ARGMAX_PARTS 16
#define ARGMAX_MAX_ROWS 4096
__device__ float g_part_val[ARGMAX_MAX_ROWS * ARGMAX_PARTS];
__device__ int g_part_idx[ARGMAX_MAX_ROWS * ARGMAX_PARTS];

__global__ void __launch_bounds__(256)
argmax_part_kernel(const float* __restrict__ logits, int V, long long row_stride) {
  __shared__ float sval[8];
  __shared__ int sidx[8];
  const int r = blockIdx.y, part = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (long long)r * row_stride;
  const int per = (V + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
  const int begin = min(V, part * per), end = min(V, begin + per);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = begin + tid; i < end; i += 256) {          // ascending per thread: the first of equals stays
    const float v = x[i];
    if (v > best) { best = v; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v = __shfl_xor_sync(0xffffffffu, best, o);
    const int i = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  if ((tid & 31) == 0) { sval[tid >> 5] = best; sidx[tid >> 5] = best_i; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 8; w++)
      if (sval[w] > best || (sval[w] == best && sidx[w] < best_i)) { best = sval[w]; best_i = sidx[w]; }
    g_part_val[r * ARGMAX_PARTS + part] = best;
    g_part_idx[r * ARGMAX_PARTS + part] = best_i;
  }
}

__global__ void argmax_pick_kernel(int n, int* __restrict__ out) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int p = 0; p < ARGMAX_PARTS; p++) {
    const float v = g_part_val[r * ARGMAX_PARTS + p];
    const int i = g_part_idx[r * ARGMAX_PARTS + p];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  out[r] = best_i == 0x7fffffff ? 0 : best_i;          // a row of -inf: token 0, as the one-block kernel gives
}

MF_API int mf_sample(const float* logits, int n, int V, long long row_stride, const float* temperature,
                     const float* u, int* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0) return MF_ERR_BAD_ARG;
  if (temperature == nullptr && V >= 16384 && n <= ARGMAX_MAX_ROWS) {
    argmax_part_kernel<<<dim3(ARGMAX_PARTS, n), 256, 0, stream>>>(logits, V, row_stride);
    argmax_pick_kernel<<<(n + 127) / 128, 128, 0, stream>>>(n, out);
    return (int)cudaGetLastError();
  }
  sample_kernel<<<n, SAMPLE_THREADS, 0, stream>>>(logits, V, row_stride, temperature, u, out);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ penalties
// Row r owns unique history ids[off[r] .. off[r+1]) with their counts.  For a seen
// token: repetition divides a positive logit and multiplies a negative one, then
// frequency subtracts penalty * count and presence subtracts penalty once
// (src/sample/sampler.cpp:95-135).
__global__ void penalties_kernel(float* __restrict__ logits, long long row_stride, const int* __restrict__ ids,
                                 const int* __restrict__ counts, const int* __restrict__ off,
                                 const float* __restrict__ rep, const float* __restrict__ freq,
                                 const float* __restrict__ pres) {
  const int r = blockIdx.x;
  float* x = logits + (long long)r * row_stride;
  const float rp = rep[r], fq = freq[r], pr = pres[r];
  for (int i = off[r] + threadIdx.x; i < off[r + 1]; i += blockDim.x) {
    const int id = ids[i];
    float v = x[id];
    if (rp != 1.0f) v = v > 0.f ? v / rp : v * rp;
    v -= fq * (float)counts[i];
    v -= pr;
    x[id] = v;
  }
}

MF_API int mf_apply_penalties(float* logits, int n, long long row_stride, const int* ids, const int* counts,
                              const int* off, const float* rep, const float* freq, const float* pres,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  penalties_kernel<<<n, 256, 0, stream>>>(logits, row_stride, ids, counts, off, rep, freq, pres);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ top-k / top-p / min-p
// In place: removed entries become -inf.  Applied to logits / temperature in the
// reference's order (src/sample/sampler.cpp:63-93,159-163): top-k keeps values >= the
// k-th largest; top-p keeps the shortest prefix in descending order whose
// probability reaches p (a token stays while the mass before it is < p); min-p
// keeps probabilities >= min_p * the largest.  Thresholds are found by an 8-bit
// radix descent over an order-preserving integer image of the floats; entries
// equal to a threshold are all kept.
__device__ __forceinline__ unsigned ordered_key(float f) {
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(unsigned k) {
  const unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
filter_kernel(float* __restrict__ logits, int V, long long row_stride, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p) {
  __shared__ float red[32];
  __shared__ unsigned hist_n[256];
  __shared__ float hist_m[256];
  __shared__ unsigned s_prefix;
  __shared__ unsigned s_remaining;
  __shared__ float s_acc;
  const int r = blockIdx.x, tid = threadIdx.x;
  float* x = logits + (long long)r * row_stride;
  const float temp = temperature[r];
  if (!(temp > 0.f) || !isfinite(temp)) return;     // greedy rows are not filtered
  const float inv_t = 1.0f / temp;
  const int k = top_k[r];
  const float p = top_p[r], mp = min_p[r];

  // ---- top-k: the k-th largest value by radix select on counts
  if (k > 0 && k < V) {
    if (tid == 0) { s_prefix = 0u; s_remaining = (unsigned)k; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < 256; b += SAMPLE_THREADS) hist_n[b] = 0u;
      __syncthreads();
      const unsigned prefix = s_prefix;
      const unsigned himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const unsigned key = ordered_key(x[i]);
        if ((key & himask) == prefix) atomicAdd(&hist_n[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned rem = s_remaining;
        int b = 255;
        for (; b > 0; b--) {
          if (hist_n[b] >= rem) break;
          rem -= hist_n[b];
        }
        s_prefix = prefix | ((unsigned)b << shift);
        s_remaining = rem;
      }
      __syncthreads();
    }
    const float kth = key_to_float(s_prefix);
    for (int i = tid; i < V; i += SAMPLE_THREADS)
      if (x[i] < kth) x[i] = -INFINITY;
    __syncthreads();
  }

  if (!(p < 1.0f) && !(mp > 0.f)) return;
  // ---- max and normaliser of softmax(x / T) over what is left
  float mx = -INFINITY;
  for (int i = tid; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, x[i]);
  mx = block_max(mx, red);
  if (p < 1.0f) {
    float z = 0.f;
    for (int i = tid; i < V; i += SAMPLE_THREADS) z += expf((x[i] - mx) * inv_t);
    z = block_sum(z, red);
    const float target = p * z;
    if (tid == 0) { s_prefix = 0u; s_acc = 0.f; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < 256; b += SAMPLE_THREADS) hist_m[b] = 0.f;
      __syncthreads();
      const unsigned prefix = s_prefix;
      const unsigned himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = x[i];
        const unsigned key = ordered_key(v);
        if ((key & himask) == prefix) atomicAdd(&hist_m[(key >> shift) & 255u], expf((v - mx) * inv_t));
      }
      __syncthreads();
      if (tid == 0) {
        float acc = s_acc;       // mass of everything strictly above the current prefix range
        int b = 255;
        for (; b > 0; b--) {
          if (acc + hist_m[b] >= target) break;
          acc += hist_m[b];
        }
        s_prefix = prefix | ((unsigned)b << shift);
        s_acc = acc;
      }
      __syncthreads();
    }
    const float cut = key_to_float(s_prefix);
    for (int i = tid; i < V; i += SAMPLE_THREADS)
      if (x[i] < cut) x[i] = -INFINITY;
    __syncthreads();
  }
  if (mp > 0.f) {
    for (int i = tid; i < V; i += SAMPLE_THREADS)
      if (expf((x[i] - mx) * inv_t) < mp) x[i] = -INFINITY;
  }
}

MF_API int mf_filter_logits(float* logits, int n, int V, long long row_stride, const float* temperature,
                            const int* top_k, const float* top_p, const float* min_p, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0) return MF_ERR_BAD_ARG;
  filter_kernel<<<n, SAMPLE_THREADS, 0, stream>>>(logits, V, row_stride, temperature, top_k, top_p, min_p);
  return (int)cudaGetLastError();
}
