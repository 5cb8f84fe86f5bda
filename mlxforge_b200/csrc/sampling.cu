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

MF_API int mf_sample(const float* logits, int n, int V, long long row_stride, const float* temperature,
                     const float* u, int* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0) return MF_ERR_BAD_ARG;
  sample_kernel<<<n, SAMPLE_THREADS, 0, stream>>>(logits, V, row_stride, temperature, u, out);
  return (int)cudaGetLastError();
}
