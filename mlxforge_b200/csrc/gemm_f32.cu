// C[M,N] = A[M,K] * W[N,K]^T in IEEE float32 on the CUDA cores: no tensor
// cores, no TF32.  This is the matrix product of the 32-bit model path (the
// reference has no such path; its products are fp16 `mx::matmul`,
// src/model/decoder_model.cpp:174-192).  Each output element is one serial FMA
// chain over k in increasing order, so its value does not depend on M, on the
// tile it falls in or on what else is in the batch.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16
#define TM 4
#define TN 4

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int accumulate) {
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[BK][BN + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k per operand = 1024 elements, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int e = threadIdx.x + i * 256;
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? A[(long long)gm * K + gk] : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? W[(long long)gn * K + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; j++) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; i++) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; j++) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float* c = C + (long long)gm * N + gn;
      *c = accumulate ? (*c + acc[i][j]) : acc[i][j];
    }
  }
}

MF_API int mf_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K, int accumulate,
                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return MF_ERR_BAD_ARG;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return MF_ERR_BAD_ARG;
  mf_count(MF_K_GEMM_F32);
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, W, C, M, N, K, accumulate);
  return (int)cudaGetLastError();
}
