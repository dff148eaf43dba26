// True float32 matrix product for the 32-bit path: C[M, N] = A[M, K] * W[N, K]^T, FMA on the
// CUDA cores, no tensor cores and no reduced-precision mode anywhere. Every output element is
// accumulated over k = 0..K-1 in that order whatever the tile shape, M or N, so a row's result
// does not depend on which other rows share the launch.
#include "common.cuh"

namespace llmie {

constexpr int kBK = 16;

template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_f32_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C, int M, int N,
                   int K, int lda, int ldw, int ldc) {
  constexpr int kThreads = (BM / TM) * (BN / TN);
  __shared__ float As[kBK][BM + 4];
  __shared__ float Ws[kBK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kBK) {
    for (int idx = tid; idx < BM * kBK; idx += kThreads) {
      const int r = idx / kBK, c = idx % kBK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
    }
    for (int idx = tid; idx < BN * kBK; idx += kThreads) {
      const int r = idx / kBK, c = idx % kBK;
      const int gn = n0 + r, gk = k0 + c;
      Ws[c][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kBK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
    }
  }
}

}  // namespace llmie

using namespace llmie;

extern "C" int llmie_gemm_f32_nt(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw,
                                 int ldc, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || lda < K || ldw < K || ldc < N) return LLMIE_ERR_BAD_ARG;
  if (M == 0) return LLMIE_OK;
  if (M <= 16) {
    dim3 grid((N + 31) / 32, (M + 15) / 16);
    gemm_f32_nt_kernel<16, 32, 2, 2><<<grid, 128, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc);
  } else {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (grid.y > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
    gemm_f32_nt_kernel<64, 64, 4, 4><<<grid, 256, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc);
  }
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
