// C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]) in true 32-bit: plain FMA on the CUDA cores, no tensor
// cores and no reduced-precision matrix mode.  This is the matrix product of the 32-bit path
// (the reference's tested path is float32 end to end, src/qwen25vl_lite/engine.py:63).
//
// Every output element is one chain acc = fma(a[m,k], w[n,k], acc) over k = 0 .. K-1 in order,
// then + bias.  The chain does not depend on the tile shape or on M, so a token's result is
// bit-identical whether it is computed alone, in a portion or in a large batch.
#include "common.cuh"

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
  pdl_trigger();
  pdl_wait();
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = threadIdx.x; e < BM * BK; e += THREADS) {
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
    }
    for (int e = threadIdx.x; e < BN * BK; e += THREADS) {
      const int r = e / BK, c = e % BK;
      const int gn = n0 + r, gk = k0 + c;
      Ws[c][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
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
      if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
    }
  }
}

// The zero padding of the K tail adds fma(0, 0, acc) = acc, which leaves the chain unchanged.
Q25_EXPORT int q25_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K, int lda,
                            int ldw, int ldc, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (M <= 16) {
    dim3 grid((N + 63) / 64, (M + 15) / 16);
    launch(gemm_f32_kernel<16, 64, 16, 1, 4>, dim3(grid), dim3(256), 0, s, A, W, bias, C, M, N, K, lda, ldw, ldc);
  } else {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    launch(gemm_f32_kernel<64, 64, 16, 4, 4>, dim3(grid), dim3(256), 0, s, A, W, bias, C, M, N, K, lda, ldw, ldc);
  }
  return launch_status();
}
