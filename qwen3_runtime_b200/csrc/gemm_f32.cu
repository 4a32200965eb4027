// C[M, N] = A[M, K] * W[N, K]^T in true fp32 on the FMA pipes: no tensor cores, no
// TF32.  Every output element is one accumulator that takes its K products in
// ascending k order, so a row of C does not depend on M, on the tile shape chosen
// for M, or on where the row sits in the batch.  This is the matrix product of the
// engine's 32-bit path (the reference's fp32 path is torch on the CPU,
// qwen3_runtime/engine/factory.py:136-137).
#include "common.cuh"

template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_f32_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                float* __restrict__ C, int ldc, int M, int N, int K) {
  constexpr int BK = 16;
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = tid; e < BM * BK; e += THREADS) {
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? A[(long)gm * lda + gk] : 0.f;
    }
    for (int e = tid; e < BN * BK; e += THREADS) {
      const int r = e / BK, c = e % BK;
      const int gn = n0 + r, gk = k0 + c;
      Ws[c][r] = (gn < N && gk < K) ? W[(long)gn * ldw + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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
      if (gn < N) C[(long)gm * ldc + gn] = acc[i][j];
    }
  }
}

// Leading dimensions are in elements.  Zero products added for k >= K do not change
// an accumulator, so K need not be a multiple of the tile.
Q3_EXPORT int q3_gemm_f32(const float* A, int lda, const float* W, int ldw, float* C, int ldc, int M, int N,
                          int K, cudaStream_t stream) {
  if (!A || !W || !C || N < 1 || K < 1 || lda < K || ldw < K || ldc < N) return Q3_ERR_ARGUMENT;
  if (M == 0) return Q3_OK;
  if (M > 64) {
    dim3 grid((N + 127) / 128, (M + 127) / 128);
    if (grid.y > 65535) return Q3_ERR_UNSUPPORTED;
    gemm_f32_kernel<128, 128, 8, 8><<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
  } else {
    dim3 grid((N + 63) / 64, (M + 31) / 32);
    gemm_f32_kernel<32, 64, 2, 4><<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
  }
  return q3_launch_status();
}
