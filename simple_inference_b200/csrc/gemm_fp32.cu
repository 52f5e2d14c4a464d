// True float32 matrix product on the CUDA cores: C[M,N] = A[M,K] * W[N,K]^T.
//
// This is the matrix product of the 32-bit path.  It uses FMA in float32 only
// (no TF32, no reduced-precision tensor-core mode), and every output element is
// the sum over k = 0..K-1 in that order in one thread, so a row's result does
// not depend on how many other rows are in the batch.  The reference's linear
// layers are torch F.linear calls (ops/attention.py:128-130,226;
// ops/mlp.py:117,128; ops/embedding.py:92).
//
// Both operands are K-contiguous (the nn.Linear weight layout [out, in]).
// A may have a row stride larger than K (lda), C a row stride ldc.
#include "common.cuh"

namespace si {

constexpr int BM = 64, BN = 64, BK = 16;
constexpr int TM = 4, TN = 4;  // per-thread tile; 16 x 16 threads

__global__ void __launch_bounds__(256)
gemm_fp32_tn_kernel(const float* __restrict__ A, const float* __restrict__ W,
                    float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
  __shared__ float sA[BK][BM + 4];
  __shared__ float sW[BK][BN + 4];
  pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  // each thread loads 4 elements of A and 4 of W per k-tile: 64 rows x 16 k
  const int lrow = tid >> 2;        // 0..63
  const int lk = (tid & 3) * 4;     // 0,4,8,12

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lrow, wn = n0 + lrow;
      sA[lk + j][lrow] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.0f;
      sW[lk + j][lrow] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = sA[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = sW[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
  pdl_trigger();
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

}  // namespace si

SI_API int si_gemm_fp32_tn(const float* A, const float* W, float* C, int M, int N, int K, int lda,
                           int ldw, int ldc, cudaStream_t stream) {
  if (!A || !W || !C || M < 0 || N <= 0 || K <= 0 || lda < K || ldw < K || ldc < N)
    return SI_ERR_ARG;
  if (M == 0) return SI_OK;
  dim3 grid((N + si::BN - 1) / si::BN, (M + si::BM - 1) / si::BM);
  if (grid.y > 65535) return SI_ERR_TOO_LARGE;
  SI_LAUNCH(si::gemm_fp32_tn_kernel, grid, 256, 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
  return SI_OK;
}
