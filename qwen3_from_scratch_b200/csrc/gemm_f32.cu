// True float32 matrix product for the 32-bit path of the model:
//   C[M, N] = A[M, K] * W[N, K]^T      (the layout of a Linear weight: y = x W^T)
// Plain FFMA on CUDA cores: no tensor cores, no TF32, no split-K.  Every output
// element is the sum over k = 0..K-1 in ascending order, accumulated in one
// register, so a row's result does not depend on M or on the rest of the batch.
// This is the slow, checkable path; the serving path uses tensor cores.
#include "common.cuh"

namespace q3 {

constexpr int GF_BM = 64, GF_BN = 64, GF_BK = 16, GF_THREADS = 256;

__global__ void __launch_bounds__(GF_THREADS)
gemm_f32_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                   int M, int N, int K, int lda, int ldw, int ldc) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float As[GF_BK][GF_BM + 4];
  __shared__ float Ws[GF_BK][GF_BN + 4];
  const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // each thread stages 4 elements of each tile: tile row = e / BK, tile col = e % BK
  for (int k0 = 0; k0 < K; k0 += GF_BK) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int e = threadIdx.x + p * GF_THREADS;
      const int r = e / GF_BK, c = e % GF_BK;
      const int k = k0 + c;
      const int am = m0 + r, wn = n0 + r;
      As[c][r] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[c][r] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GF_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

}  // namespace q3

// C[M, N] = A[M, K] * W[N, K]^T, all float32, row pitches lda / ldw / ldc in elements.
extern "C" int q3_gemm_f32_nt(const float* A, const float* W, float* C, int M, int N, int K, int lda,
                              int ldw, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return Q3_ERR_SIZE;
  dim3 grid((N + q3::GF_BN - 1) / q3::GF_BN, (M + q3::GF_BM - 1) / q3::GF_BM);
  if (grid.y > 65535) return Q3_ERR_SIZE;
  q3::launch(q3::gemm_f32_nt_kernel, dim3(grid), dim3(q3::GF_THREADS), 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
  return q3::launch_status();
}
