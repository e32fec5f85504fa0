// True 32-bit matrix product for the verification path: C[M,N] = A[M,K] * W[N,K]^T (+ bias).
// Plain FFMA on CUDA cores: no tensor-core instruction is issued, so no operand is
// ever rounded to TF32 or bfloat16.  Every output element accumulates k = 0..K-1 in
// ascending order in one thread, so a row's result does not depend on how many other
// rows are in the batch (nn.Linear layout, mini_llm/nn/attention.py:102-111).
#include "common.cuh"

namespace b200 {

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                const float* __restrict__ bias, float* __restrict__ C, int M, int N, int K,
                int lda, int ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 4 x 4 outputs
  float acc[4][4] = {};
  // each thread loads 4 consecutive k of one row for A and for W
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + i][lrow] = (am < M && k < K) ? A[static_cast<size_t>(am) * lda + k] : 0.f;
      Ws[lk + i][lrow] = (wn < N && k < K) ? W[static_cast<size_t>(wn) * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
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
      if (n < N) C[static_cast<size_t>(m) * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

}  // namespace b200

extern "C" int b200_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M,
                             int N, int K, int lda, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldc < N) return B200_ERR_BAD_SIZE;
  dim3 grid((N + b200::BN - 1) / b200::BN, (M + b200::BM - 1) / b200::BM);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  b200::launch(b200::gemm_f32_kernel, dim3(grid), dim3(256), 0, stream, A, W, bias, C, M, N, K, lda, ldc);
  return b200::launch_status();
}
