// Weight-streaming projection for a few tokens (decoding): C[M,N] = X[M,K] * W[N,K]^T (+ bias),
// M <= 16, bfloat16 operands, float32 accumulation.
//
// The product is bound by reading W once from HBM, so W never touches shared memory: each
// warp streams 16 rows of W straight into the A fragments of mma.sync.m16n8k16 with 16-byte
// loads, the tokens are the 8-wide N side, and X (a few KB, hot in L1) supplies the B
// fragments.  The K order inside a 32-element chunk is permuted identically for both
// operands (a dot product does not care), which is what lets every lane fetch 16
// contiguous bytes instead of 4.  The eight warps of a CTA split K between them in
// interleaved 512-byte pieces and add their partial tiles through shared memory in a fixed
// order: no atomics, no scratch memory, the same bits every run.
// nn.Linear layout, no transposition (mini_llm/nn/attention.py:102-111).
#include "common.cuh"
#include "mma.cuh"

namespace b200 {

constexpr int kChunk = 256;   // K elements one warp takes at a time (8 loads of 32 elements)

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int NT, int UNROLL, int kSkinnyWarps, bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ X,
                   const float* __restrict__ bias, OutT* __restrict__ C, int M, int N, int K, int ldc) {
  __shared__ float red[kSkinnyWarps][16][NT * 8 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const __nv_bfloat16* wa = W + static_cast<size_t>(min(n0 + g, N - 1)) * K + t * 8;
  const __nv_bfloat16* wb = W + static_cast<size_t>(min(n0 + g + 8, N - 1)) * K + t * 8;
  const __nv_bfloat16* xr[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) xr[j] = X + static_cast<size_t>(min(j * 8 + g, M - 1)) * K + t * 8;
  float c[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) c[j][e] = 0.f;

  const uint4 zero = make_uint4(0, 0, 0, 0);
  // The weights do not depend on the kernel before this one: fetch the first piece of them
  // while that kernel is still finishing, and only then wait for the activations.
  pdl_trigger();
  uint4 a[UNROLL], b[UNROLL];
  {
    const int k0 = warp * kChunk;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = k0 + u * 32;
      const bool ok = k + t * 8 < K;
      a[u] = ok ? ldg_stream(wa + k) : zero;
      b[u] = ok ? ldg_stream(wb + k) : zero;
    }
  }
  pdl_wait();
  for (int k0 = warp * kChunk; k0 < K; k0 += kSkinnyWarps * kChunk) {
#pragma unroll
    for (int h = 0; h < kChunk / 32; h += UNROLL) {
      uint4 x[NT][UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int k = k0 + (h + u) * 32;
        const bool ok = k + t * 8 < K;
        if (h != 0 || k0 != warp * kChunk) {   // the very first piece is already in registers
          a[u] = ok ? ldg_stream(wa + k) : zero;
          b[u] = ok ? ldg_stream(wb + k) : zero;
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) x[j][u] = ok ? *reinterpret_cast<const uint4*>(xr[j] + k) : zero;
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const uint32_t lo[4] = {a[u].x, b[u].x, a[u].y, b[u].y};
        const uint32_t hi[4] = {a[u].z, b[u].z, a[u].w, b[u].w};
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          mma_bf16(c[j], lo, x[j][u].x, x[j][u].y);
          mma_bf16(c[j], hi, x[j][u].z, x[j][u].w);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    red[warp][g][j * 8 + 2 * t] = c[j][0];
    red[warp][g][j * 8 + 2 * t + 1] = c[j][1];
    red[warp][g + 8][j * 8 + 2 * t] = c[j][2];
    red[warp][g + 8][j * 8 + 2 * t + 1] = c[j][3];
  }
  __syncthreads();
  if constexpr (SWIGLU) {
    // rows 0..7 of the tile are gate features, rows 8..15 the matching up features
    for (int idx = threadIdx.x; idx < 8 * NT * 8; idx += kSkinnyWarps * 32) {
      const int m = idx >> 3, f = idx & 7;
      const int n = n0 + f;                      // gate row in W; the output feature is n0 / 2 + f
      if (m >= M || n + 8 >= N) continue;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int w = 0; w < kSkinnyWarps; ++w) {
        gate += red[w][f][m];
        up += red[w][f + 8][m];
      }
      if (bias) {
        gate += bias[n];
        up += bias[n + 8];
      }
      C[static_cast<size_t>(m) * ldc + (n0 >> 1) + f] = from_float<OutT>(gate / (1.f + expf(-gate)) * up);
    }
  } else {
    for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += kSkinnyWarps * 32) {
      const int m = idx >> 4, row = idx & 15;   // consecutive threads -> consecutive output features
      const int n = n0 + row;
      if (m >= M || n >= N) continue;
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < kSkinnyWarps; ++w) acc += red[w][row][m];
      acc += bias ? bias[n] : 0.f;
      C[static_cast<size_t>(m) * ldc + n] = from_float<OutT>(acc);
    }
  }
}

}  // namespace b200

using namespace b200;

// M <= 16, K a multiple of 8, W and X 16-byte aligned; otherwise refused.
template <int NT, int UNROLL, int WARPS>
static void launch_skinny(const __nv_bfloat16* w, const __nv_bfloat16* x, const float* bias, void* C, int M, int N, int K,
                          int ldc, int out_f32, int swiglu, cudaStream_t stream) {
  const int grid = (N + 15) / 16;
  if (swiglu) {
    if (out_f32)
      launch(gemm_skinny_kernel<NT, UNROLL, WARPS, true, float>, dim3(grid), dim3(WARPS * 32), 0, stream, w, x, bias,
             static_cast<float*>(C), M, N, K, ldc);
    else
      launch(gemm_skinny_kernel<NT, UNROLL, WARPS, true, __nv_bfloat16>, dim3(grid), dim3(WARPS * 32), 0, stream, w, x, bias,
             static_cast<__nv_bfloat16*>(C), M, N, K, ldc);
    return;
  }
  if (out_f32)
    launch(gemm_skinny_kernel<NT, UNROLL, WARPS, false, float>, dim3(grid), dim3(WARPS * 32), 0, stream, w, x, bias,
           static_cast<float*>(C), M, N, K, ldc);
  else
    launch(gemm_skinny_kernel<NT, UNROLL, WARPS, false, __nv_bfloat16>, dim3(grid), dim3(WARPS * 32), 0, stream, w, x, bias,
           static_cast<__nv_bfloat16*>(C), M, N, K, ldc);
}

// M <= 16, K a multiple of 8, W and X 16-byte aligned; otherwise refused.
// `variant` picks the shape of a CTA (0: the default for the size; 1..3: experiments).
// `swiglu` = 1: W holds gate and up rows interleaved in blocks of eight (N a multiple of 16);
// the output is silu(gate) * up, N / 2 columns wide (ldc >= N / 2).
extern "C" int b200_gemm_skinny_variant(const void* X, const void* W, const float* bias, void* C, int M, int N, int K,
                                        int ldc, int out_f32, int variant, int swiglu, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 8 != 0 || ldc < (swiglu ? N / 2 : N)) return B200_ERR_BAD_SIZE;
  if (swiglu && N % 16 != 0) return B200_ERR_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) & 15) return B200_ERR_BAD_SIZE;
  const auto* w = static_cast<const __nv_bfloat16*>(W);
  const auto* x = static_cast<const __nv_bfloat16*>(X);
  if (variant == 0) {
    // With fewer loads in flight per thread a CTA needs fewer registers and three fit on an SM
    // instead of two: that pays when it lets all CTAs be resident at once (measured on the
    // 6144 x 4096 projection: 13.2 -> 10.4 us), and costs otherwise.
    const int ctas = (N + 15) / 16;
    static DeviceOnce once;
    int sms = 0;
    if (int e = configure_once(once, gemm_skinny_kernel<1, 8, 8, false, float>, 0, &sms)) return e;
    if (ctas > 2 * sms && ctas <= 3 * sms) variant = 2;
  }
  if (M <= 8) {
    switch (variant) {
      case 1: launch_skinny<1, 8, 4>(w, x, bias, C, M, N, K, ldc, out_f32, swiglu, stream); break;
      case 2: launch_skinny<1, 4, 8>(w, x, bias, C, M, N, K, ldc, out_f32, swiglu, stream); break;
      case 3: launch_skinny<1, 4, 4>(w, x, bias, C, M, N, K, ldc, out_f32, swiglu, stream); break;
      default: launch_skinny<1, 8, 8>(w, x, bias, C, M, N, K, ldc, out_f32, swiglu, stream); break;
    }
  } else {
    switch (variant) {
      case 1: launch_skinny<2, 4, 4>(w, x, bias, C, M, N, K, ldc, out_f32, swiglu, stream); break;
      case 2: launch_skinny<2, 2, 8>(w, x, bias, C, M, N, K, ldc, out_f32, swiglu, stream); break;
      default: launch_skinny<2, 4, 8>(w, x, bias, C, M, N, K, ldc, out_f32, swiglu, stream); break;
    }
  }
  return launch_status();
}

extern "C" int b200_gemm_skinny(const void* X, const void* W, const float* bias, void* C, int M, int N, int K,
                                int ldc, int out_f32, cudaStream_t stream) {
  return b200_gemm_skinny_variant(X, W, bias, C, M, N, K, ldc, out_f32, 0, 0, stream);
}
