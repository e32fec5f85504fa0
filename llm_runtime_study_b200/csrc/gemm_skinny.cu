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
//
// Two fusions keep the RMS norms of a decode step out of kernels of their own
// (y = w * x * rsqrt(mean(x^2) + eps), mini_llm/nn/norm.py:42-46; h = r + f(x), mini_llm/model/qwen.py:67, 72):
//   * EPI_RESIDUAL: the product is added into the float32 residual rows in place; the same pass writes
//     the rows multiplied by the *next* norm's weight, rounded to bfloat16, and every CTA leaves the sum
//     of squares of its 16 columns of every row (`partials`, [CTAs][16 rows]).
//   * SCALED: the rows this kernel multiplies are such weighted, not yet normalised rows.  The factor
//     rsqrt(mean + eps) is one number per row and commutes with the product, so it is applied to the
//     accumulators instead: each CTA adds up the partial sums (fetched into shared memory by cp.async
//     behind the main loop, added in a fixed order) and scales its results.
// Rounding r * w to bfloat16 before the scale instead of after changes nothing in relative terms.
#include "common.cuh"
#include "mma.cuh"

namespace b200 {

constexpr int kChunk = 256;   // K elements one warp takes at a time (8 loads of 32 elements)

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

enum Epilogue : int { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESIDUAL = 2 };
constexpr int kMaxPartials = 512;   // CTAs of the kernel that left the partial sums of squares (its N / 16)

// What the two fusions need beyond the product itself.
struct NormFusion {
  const float* partials;      // SCALED: [num_partials][16] sums of squares of the rows being multiplied
  int num_partials;
  float eps;                  // SCALED: rows are scaled by rsqrt(sum / K + eps)
  const float* next_weight;   // EPI_RESIDUAL: weight of the norm that follows, [N]
  __nv_bfloat16* weighted;    // EPI_RESIDUAL: out, [M][N] = (residual + product) * next_weight
  float* partials_out;        // EPI_RESIDUAL: out, [gridDim.x][16]
};

template <int NT, int UNROLL, int kSkinnyWarps, int EPI, bool SCALED, typename OutT>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ X,
                   const float* __restrict__ bias, OutT* __restrict__ C, int M, int N, int K, int ldc, NormFusion fuse) {
  constexpr bool SWIGLU = EPI == EPI_SWIGLU;
  __shared__ float red[kSkinnyWarps][16][NT * 8 + 1];
  __shared__ __align__(16) float part[SCALED ? kMaxPartials : 1][16];
  __shared__ float slice_sum[SCALED ? kSkinnyWarps * 2 : 1][16];
  __shared__ float row_scale[16];
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
  if constexpr (SCALED) {
    // the partial sums of squares are needed only after the main loop: let them trickle into shared memory meanwhile
    for (int i = threadIdx.x; i < fuse.num_partials * 4; i += kSkinnyWarps * 32)
      cp_async_16(&part[0][0] + 4 * i, fuse.partials + 4 * i, 16);
    cp_async_commit();
  }
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
  if constexpr (SCALED) cp_async_wait<0>();
  __syncthreads();
  if constexpr (SCALED) {
    // rsqrt(mean of squares + eps) of every row: thread (row = t % 16, slice = t / 16) adds every
    // (threads / 16)-th partial sum, then one thread per row adds the slices; the order is fixed by the launch shape
    constexpr int kSlices = kSkinnyWarps * 2;
    const int r = threadIdx.x & 15, slice = threadIdx.x >> 4;
    float s = 0.f;
    for (int i = slice; i < fuse.num_partials; i += kSlices) s += part[i][r];
    slice_sum[slice][r] = s;
    __syncthreads();
    if (threadIdx.x < 16) {
      float total = 0.f;
#pragma unroll
      for (int i = 0; i < kSlices; ++i) total += slice_sum[i][threadIdx.x];
      row_scale[threadIdx.x] = rsqrtf(total / static_cast<float>(K) + fuse.eps);
    }
    __syncthreads();
  }
  if constexpr (EPI == EPI_RESIDUAL) {
    // C is the float32 residual stream: add the product in place, write the rows weighted for the next norm,
    // and leave this CTA's share of every row's sum of squares.  All lanes stay in the loop for the shuffles.
    float* resid = reinterpret_cast<float*>(C);
    for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += kSkinnyWarps * 32) {
      const int m = idx >> 4, row = idx & 15;
      const int n = n0 + row;
      const bool valid = m < M && n < N;
      float r = 0.f;
      if (valid) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < kSkinnyWarps; ++w) acc += red[w][row][m];
        acc += bias ? bias[n] : 0.f;
        r = resid[static_cast<size_t>(m) * ldc + n] + acc;
        resid[static_cast<size_t>(m) * ldc + n] = r;
        fuse.weighted[static_cast<size_t>(m) * N + n] = __float2bfloat16_rn(r * fuse.next_weight[n]);
      }
      float sq = r * r;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (row == 0) fuse.partials_out[static_cast<size_t>(blockIdx.x) * 16 + m] = sq;
    }
  } else if constexpr (SWIGLU) {
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
      if constexpr (SCALED) {
        gate *= row_scale[m];
        up *= row_scale[m];
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
      if constexpr (SCALED) acc *= row_scale[m];
      acc += bias ? bias[n] : 0.f;
      C[static_cast<size_t>(m) * ldc + n] = from_float<OutT>(acc);
    }
  }
}

}  // namespace b200

using namespace b200;

template <int NT, int UNROLL, int WARPS, int EPI, bool SCALED, typename OutT>
static void launch_one(const __nv_bfloat16* w, const __nv_bfloat16* x, const float* bias, void* C, int M, int N, int K,
                       int ldc, const NormFusion& fuse, cudaStream_t stream) {
  launch(gemm_skinny_kernel<NT, UNROLL, WARPS, EPI, SCALED, OutT>, dim3((N + 15) / 16), dim3(WARPS * 32), 0, stream, w, x,
         bias, static_cast<OutT*>(C), M, N, K, ldc, fuse);
}

// epi: 0 store, 1 SwiGLU, 2 add into the residual rows (C float32) and weight for the next norm
template <int NT, int UNROLL, int WARPS>
static void launch_skinny(const __nv_bfloat16* w, const __nv_bfloat16* x, const float* bias, void* C, int M, int N, int K,
                          int ldc, int out_f32, int epi, const NormFusion& fuse, cudaStream_t stream) {
  const bool scaled = fuse.partials != nullptr;
  if (epi == EPI_RESIDUAL) {
    launch_one<NT, UNROLL, WARPS, EPI_RESIDUAL, false, float>(w, x, bias, C, M, N, K, ldc, fuse, stream);
  } else if (epi == EPI_SWIGLU) {
    if (scaled) {
      if (out_f32) launch_one<NT, UNROLL, WARPS, EPI_SWIGLU, true, float>(w, x, bias, C, M, N, K, ldc, fuse, stream);
      else launch_one<NT, UNROLL, WARPS, EPI_SWIGLU, true, __nv_bfloat16>(w, x, bias, C, M, N, K, ldc, fuse, stream);
    } else {
      if (out_f32) launch_one<NT, UNROLL, WARPS, EPI_SWIGLU, false, float>(w, x, bias, C, M, N, K, ldc, fuse, stream);
      else launch_one<NT, UNROLL, WARPS, EPI_SWIGLU, false, __nv_bfloat16>(w, x, bias, C, M, N, K, ldc, fuse, stream);
    }
  } else {
    if (scaled) {
      if (out_f32) launch_one<NT, UNROLL, WARPS, EPI_STORE, true, float>(w, x, bias, C, M, N, K, ldc, fuse, stream);
      else launch_one<NT, UNROLL, WARPS, EPI_STORE, true, __nv_bfloat16>(w, x, bias, C, M, N, K, ldc, fuse, stream);
    } else {
      if (out_f32) launch_one<NT, UNROLL, WARPS, EPI_STORE, false, float>(w, x, bias, C, M, N, K, ldc, fuse, stream);
      else launch_one<NT, UNROLL, WARPS, EPI_STORE, false, __nv_bfloat16>(w, x, bias, C, M, N, K, ldc, fuse, stream);
    }
  }
}

static int skinny(const void* X, const void* W, const float* bias, void* C, int M, int N, int K, int ldc, int out_f32,
                  int variant, int epi, const NormFusion& fuse, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 8 != 0 || ldc < (epi == EPI_SWIGLU ? N / 2 : N)) return B200_ERR_BAD_SIZE;
  if (epi == EPI_SWIGLU && N % 16 != 0) return B200_ERR_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) & 15) return B200_ERR_BAD_SIZE;
  if (fuse.partials && (fuse.num_partials <= 0 || fuse.num_partials > kMaxPartials ||
                        (reinterpret_cast<uintptr_t>(fuse.partials) & 15)))
    return B200_ERR_BAD_SIZE;
  const auto* w = static_cast<const __nv_bfloat16*>(W);
  const auto* x = static_cast<const __nv_bfloat16*>(X);
  if (variant == 0) {
    // With fewer loads in flight per thread a CTA needs fewer registers and three fit on an SM
    // instead of two: that pays when it lets all CTAs be resident at once (measured on the
    // 6144 x 4096 projection: 13.2 -> 10.4 us), and costs otherwise.
    const int ctas = (N + 15) / 16;
    static DeviceOnce once;
    int sms = 0;
    if (int e = configure_once(once, gemm_skinny_kernel<1, 8, 8, EPI_STORE, false, float>, 0, &sms)) return e;
    if (ctas > 2 * sms && ctas <= 3 * sms) variant = 2;
  }
  if (M <= 8) {
    if (variant == 2) launch_skinny<1, 4, 8>(w, x, bias, C, M, N, K, ldc, out_f32, epi, fuse, stream);
    else launch_skinny<1, 8, 8>(w, x, bias, C, M, N, K, ldc, out_f32, epi, fuse, stream);
  } else {
    if (variant == 2) launch_skinny<2, 2, 8>(w, x, bias, C, M, N, K, ldc, out_f32, epi, fuse, stream);
    else launch_skinny<2, 4, 8>(w, x, bias, C, M, N, K, ldc, out_f32, epi, fuse, stream);
  }
  return launch_status();
}

// M <= 16, K a multiple of 8, W and X 16-byte aligned; otherwise refused.
// `variant` picks the shape of a CTA (0: the default for the size; 2: fewer loads in flight, more CTAs per SM).
// `swiglu` = 1: W holds gate and up rows interleaved in blocks of eight (N a multiple of 16);
// the output is silu(gate) * up, N / 2 columns wide (ldc >= N / 2).
// `partials` (optional, [num_partials][16] floats): X holds rows that still lack their factor
// rsqrt(sum of squares / K + eps), the sums of squares being the column sums of `partials`; the factor is
// applied to the product (before the bias).
extern "C" int b200_gemm_skinny_variant(const void* X, const void* W, const float* bias, void* C, int M, int N, int K,
                                        int ldc, int out_f32, int variant, int swiglu, const float* partials,
                                        int num_partials, float eps, cudaStream_t stream) {
  NormFusion fuse{};
  fuse.partials = partials;
  fuse.num_partials = num_partials;
  fuse.eps = eps;
  return skinny(X, W, bias, C, M, N, K, ldc, out_f32, variant, swiglu ? EPI_SWIGLU : EPI_STORE, fuse, stream);
}

extern "C" int b200_gemm_skinny(const void* X, const void* W, const float* bias, void* C, int M, int N, int K,
                                int ldc, int out_f32, cudaStream_t stream) {
  return b200_gemm_skinny_variant(X, W, bias, C, M, N, K, ldc, out_f32, 0, 0, nullptr, 0, 0.f, stream);
}

// resid[M][N] (float32, row stride ldc) += X W^T (+ bias); weighted[M][N] (bfloat16) = resid * next_weight;
// partials_out[(N + 15) / 16][16] = per CTA, the sum of squares of its 16 columns of every row of the new resid.
// N / 16 (rounded up) may not exceed b200_gemm_skinny_max_partials() if a SCALED product is to consume them.
extern "C" int b200_gemm_skinny_residual(const void* X, const void* W, const float* bias, float* resid, int M, int N, int K,
                                         int ldc, const float* next_weight, void* weighted, float* partials_out,
                                         cudaStream_t stream) {
  if (!resid || !next_weight || !weighted || !partials_out) return B200_ERR_BAD_SIZE;
  NormFusion fuse{};
  fuse.next_weight = next_weight;
  fuse.weighted = static_cast<__nv_bfloat16*>(weighted);
  fuse.partials_out = partials_out;
  return skinny(X, W, bias, resid, M, N, K, ldc, 1, 0, EPI_RESIDUAL, fuse, stream);
}

extern "C" int b200_gemm_skinny_max_partials() { return kMaxPartials; }
