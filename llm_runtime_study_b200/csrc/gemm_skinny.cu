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
//     of squares of its 16 columns of every row in scratch memory ([CTAs][16 rows]).  A one-CTA kernel
//     behind it adds those up in CTA order and writes the rows' factors rsqrt(mean of squares + eps); it
//     releases the kernel after it at its first instruction, so the next projection fetches its first
//     weights meanwhile.  (Adding them up in every CTA of the consuming kernel, or in the producing
//     kernel's last CTA behind a ticket, cost 4 to 6 us per layer more: measured.)
//   * SCALED: the rows this kernel multiplies are such weighted, not yet normalised rows.  The factor
//     is one number per row and commutes with the product, so it is applied to the accumulators.
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

// What the two fusions need beyond the product itself.
struct NormFusion {
  const float* row_scale;     // SCALED: [16] factors the rows being multiplied still lack
  const float* next_weight;   // EPI_RESIDUAL: weight of the norm that follows, [N]
  float eps;                  // EPI_RESIDUAL: its eps
  __nv_bfloat16* weighted;    // EPI_RESIDUAL: out, [M][N] = (residual + product) * next_weight
  float* partials;            // EPI_RESIDUAL: out, [gridDim.x][16] sums of squares of the new residual rows, per CTA
};

template <int NT, int UNROLL, int kSkinnyWarps, int EPI, bool SCALED, typename OutT>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ X,
                   const float* __restrict__ bias, OutT* __restrict__ C, int M, int N, int K, int ldc, NormFusion fuse) {
  constexpr bool SWIGLU = EPI == EPI_SWIGLU;
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
      if (row == 0) fuse.partials[static_cast<size_t>(blockIdx.x) * 16 + m] = sq;
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
        gate *= fuse.row_scale[m];
        up *= fuse.row_scale[m];
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
      if constexpr (SCALED) acc *= fuse.row_scale[m];
      acc += bias ? bias[n] : 0.f;
      C[static_cast<size_t>(m) * ldc + n] = from_float<OutT>(acc);
    }
  }
}

// row_scale[r] = rsqrt(sum over CTAs of partials[cta][r] / width + eps) for the 16 rows: thread (row = t % 16,
// slice = t / 16) adds every 16th CTA's share, one thread per row adds the slices.  One CTA of 256 threads.
__global__ void __launch_bounds__(256) rms_finish_kernel(const float* __restrict__ partials, int ctas, int rows, float width,
                                                          float eps, float* __restrict__ row_scale) {
  __shared__ float slice_sum[16][16];
  pdl_launch_dependents();     // what follows is a projection: it may fetch its first weights while this runs
  pdl_wait();
  const int r = threadIdx.x & 15, slice = threadIdx.x >> 4;
  float s = 0.f;
  for (int i = slice; i < ctas; i += 16) s += partials[static_cast<size_t>(i) * 16 + r];
  slice_sum[slice][r] = s;
  __syncthreads();
  if (threadIdx.x < 16) {
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) total += slice_sum[i][threadIdx.x];
    row_scale[threadIdx.x] = static_cast<int>(threadIdx.x) < rows ? rsqrtf(total / width + eps) : 0.f;
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
  const bool scaled = fuse.row_scale != nullptr;
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
// `row_scale` (optional, 16 floats): X holds rows that still lack these factors (an RMS norm left half
// done); they are applied to the product, before the bias.
extern "C" int b200_gemm_skinny_variant(const void* X, const void* W, const float* bias, void* C, int M, int N, int K,
                                        int ldc, int out_f32, int variant, int swiglu, const float* row_scale,
                                        cudaStream_t stream) {
  NormFusion fuse{};
  fuse.row_scale = row_scale;
  return skinny(X, W, bias, C, M, N, K, ldc, out_f32, variant, swiglu ? EPI_SWIGLU : EPI_STORE, fuse, stream);
}

extern "C" int b200_gemm_skinny(const void* X, const void* W, const float* bias, void* C, int M, int N, int K,
                                int ldc, int out_f32, cudaStream_t stream) {
  return b200_gemm_skinny_variant(X, W, bias, C, M, N, K, ldc, out_f32, 0, 0, nullptr, stream);
}

// resid[M][N] (float32, row stride ldc) += X W^T (+ bias); weighted[M][N] (bfloat16) = resid * next_weight;
// row_scale_out[16] = rsqrt(mean of squares of each new row of resid + eps) (rows from M on: 0).
// `partials` is scratch of b200_gemm_skinny_partial_floats(N) floats.  Two launches.
extern "C" int b200_gemm_skinny_residual(const void* X, const void* W, const float* bias, float* resid, int M, int N, int K,
                                         int ldc, const float* next_weight, float eps, void* weighted, float* row_scale_out,
                                         float* partials, cudaStream_t stream) {
  if (!resid || !next_weight || !weighted || !row_scale_out || !partials) return B200_ERR_BAD_SIZE;
  NormFusion fuse{};
  fuse.next_weight = next_weight;
  fuse.eps = eps;
  fuse.weighted = static_cast<__nv_bfloat16*>(weighted);
  fuse.partials = partials;
  if (int e = skinny(X, W, bias, resid, M, N, K, ldc, 1, 0, EPI_RESIDUAL, fuse, stream)) return e;
  if (M <= 0 || N <= 0) return 0;
  launch(rms_finish_kernel, dim3(1), dim3(256), 0, stream, static_cast<const float*>(partials), (N + 15) / 16, M,
         static_cast<float>(N), eps, row_scale_out);
  return launch_status();
}

extern "C" long b200_gemm_skinny_partial_floats(int N) { return static_cast<long>((N + 15) / 16) * 16; }
