// Embedding gather, fused residual-add + RMSNorm, SiLU*mul, and the fused
// q/k-norm + rotary + paged K/V write.  One row (token) per thread block, so a
// token's arithmetic never depends on what else is in the batch.
//
// Formulas (reference, file:line):
//   embedding   h = E[token]                       mini_llm/model/base.py:72
//   RMSNorm     y = w * x * rsqrt(mean(x^2) + eps) mini_llm/nn/norm.py:42-46
//   residual    h = r + f(x)                       mini_llm/model/qwen.py:67,72
//   SwiGLU      m = silu(g) * u                    mini_llm/nn/mlp.py:86
//   rotary      x' = x*cos + rot(x)*sin, pairs (i, i+d/2), angle = pos * inv_freq[i]
//                                                  mini_llm/nn/rope.py:74-80,110-146
//   K/V write   page = table[pos / page_size], slot = pos % page_size
//                                                  mini_llm/cache/paged/store.py:51-60
#include "common.cuh"

namespace b200 {

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab, float scale) {
  pdl_trigger();
#ifdef B200_EARLY_EMBED
  pdl_launch_dependents();
#endif
  pdl_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  float* dst = out + static_cast<size_t>(row) * hidden;
  if (id < 0 || id >= vocab) {  // ids are validated on the host; never read out of range
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + static_cast<size_t>(id) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(src[i]) * scale;
}

// 16-byte loads of the table row, two 16-byte stores of floats per load
template <typename T>
__global__ void embedding_vec_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                     float* __restrict__ out, int hidden, int vocab, float scale) {
  constexpr int VN = Vec<T>::n;
  using V = typename Vec<T>::type;
  pdl_trigger();
#ifdef B200_EARLY_EMBED
  pdl_launch_dependents();
#endif
  pdl_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + static_cast<size_t>(ok ? id : 0) * hidden;
  float* dst = out + static_cast<size_t>(row) * hidden;
  for (int i = threadIdx.x * VN; i < hidden; i += blockDim.x * VN) {
    float f[VN];
    Vec<T>::unpack(*reinterpret_cast<const V*>(src + i), f);
#pragma unroll
    for (int e = 0; e < VN; e += 4)
      *reinterpret_cast<float4*>(dst + i + e) =
          ok ? make_float4(f[e] * scale, f[e + 1] * scale, f[e + 2] * scale, f[e + 3] * scale) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// The same gather for the first layer of a decode step of at most 16 tokens, which has no norm kernel of its
// own: besides the float32 row it writes the row multiplied by the first norm's weight, rounded to bfloat16,
// and the row's factor rsqrt(mean of squares + eps) (row_scale[row]), which the projection that follows
// applies to its accumulators (see gemm_skinny.cu).  16-byte loads of the table row, the row kept in registers.
template <typename T, int VPT>
__global__ void embedding_weighted_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                          const float* __restrict__ norm_weight, __nv_bfloat16* __restrict__ weighted,
                                          float* __restrict__ row_scale, int hidden, int vocab, float scale, float eps) {
  constexpr int VN = Vec<T>::n;
  using V = typename Vec<T>::type;
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + static_cast<size_t>(ok ? id : 0) * hidden;
  float x[VPT][VN];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = (threadIdx.x + v * blockDim.x) * VN;
#pragma unroll
    for (int e = 0; e < VN; ++e) x[v][e] = 0.f;
    if (i < hidden && ok) Vec<T>::unpack(*reinterpret_cast<const V*>(src + i), x[v]);
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      x[v][e] *= scale;
      ss += x[v][e] * x[v][e];
    }
  }
  const float total = block_sum(ss, scratch);
  if (threadIdx.x == 0) row_scale[row] = rsqrtf(total / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = (threadIdx.x + v * blockDim.x) * VN;
    if (i >= hidden) continue;
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      out[static_cast<size_t>(row) * hidden + i + e] = x[v][e];
      weighted[static_cast<size_t>(row) * hidden + i + e] = __float2bfloat16_rn(x[v][e] * norm_weight[i + e]);
    }
  }
}

// ------------------------------------------------- residual add + RMS norm
// x = resid[src] (+ delta[src]);  if write_resid: resid[src] = x
// out[row] = x * rsqrt(mean(x^2) + eps) * weight
// `rows` (optional) gathers source rows; then resid is left untouched.
template <typename OutT>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const float* __restrict__ delta,
                                   const float* __restrict__ weight, OutT* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps,
                                   int write_resid) {
  extern __shared__ float smem[];
  float* x = smem;            // [hidden]
  float* scratch = smem + hidden;  // [32]
  pdl_trigger();
#ifdef B200_EARLY_NORM
  pdl_launch_dependents();
#endif
  pdl_wait();
  const int row = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[row] : row) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = resid[src + i];
    if (delta) v += delta[src + i];
    x[i] = v;
    ss += v * v;
    if (write_resid) resid[src + i] = v;
  }
  const float total = block_sum(ss, scratch);
  const float r = rsqrtf(total / static_cast<float>(hidden) + eps);
  OutT* dst = out + static_cast<size_t>(row) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    dst[i] = from_float<OutT>(x[i] * r * weight[i]);
}

// Rows up to 4 * VPT * blockDim wide stay in registers: all loads are issued before any
// store, 16 bytes at a time.  The order of the sum depends on the width and the block
// size only.
template <typename OutT, int VPT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const float* __restrict__ delta,
                                       const float* __restrict__ weight, OutT* __restrict__ out,
                                       const int* __restrict__ rows, int hidden, float eps, int write_resid) {
  __shared__ float scratch[32];
  pdl_trigger();
#ifdef B200_EARLY_NORM
  pdl_launch_dependents();
#endif
  pdl_wait();
  const int row = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[row] : row) * hidden;
  const int nvec = hidden >> 2;
  float4 x[VPT];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * blockDim.x;
    x[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < nvec) {
      x[v] = *reinterpret_cast<const float4*>(resid + src + 4 * i);
      if (delta) {
        const float4 d = *reinterpret_cast<const float4*>(delta + src + 4 * i);
        x[v].x += d.x; x[v].y += d.y; x[v].z += d.z; x[v].w += d.w;
      }
    }
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v) ss += x[v].x * x[v].x + x[v].y * x[v].y + x[v].z * x[v].z + x[v].w * x[v].w;
  const float r = rsqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
  OutT* dst = out + static_cast<size_t>(row) * hidden;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * blockDim.x;
    if (i >= nvec) continue;
    if (write_resid) *reinterpret_cast<float4*>(resid + src + 4 * i) = x[v];
    const float4 w = *reinterpret_cast<const float4*>(weight + 4 * i);
    const float y[4] = {x[v].x * r * w.x, x[v].y * r * w.y, x[v].z * r * w.z, x[v].w * r * w.w};
    if constexpr (sizeof(OutT) == 4) {
      *reinterpret_cast<float4*>(dst + 4 * i) = make_float4(y[0], y[1], y[2], y[3]);
    } else {
      uint2 packed;
      __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst + 4 * i) = packed;
    }
  }
}

// ------------------------------------------------------------------ SiLU * up
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  const float g = to_float(gate_up[row * 2 * inter + i]);
  const float u = to_float(gate_up[row * 2 * inter + inter + i]);
  const float s = g / (1.f + expf(-g));
  out[row * inter + i] = from_float<T>(s * u);
}

// 16-byte loads and stores when the row width allows it
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
  constexpr int VN = Vec<T>::n;
  using V = typename Vec<T>::type;
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.y;
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * VN;
  if (i >= inter) return;
  float g[VN], u[VN];
  Vec<T>::unpack(*reinterpret_cast<const V*>(gate_up + row * 2 * inter + i), g);
  Vec<T>::unpack(*reinterpret_cast<const V*>(gate_up + row * 2 * inter + inter + i), u);
#pragma unroll
  for (int e = 0; e < VN; ++e) g[e] = g[e] / (1.f + expf(-g[e])) * u[e];
  *reinterpret_cast<V*>(out + row * inter + i) = Vec<T>::pack(g);
}

// ------------------------------- q/k norm + rotary + paged K/V write (fused)
// qkv row layout: [q heads | k heads | v heads], each head `d` wide.  One warp per
// (token, head), everything in registers: a lane owns the rotation pairs (j, j + half)
// for j = lane, lane + 32, ... and the unrotated tail columns lane-strided.
constexpr int kMaxPairs = 4;   // rotary_dim / 2 <= 128
constexpr int kMaxTail = 8;    // head_dim <= 256

constexpr int kRopeWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kRopeWarps * 32) qk_norm_rope_write_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_weight,
    const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
    int rotary_dim, const int* __restrict__ positions, const int* __restrict__ token_entry,
    const int* __restrict__ block_table, int table_stride, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool, int nq, int nkv, int d, int qkv_stride) {
  __shared__ float cs[32 * kMaxPairs], sn[32 * kMaxPairs];
  pdl_trigger();
#ifdef B200_EARLY_ROPE
  pdl_launch_dependents();
#endif
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x;
  const int pos = positions[token];
  const int rot_half = inv_freq ? rotary_dim / 2 : 0;
  // sine and cosine once per token, shared by all its heads
  for (int j = threadIdx.x; j < rot_half; j += blockDim.x)
    sincosf(static_cast<float>(pos) * inv_freq[j], &sn[j], &cs[j]);
  __syncthreads();
  int64_t kv_base = -1;   // element offset of this token's slot for kv head 0
  if (nkv > 0) {
    const int page = block_table[static_cast<size_t>(token_entry[token]) * table_stride + pos / page_size];
    if (page >= 0) kv_base = (static_cast<int64_t>(page) * nkv * page_size + pos % page_size) * d;
  }
  // gridDim.y blocks share a token's heads (few tokens: more blocks, one head per warp)
  for (int h = blockIdx.y * kRopeWarps + warp; h < nq + 2 * nkv; h += gridDim.y * kRopeWarps) {
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    const T* src = qkv + static_cast<size_t>(token) * qkv_stride + static_cast<size_t>(h) * d;
    T* dst;
    if (is_q) {
      dst = q_out + (static_cast<size_t>(token) * nq + h) * d;
    } else {
      if (kv_base < 0) continue;
      const int kvh = is_k ? h - nq : h - nq - nkv;
      dst = (is_k ? k_pool : v_pool) + kv_base + static_cast<int64_t>(kvh) * page_size * d;
    }
    const int half = (is_q || is_k) ? rot_half : 0;
    const int tail0 = 2 * half;
    float lo[kMaxPairs], hi[kMaxPairs], tail[kMaxTail];
    float ss = 0.f;
#pragma unroll
    for (int p = 0; p < kMaxPairs; ++p) {
      const int j = lane + 32 * p;
      lo[p] = hi[p] = 0.f;
      if (j < half) {
        lo[p] = to_float(src[j]);
        hi[p] = to_float(src[j + half]);
        ss += lo[p] * lo[p] + hi[p] * hi[p];
      }
    }
#pragma unroll
    for (int q = 0; q < kMaxTail; ++q) {
      const int i = tail0 + lane + 32 * q;
      tail[q] = 0.f;
      if (i < d) {
        tail[q] = to_float(src[i]);
        ss += tail[q] * tail[q];
      }
    }
    const float* w = is_q ? q_weight : (is_k ? k_weight : nullptr);
    const float r = w ? rsqrtf(warp_sum(ss) / static_cast<float>(d) + eps) : 1.f;
#pragma unroll
    for (int p = 0; p < kMaxPairs; ++p) {
      const int j = lane + 32 * p;
      if (j >= half) continue;
      float a = lo[p], b = hi[p];
      if (w) {
        a *= r * w[j];
        b *= r * w[j + half];
      }
      dst[j] = from_float<T>(a * cs[j] - b * sn[j]);
      dst[j + half] = from_float<T>(b * cs[j] + a * sn[j]);
    }
#pragma unroll
    for (int q = 0; q < kMaxTail; ++q) {
      const int i = tail0 + lane + 32 * q;
      if (i >= d) continue;
      dst[i] = from_float<T>(w ? tail[q] * r * w[i] : tail[q]);
    }
  }
}

// Gate and up columns interleaved in blocks of eight: [g0..g7 | u0..u7 | g8..g15 | u8..u15 | ...],
// the layout in which the stacked gate/up projection is stored so that a projection kernel
// can apply SiLU * up in its epilogue.  `inter` is a multiple of 8.
template <typename T>
__global__ void silu_mul_interleaved_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.y;
  const int block8 = blockIdx.x * blockDim.x + threadIdx.x;     // which group of eight features
  if (block8 * 8 >= inter) return;
  const T* src = gate_up + row * 2 * inter + static_cast<size_t>(block8) * 16;
  T* dst = out + row * inter + static_cast<size_t>(block8) * 8;
  constexpr int VN = Vec<T>::n;
  using V = typename Vec<T>::type;
  float g[8], u[8];
#pragma unroll
  for (int i = 0; i < 8; i += VN) {
    Vec<T>::unpack(*reinterpret_cast<const V*>(src + i), g + i);
    Vec<T>::unpack(*reinterpret_cast<const V*>(src + 8 + i), u + i);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) g[i] = g[i] / (1.f + expf(-g[i])) * u[i];
#pragma unroll
  for (int i = 0; i < 8; i += VN) *reinterpret_cast<V*>(dst + i) = Vec<T>::pack(g + i);
}

// The common case - the whole head is rotated (or none of it) and the head size is a multiple
// of 4 - with two neighbouring pairs per lane: 4- or 8-byte loads and stores, no unused loop
// iterations.  PITER = ceil(head_dim / 128).
template <typename T> struct Pair;
template <> struct Pair<float> {
  using type = float2;
  __device__ static float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  __device__ static void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Pair<__nv_bfloat16> {
  using type = float2;
  __device__ static float2 load(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
  __device__ static void store(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }
};

template <typename T, int PITER>
__global__ void __launch_bounds__(kRopeWarps * 32) qk_norm_rope_write_vec_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_weight,
    const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
    const int* __restrict__ positions, const int* __restrict__ token_entry,
    const int* __restrict__ block_table, int table_stride, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool, int nq, int nkv, int d, int qkv_stride) {
  __shared__ float cs[32 * kMaxPairs], sn[32 * kMaxPairs];
  pdl_trigger();
#ifdef B200_EARLY_ROPE
  pdl_launch_dependents();
#endif
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x;
  const int pos = positions[token];
  const int half = d / 2;
  if (inv_freq) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(static_cast<float>(pos) * inv_freq[j], &sn[j], &cs[j]);
  }
  __syncthreads();
  int64_t kv_base = -1;
  if (nkv > 0) {
    const int page = block_table[static_cast<size_t>(token_entry[token]) * table_stride + pos / page_size];
    if (page >= 0) kv_base = (static_cast<int64_t>(page) * nkv * page_size + pos % page_size) * d;
  }
  for (int h = blockIdx.y * kRopeWarps + warp; h < nq + 2 * nkv; h += gridDim.y * kRopeWarps) {
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    const T* src = qkv + static_cast<size_t>(token) * qkv_stride + static_cast<size_t>(h) * d;
    T* dst;
    if (is_q) {
      dst = q_out + (static_cast<size_t>(token) * nq + h) * d;
    } else {
      if (kv_base < 0) continue;
      const int kvh = is_k ? h - nq : h - nq - nkv;
      dst = (is_k ? k_pool : v_pool) + kv_base + static_cast<int64_t>(kvh) * page_size * d;
    }
    float2 lo[PITER], hi[PITER];
    float ss = 0.f;
#pragma unroll
    for (int p = 0; p < PITER; ++p) {
      const int j = 2 * lane + 64 * p;
      lo[p] = hi[p] = make_float2(0.f, 0.f);
      if (j < half) {
        lo[p] = Pair<T>::load(src + j);
        hi[p] = Pair<T>::load(src + j + half);
        ss += lo[p].x * lo[p].x + lo[p].y * lo[p].y + hi[p].x * hi[p].x + hi[p].y * hi[p].y;
      }
    }
    const float* w = is_q ? q_weight : (is_k ? k_weight : nullptr);
    const float r = w ? rsqrtf(warp_sum(ss) / static_cast<float>(d) + eps) : 1.f;
    const bool rotate = inv_freq != nullptr && (is_q || is_k);
#pragma unroll
    for (int p = 0; p < PITER; ++p) {
      const int j = 2 * lane + 64 * p;
      if (j >= half) continue;
      float2 a = lo[p], b = hi[p];
      if (w) {
        a.x *= r * w[j]; a.y *= r * w[j + 1];
        b.x *= r * w[j + half]; b.y *= r * w[j + half + 1];
      }
      if (rotate) {
        const float c0 = cs[j], s0 = sn[j], c1 = cs[j + 1], s1 = sn[j + 1];
        Pair<T>::store(dst + j, a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
        Pair<T>::store(dst + j + half, b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
      } else {
        Pair<T>::store(dst + j, a.x, a.y);
        Pair<T>::store(dst + j + half, b.x, b.y);
      }
    }
  }
}

// Head sizes 64, 128 and 256 with the whole head rotated (or none of it): LANES = d / 16 lanes hold
// one head, eight neighbouring elements of its lower half and the matching eight of its upper half
// each (16-byte loads and stores for bfloat16), so a warp works on 32 / LANES heads at once.  A
// task is such a group of heads; the tasks of a token may be spread over several CTAs (grid.y)
// when there are few tokens.  The arithmetic of a head does not depend on that spread.
template <typename T> __device__ __forceinline__ void load8(const T* p, float* f);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* f) {
  Vec<float>::unpack(*reinterpret_cast<const float4*>(p), f);
  Vec<float>::unpack(*reinterpret_cast<const float4*>(p + 4), f + 4);
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  Vec<__nv_bfloat16>::unpack(*reinterpret_cast<const uint4*>(p), f);
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* f);
template <> __device__ __forceinline__ void store8<float>(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = Vec<float>::pack(f);
  *reinterpret_cast<float4*>(p + 4) = Vec<float>::pack(f + 4);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
  *reinterpret_cast<uint4*>(p) = Vec<__nv_bfloat16>::pack(f);
}

template <typename T, int LANES>
__global__ void __launch_bounds__(512) qk_norm_rope_write_wide_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_weight,
    const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
    const int* __restrict__ positions, const int* __restrict__ token_entry,
    const int* __restrict__ block_table, int table_stride, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool, int nq, int nkv, int qkv_stride) {
  constexpr int D = 16 * LANES, HALF = D / 2, HEADS_PER_WARP = 32 / LANES;
  __shared__ float cs[HALF], sn[HALF];
  pdl_trigger();
#ifdef B200_EARLY_ROPE
  pdl_launch_dependents();
#endif
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int token = blockIdx.x;
  const int pos = positions[token];
  if (inv_freq) {
    for (int j = threadIdx.x; j < HALF; j += blockDim.x) sincosf(static_cast<float>(pos) * inv_freq[j], &sn[j], &cs[j]);
  }
  __syncthreads();
  int64_t kv_base = -1;
  if (nkv > 0) {
    const int page = block_table[static_cast<size_t>(token_entry[token]) * table_stride + pos / page_size];
    if (page >= 0) kv_base = (static_cast<int64_t>(page) * nkv * page_size + pos % page_size) * D;
  }
  const int heads = nq + 2 * nkv;
  const int sub = lane / LANES, li = lane % LANES;
  for (int task = blockIdx.y * warps + warp; task * HEADS_PER_WARP < heads; task += gridDim.y * warps) {
    const int h = task * HEADS_PER_WARP + sub;
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv, is_v = !is_q && !is_k && h < heads;
    T* dst = nullptr;
    if (is_q) {
      dst = q_out + (static_cast<size_t>(token) * nq + h) * D;
    } else if ((is_k || is_v) && kv_base >= 0) {
      const int kvh = is_k ? h - nq : h - nq - nkv;
      dst = (is_k ? k_pool : v_pool) + kv_base + static_cast<int64_t>(kvh) * page_size * D;
    }
    float lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) lo[i] = hi[i] = 0.f;
    if (dst) {
      const T* src = qkv + static_cast<size_t>(token) * qkv_stride + static_cast<size_t>(h) * D + 8 * li;
      load8<T>(src, lo);
      load8<T>(src + HALF, hi);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += lo[i] * lo[i];
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += hi[i] * hi[i];
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!dst) continue;
    const float* w = is_q ? q_weight : (is_k ? k_weight : nullptr);
    if (w) {
      const float r = rsqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        lo[i] *= r * w[8 * li + i];
        hi[i] *= r * w[8 * li + i + HALF];
      }
    }
    if (inv_freq != nullptr && (is_q || is_k)) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float c = cs[8 * li + i], sine = sn[8 * li + i];
        const float a = lo[i], b = hi[i];
        lo[i] = a * c - b * sine;
        hi[i] = b * c + a * sine;
      }
    }
    store8<T>(dst + 8 * li, lo);
    store8<T>(dst + 8 * li + HALF, hi);
  }
}

template <typename T>
static void launch_norm_vec(float* resid, const float* delta, const float* weight, T* out, const int* rows, int n,
                            int hidden, float eps, int write_resid, cudaStream_t stream) {
  const int nvec = hidden / 4;
  if (nvec <= 128) launch(add_rmsnorm_vec_kernel<T, 1>, dim3(n), dim3(128), 0, stream, resid, delta, weight, out, rows, hidden, eps, write_resid);
  else if (nvec <= 256) launch(add_rmsnorm_vec_kernel<T, 1>, dim3(n), dim3(256), 0, stream, resid, delta, weight, out, rows, hidden, eps, write_resid);
  else if (nvec <= 512) launch(add_rmsnorm_vec_kernel<T, 2>, dim3(n), dim3(256), 0, stream, resid, delta, weight, out, rows, hidden, eps, write_resid);
  else if (nvec <= 1024) launch(add_rmsnorm_vec_kernel<T, 4>, dim3(n), dim3(256), 0, stream, resid, delta, weight, out, rows, hidden, eps, write_resid);
  else if (nvec <= 2048) launch(add_rmsnorm_vec_kernel<T, 4>, dim3(n), dim3(512), 0, stream, resid, delta, weight, out, rows, hidden, eps, write_resid);
  else if (nvec <= 4096) launch(add_rmsnorm_vec_kernel<T, 4>, dim3(n), dim3(1024), 0, stream, resid, delta, weight, out, rows, hidden, eps, write_resid);
  else launch(add_rmsnorm_vec_kernel<T, 8>, dim3(n), dim3(1024), 0, stream, resid, delta, weight, out, rows, hidden, eps, write_resid);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_embedding(const int* ids, const void* table, float* out, int n, int hidden,
                              int vocab, float scale, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) return B200_ERR_BAD_SIZE;
  const int threads = hidden >= 1024 ? 256 : 128;
  const bool aligned = ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  B200_DISPATCH_DTYPE(dtype, T, {
    if (aligned && hidden % Vec<T>::n == 0)
      launch(embedding_vec_kernel<T>, dim3(n), dim3(threads), 0, stream, ids, static_cast<const T*>(table), out, hidden, vocab, scale);
    else
      launch(embedding_kernel<T>, dim3(n), dim3(threads), 0, stream, ids, static_cast<const T*>(table), out, hidden, vocab, scale);
  });
  return launch_status();
}

// n <= 16 rows, hidden a multiple of the 16-byte vector of the table's type and at most 8 x 256 vectors;
// row_scale receives n floats.
extern "C" int b200_embedding_weighted(const int* ids, const void* table, float* out, const float* norm_weight, void* weighted,
                                       float* row_scale, int n, int hidden, int vocab, float scale, float eps, int dtype,
                                       cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n > 16 || hidden <= 0 || vocab <= 0) return B200_ERR_BAD_SIZE;
  if (reinterpret_cast<uintptr_t>(table) & 15) return B200_ERR_BAD_SIZE;
  B200_DISPATCH_DTYPE(dtype, T, {
    constexpr int VN = Vec<T>::n;
    if (hidden % VN != 0) return B200_ERR_BAD_SIZE;
    const int vectors = hidden / VN;
    auto* tab = static_cast<const T*>(table);
    auto* wt = static_cast<__nv_bfloat16*>(weighted);
    if (vectors <= 256)
      launch(embedding_weighted_kernel<T, 1>, dim3(n), dim3(256), 0, stream, ids, tab, out, norm_weight, wt, row_scale, hidden, vocab, scale, eps);
    else if (vectors <= 512)
      launch(embedding_weighted_kernel<T, 2>, dim3(n), dim3(256), 0, stream, ids, tab, out, norm_weight, wt, row_scale, hidden, vocab, scale, eps);
    else if (vectors <= 1024)
      launch(embedding_weighted_kernel<T, 4>, dim3(n), dim3(256), 0, stream, ids, tab, out, norm_weight, wt, row_scale, hidden, vocab, scale, eps);
    else if (vectors <= 2048)
      launch(embedding_weighted_kernel<T, 8>, dim3(n), dim3(256), 0, stream, ids, tab, out, norm_weight, wt, row_scale, hidden, vocab, scale, eps);
    else
      return B200_ERR_TOO_LARGE;
  });
  return launch_status();
}

extern "C" int b200_add_rmsnorm(float* resid, const float* delta, const float* weight, void* out,
                                const int* rows, int n, int hidden, float eps, int write_resid,
                                int out_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hidden <= 0) return B200_ERR_BAD_SIZE;
  const bool aligned = ((reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(delta) |
                         reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (aligned && hidden % 4 == 0 && hidden <= 4 * 8 * 1024) {
    B200_DISPATCH_DTYPE(out_dtype, T,
        launch_norm_vec<T>(resid, delta, weight, static_cast<T*>(out), rows, n, hidden, eps, write_resid, stream));
    return launch_status();
  }
  const size_t smem = (static_cast<size_t>(hidden) + 32) * sizeof(float);
  if (smem > 200 * 1024) return B200_ERR_TOO_LARGE;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  B200_DISPATCH_DTYPE(out_dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    launch(add_rmsnorm_kernel<T>, dim3(n), dim3(threads), smem, stream, resid, delta, weight, static_cast<T*>(out),
                                                         rows, hidden, eps, write_resid);
  });
  return launch_status();
}

extern "C" int b200_silu_mul(const void* gate_up, void* out, int n, int inter, int dtype,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  if (inter <= 0) return B200_ERR_BAD_SIZE;
  if (n > 65535) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(dtype, T, {
    constexpr int VN = Vec<T>::n;
    const bool aligned = ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (inter % VN == 0 && aligned) {
      dim3 grid((inter / VN + 255) / 256, n);
      launch(silu_mul_vec_kernel<T>, dim3(grid), dim3(256), 0, stream, static_cast<const T*>(gate_up), static_cast<T*>(out), inter);
    } else {
      dim3 grid((inter + 255) / 256, n);
      launch(silu_mul_kernel<T>, dim3(grid), dim3(256), 0, stream, static_cast<const T*>(gate_up), static_cast<T*>(out), inter);
    }
  });
  return launch_status();
}

extern "C" int b200_silu_mul_interleaved(const void* gate_up, void* out, int n, int inter, int dtype,
                                         cudaStream_t stream) {
  if (n <= 0) return 0;
  if (inter <= 0 || inter % 8 != 0 || n > 65535) return B200_ERR_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) return B200_ERR_BAD_SIZE;
  dim3 grid((inter / 8 + 127) / 128, n);
  B200_DISPATCH_DTYPE(dtype, T,
      launch(silu_mul_interleaved_kernel<T>, grid, dim3(128), 0, stream, static_cast<const T*>(gate_up),
             static_cast<T*>(out), inter));
  return launch_status();
}

extern "C" int b200_qk_norm_rope_write(
    const void* qkv, void* q_out, const float* q_weight, const float* k_weight, float eps,
    const float* inv_freq, int rotary_dim, const int* positions, const int* token_entry,
    const int* block_table, int table_stride, int page_size, void* k_pool, void* v_pool, int n,
    int nq, int nkv, int d, int qkv_stride, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (d <= 0 || nq < 0 || nkv < 0 || rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) ||
      page_size <= 0)
    return B200_ERR_BAD_SIZE;
  if (rotary_dim / 2 > 32 * kMaxPairs || d > 32 * kMaxTail) return B200_ERR_TOO_LARGE;
  const int heads = nq + 2 * nkv;
  const int head_blocks = n >= 512 ? 1 : (heads + kRopeWarps - 1) / kRopeWarps;
  const bool whole_head = inv_freq == nullptr || rotary_dim == d;
  const bool aligned4 = ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                          reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 7) == 0;
  const bool aligned16 = ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                           reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 15) == 0;
  if (whole_head && (d == 64 || d == 128 || d == 256) && qkv_stride % 8 == 0 && aligned16) {
    const int heads_per_warp = 32 / (d / 16);
    const int tasks = (heads + heads_per_warp - 1) / heads_per_warp;
    const int warps = tasks < (n >= 256 ? 16 : 2) ? tasks : (n >= 256 ? 16 : 2);
    const dim3 grid(n, n >= 256 ? 1 : (tasks + warps - 1) / warps);
    B200_DISPATCH_DTYPE(dtype, T, {
      auto* in = static_cast<const T*>(qkv);
      auto* qo = static_cast<T*>(q_out);
      auto* kp = static_cast<T*>(k_pool);
      auto* vp = static_cast<T*>(v_pool);
      if (d == 64)
        launch(qk_norm_rope_write_wide_kernel<T, 4>, grid, dim3(warps * 32), 0, stream, in, qo, q_weight, k_weight, eps, inv_freq,
               positions, token_entry, block_table, table_stride, page_size, kp, vp, nq, nkv, qkv_stride);
      else if (d == 128)
        launch(qk_norm_rope_write_wide_kernel<T, 8>, grid, dim3(warps * 32), 0, stream, in, qo, q_weight, k_weight, eps, inv_freq,
               positions, token_entry, block_table, table_stride, page_size, kp, vp, nq, nkv, qkv_stride);
      else
        launch(qk_norm_rope_write_wide_kernel<T, 16>, grid, dim3(warps * 32), 0, stream, in, qo, q_weight, k_weight, eps, inv_freq,
               positions, token_entry, block_table, table_stride, page_size, kp, vp, nq, nkv, qkv_stride);
    });
    return launch_status();
  }
  if (whole_head && d % 4 == 0 && d <= 256 && qkv_stride % 2 == 0 && aligned4) {
    B200_DISPATCH_DTYPE(dtype, T, {
      auto* in = static_cast<const T*>(qkv);
      auto* qo = static_cast<T*>(q_out);
      auto* kp = static_cast<T*>(k_pool);
      auto* vp = static_cast<T*>(v_pool);
      if (d <= 128)
        launch(qk_norm_rope_write_vec_kernel<T, 1>, dim3(n, head_blocks), dim3(kRopeWarps * 32), 0, stream, in, qo, q_weight,
               k_weight, eps, inv_freq, positions, token_entry, block_table, table_stride, page_size, kp, vp, nq, nkv, d, qkv_stride);
      else
        launch(qk_norm_rope_write_vec_kernel<T, 2>, dim3(n, head_blocks), dim3(kRopeWarps * 32), 0, stream, in, qo, q_weight,
               k_weight, eps, inv_freq, positions, token_entry, block_table, table_stride, page_size, kp, vp, nq, nkv, d, qkv_stride);
    });
    return launch_status();
  }
  B200_DISPATCH_DTYPE(dtype, T,
      launch(qk_norm_rope_write_kernel<T>, dim3(n, head_blocks), dim3(kRopeWarps * 32), 0, stream, 
          static_cast<const T*>(qkv), static_cast<T*>(q_out), q_weight, k_weight, eps, inv_freq,
          rotary_dim, positions, token_entry, block_table, table_stride, page_size,
          static_cast<T*>(k_pool), static_cast<T*>(v_pool), nq, nkv, d, qkv_stride));
  return launch_status();
}
