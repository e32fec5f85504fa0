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

// ------------------------------------------------------------------ SiLU * up
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
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
// qkv row layout: [q heads | k heads | v heads], each head `d` wide.
// One block per token; each warp takes heads in turn.
template <typename T>
__global__ void qk_norm_rope_write_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_weight,
    const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
    int rotary_dim, const int* __restrict__ positions, const int* __restrict__ token_entry,
    const int* __restrict__ block_table, int table_stride, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool, int nq, int nkv, int d, int qkv_stride) {
  extern __shared__ float smem[];
  const int half = rotary_dim / 2;
  float* cs = smem;                 // [half] cos
  float* sn = smem + half;          // [half] sin
  float* work = smem + 2 * half;    // [warps][d]
  const int token = blockIdx.x;
  const int pos = positions[token];
  if (inv_freq) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      const float angle = static_cast<float>(pos) * inv_freq[j];
      float s, c;
      sincosf(angle, &s, &c);
      cs[j] = c;
      sn[j] = s;
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* x = work + warp * d;
  const T* row = qkv + static_cast<size_t>(token) * qkv_stride;

  int64_t kv_base = -1;  // element offset of this token's slot for kv head 0
  if (nkv > 0) {
    const int page = block_table[static_cast<size_t>(token_entry[token]) * table_stride + pos / page_size];
    if (page >= 0)
      kv_base = (static_cast<int64_t>(page) * nkv * page_size + pos % page_size) * d;
  }

  for (int h = warp; h < nq + 2 * nkv; h += nwarps) {
    const T* src = row + static_cast<size_t>(h) * d;
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    const float* w = is_q ? q_weight : (is_k ? k_weight : nullptr);
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float v = to_float(src[i]);
      x[i] = v;
      ss += v * v;
    }
    if (w) {
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / static_cast<float>(d) + eps);
      __syncwarp();
      for (int i = lane; i < d; i += 32) x[i] = x[i] * r * w[i];
    }
    __syncwarp();
    T* dst;
    if (is_q) {
      dst = q_out + (static_cast<size_t>(token) * nq + h) * d;
    } else {
      if (kv_base < 0) continue;
      const int kvh = is_k ? h - nq : h - nq - nkv;
      dst = (is_k ? k_pool : v_pool) + kv_base + static_cast<int64_t>(kvh) * page_size * d;
    }
    const bool rotate = inv_freq && (is_q || is_k);
    for (int i = lane; i < d; i += 32) {
      float v = x[i];
      if (rotate && i < rotary_dim) {
        if (i < half) v = x[i] * cs[i] - x[i + half] * sn[i];
        else          v = x[i] * cs[i - half] + x[i - half] * sn[i - half];
      }
      dst[i] = from_float<T>(v);
    }
    __syncwarp();
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_embedding(const int* ids, const void* table, float* out, int n, int hidden,
                              int vocab, float scale, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) return B200_ERR_BAD_SIZE;
  const int threads = hidden >= 1024 ? 256 : 128;
  B200_DISPATCH_DTYPE(dtype, T,
      embedding_kernel<T><<<n, threads, 0, stream>>>(ids, static_cast<const T*>(table), out,
                                                      hidden, vocab, scale));
  return launch_status();
}

extern "C" int b200_add_rmsnorm(float* resid, const float* delta, const float* weight, void* out,
                                const int* rows, int n, int hidden, float eps, int write_resid,
                                int out_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hidden <= 0) return B200_ERR_BAD_SIZE;
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
    add_rmsnorm_kernel<T><<<n, threads, smem, stream>>>(resid, delta, weight, static_cast<T*>(out),
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
      silu_mul_vec_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(gate_up), static_cast<T*>(out), inter);
    } else {
      dim3 grid((inter + 255) / 256, n);
      silu_mul_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(gate_up), static_cast<T*>(out), inter);
    }
  });
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
  const int warps = 4;
  const size_t smem = (static_cast<size_t>(rotary_dim) + static_cast<size_t>(warps) * d) * sizeof(float);
  if (smem > 48 * 1024) return B200_ERR_TOO_LARGE;
  B200_DISPATCH_DTYPE(dtype, T,
      qk_norm_rope_write_kernel<T><<<n, warps * 32, smem, stream>>>(
          static_cast<const T*>(qkv), static_cast<T*>(q_out), q_weight, k_weight, eps, inv_freq,
          rotary_dim, positions, token_entry, block_table, table_stride, page_size,
          static_cast<T*>(k_pool), static_cast<T*>(v_pool), nq, nkv, d, qkv_stride));
  return launch_status();
}
