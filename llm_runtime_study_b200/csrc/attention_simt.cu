// Causal attention over the paged cache on CUDA cores, 32-bit arithmetic throughout.
// It serves prompt portions and single decoded tokens alike: every query token is
// handled by itself (one warp per token and query head), reading keys 0..p of its
// request through the block table, in tiles of 32 keys that start at key 0.  The
// order of every sum is therefore a function of the token's own position only, so a
// token's output is bit-identical however the batch was cut.
//
// Formula (mini_llm/nn/attention.py:95-99, 231-248): S = q.k^T * scale, key t visible
// iff t <= p (and t > p - window when a window is set), P = softmax(S), o = P.v;
// query head j reads KV head j / (nq / nkv)  (mini_llm/nn/attention.py:18-33).
#include "common.cuh"

namespace b200 {

constexpr int kMaxChunks = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(128)
paged_attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                            const T* __restrict__ v_pool, T* __restrict__ out,
                            const int* __restrict__ positions, const int* __restrict__ token_entry,
                            const int* __restrict__ block_table, int table_stride, int page_size,
                            int nq, int nkv, int d, float scale, int window) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x;
  const int head = blockIdx.y * 4 + warp;
  if (head >= nq) return;
  const int kvh = head / (nq / nkv);
  const int p = positions[token];
  const int* table = block_table + static_cast<size_t>(token_entry[token]) * table_stride;
  float* qs = smem + warp * d;
  const T* qrow = q + (static_cast<size_t>(token) * nq + head) * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_float(qrow[i]);
  __syncwarp();

  const int w0 = window > 0 ? max(0, p - window + 1) : 0;
  float m = -INFINITY, l = 0.f;
  float acc[kMaxChunks];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) acc[c] = 0.f;

  constexpr int VN = Vec<T>::n;
  for (int t0 = (w0 / 32) * 32; t0 <= p; t0 += 32) {
    const int t = t0 + lane;
    bool valid = t <= p && t >= w0;
    float s = -INFINITY;
    const int page = valid ? table[t / page_size] : -1;
    valid = valid && page >= 0;      // a page given back (window) or a padding row without pages
    if (valid) {
      const T* krow = k_pool + ((static_cast<size_t>(page) * nkv + kvh) * page_size + t % page_size) * d;
      float dot = 0.f;
      for (int i = 0; i < d; i += VN) {
        float f[VN];
        Vec<T>::unpack(*reinterpret_cast<const typename Vec<T>::type*>(krow + i), f);
#pragma unroll
        for (int e = 0; e < VN; ++e) dot = fmaf(qs[i + e], f[e], dot);
      }
      s = dot * scale;
    }
    const float m_tile = warp_max(s);
    if (m_tile == -INFINITY) continue;
    const float m_new = fmaxf(m, m_tile);
    const float corr = expf(m - m_new);  // m = -inf -> 0
    const float pl = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pl);
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) acc[c] *= corr;
    const int count = min(32, p - t0 + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pl, j);
      if (pj == 0.f) continue;
      const int tj = t0 + j;
      const int page = table[tj / page_size];
      const T* vrow = v_pool + ((static_cast<size_t>(page) * nkv + kvh) * page_size + tj % page_size) * d;
#pragma unroll
      for (int c = 0; c < kMaxChunks; ++c) {
        const int i = lane + 32 * c;
        if (i < d) acc[c] = fmaf(pj, to_float(vrow[i]), acc[c]);
      }
    }
    m = m_new;
  }
  T* orow = out + (static_cast<size_t>(token) * nq + head) * d;
  const float inv = l > 0.f ? 1.f / l : 0.f;   // a row without any visible key (padding) gives zeros
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int i = lane + 32 * c;
    if (i < d) orow[i] = from_float<T>(acc[c] * inv);
  }
}

}  // namespace b200

extern "C" int b200_paged_attention_simt(
    const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
    const int* token_entry, const int* block_table, int table_stride, int page_size, int n,
    int nq, int nkv, int d, float scale, int window, int dtype, cudaStream_t stream) {
  using namespace b200;
  if (n <= 0) return 0;
  if (d <= 0 || d % 8 != 0 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0)
    return B200_ERR_BAD_SIZE;
  if (d > 32 * kMaxChunks) return B200_ERR_TOO_LARGE;
  dim3 grid(n, (nq + 3) / 4);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  const size_t smem = static_cast<size_t>(4) * d * sizeof(float);
  B200_DISPATCH_DTYPE(dtype, T,
      launch(paged_attention_simt_kernel<T>, dim3(grid), dim3(128), smem, stream, 
          static_cast<const T*>(q), static_cast<const T*>(k_pool), static_cast<const T*>(v_pool),
          static_cast<T*>(out), positions, token_entry, block_table, table_stride, page_size, nq,
          nkv, d, scale, window));
  return launch_status();
}
