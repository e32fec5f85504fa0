// Next-token selection on the device, one thread block per row of logits.
//
// temperature == 0: argmax (the lowest index wins a tie)      mini_llm/sampling.py:80-82
// temperature  > 0: x = logits / temperature; keep the top_k largest; of those keep
//   the smallest set of largest-probability tokens whose mass reaches top_p (a token
//   stays iff the mass of the tokens strictly above it is < top_p, so at least one
//   stays); draw from softmax over what is left              mini_llm/sampling.py:51-69, 87-91
// The draw is Gumbel-max: argmax(x_i + g_i), g_i = -log(-log(u_i)), which samples
// softmax(x) exactly.  u_i comes from a counter-based generator keyed by (request
// seed, index of the token being generated, vocabulary index), so a request's draws
// do not depend on what else is in the batch.  The thresholds for top_k and top_p
// are found by bisection over the 32 bits of an order-preserving integer key of x,
// which needs no sort and no scratch memory.
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ uint32_t ordered_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// uniform in (0, 1) from (stream key, vocabulary index): 23 random bits plus one half,
// which float32 holds exactly, so neither 0 nor 1 can come out
__device__ __forceinline__ float uniform23(uint64_t stream, uint32_t index) {
  const uint64_t z = splitmix64(stream + static_cast<uint64_t>(index) * 0xD1B54A32D192ED03ull);
  return (static_cast<float>(static_cast<uint32_t>(z >> 41)) + 0.5f) * (1.0f / 8388608.0f);
}

struct ArgMax {
  float value;
  int index;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax v, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, v.value, o), __shfl_xor_sync(0xffffffffu, v.index, o)};
    v = better(v, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  ArgMax t = lane < nwarps ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, t.value, o), __shfl_xor_sync(0xffffffffu, t.index, o)};
    t = better(t, other);
  }
  return t;  // every thread holds the result
}

// params per row: [temperature bits, top_k, top_p bits, seed lo, seed hi, counter]
constexpr int kParamWords = 6;

__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, const int* __restrict__ params,
              int* __restrict__ out, int filtered_only) {
  __shared__ ArgMax arg_scratch[32];
  __shared__ float sum_scratch[32];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const float* x = logits + static_cast<size_t>(row) * ld;
  const int* p = params + row * kParamWords;
  if (filtered_only && !(__int_as_float(p[0]) != 0.f && ((p[1] > 0 && p[1] < vocab) || __int_as_float(p[2]) < 1.f))) return;
  const float temperature = __int_as_float(p[0]);
  const int top_k = p[1];
  const float top_p = __int_as_float(p[2]);
  const uint64_t seed = (static_cast<uint64_t>(static_cast<uint32_t>(p[4])) << 32) | static_cast<uint32_t>(p[3]);
  const uint32_t counter = static_cast<uint32_t>(p[5]);

  // non-finite logits are an error (mini_llm/sampling.py:104-113): report -1
  float bad = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) bad += isfinite(x[i]) ? 0.f : 1.f;
  if (block_sum(bad, sum_scratch) > 0.f) {
    if (threadIdx.x == 0) out[row] = -1;
    return;
  }

  if (temperature == 0.f) {
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{x[i], i});
    best = block_argmax(best, arg_scratch);
    if (threadIdx.x == 0) out[row] = best.index;
    return;
  }

  uint32_t low_key = 0;  // tokens with key >= low_key stay
  if (top_k > 0 && top_k < vocab) {
    uint32_t k = 0;
    for (int b = 31; b >= 0; --b) {
      const uint32_t cand = k | (1u << b);
      float count = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x)
        count += ordered_key(x[i] / temperature) >= cand ? 1.f : 0.f;
      if (block_sum(count, sum_scratch) >= static_cast<float>(top_k)) k = cand;
    }
    low_key = k;
  }
  if (top_p < 1.f) {
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, x[i] / temperature);
    mx = block_argmax(ArgMax{mx, 0}, arg_scratch).value;
    float z = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = x[i] / temperature;
      if (ordered_key(v) >= low_key) z += expf(v - mx);
    }
    const float target = top_p * block_sum(z, sum_scratch);
    uint32_t k = 0;
    for (int b = 31; b >= 0; --b) {
      const uint32_t cand = k | (1u << b);
      float mass = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = x[i] / temperature;
        const uint32_t key = ordered_key(v);
        if (key >= cand && key >= low_key) mass += expf(v - mx);
      }
      if (block_sum(mass, sum_scratch) >= target) k = cand;
    }
    low_key = max(low_key, k);
  }
  const uint64_t stream = splitmix64(seed ^ splitmix64(static_cast<uint64_t>(counter)));
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = x[i] / temperature;
    if (ordered_key(v) < low_key) continue;
    const float u = uniform23(stream, static_cast<uint32_t>(i));
    best = better(best, ArgMax{v - logf(-logf(u)), i});
  }
  best = block_argmax(best, arg_scratch);
  if (threadIdx.x == 0) out[row] = best.index;
}

// ---------------------------------------------------------------- two-stage selection
// Rows without top_k / top_p need one pass only (argmax of the logits, or of the logits
// plus Gumbel noise), so the vocabulary is cut into `chunks` parts handled by different
// CTAs; the second stage picks the best of the partial results.  Rows with filters take
// the single-CTA kernel above.
__device__ __forceinline__ bool row_is_filtered(const int* p, int vocab) {
  const float temperature = __int_as_float(p[0]);
  return temperature != 0.f && ((p[1] > 0 && p[1] < vocab) || __int_as_float(p[2]) < 1.f);
}

__global__ void __launch_bounds__(256)
sample_partial_kernel(const float* __restrict__ logits, int ld, int vocab, const int* __restrict__ params,
                      float* __restrict__ part_value, int* __restrict__ part_index, int chunks) {
  __shared__ ArgMax arg_scratch[32];
  __shared__ float sum_scratch[32];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.y, chunk = blockIdx.x;
  const int* p = params + row * kParamWords;
  if (row_is_filtered(p, vocab)) return;
  const float* x = logits + static_cast<size_t>(row) * ld;
  const float temperature = __int_as_float(p[0]);
  const uint64_t seed = (static_cast<uint64_t>(static_cast<uint32_t>(p[4])) << 32) | static_cast<uint32_t>(p[3]);
  const uint64_t stream = splitmix64(seed ^ splitmix64(static_cast<uint64_t>(static_cast<uint32_t>(p[5]))));
  const int per = (vocab + chunks - 1) / chunks;
  const int begin = chunk * per, end = min(vocab, begin + per);
  ArgMax best{-INFINITY, 0x7fffffff};
  float bad = 0.f;
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float raw = x[i];
    bad += isfinite(raw) ? 0.f : 1.f;
    float v = raw;
    if (temperature != 0.f) v = raw / temperature - logf(-logf(uniform23(stream, static_cast<uint32_t>(i))));
    best = better(best, ArgMax{v, i});
  }
  best = block_argmax(best, arg_scratch);
  bad = block_sum(bad, sum_scratch);
  if (threadIdx.x == 0) {
    part_value[row * chunks + chunk] = best.value;
    part_index[row * chunks + chunk] = bad > 0.f ? -1 : best.index;
  }
}

__global__ void sample_final_kernel(const float* __restrict__ part_value, const int* __restrict__ part_index,
                                    const int* __restrict__ params, int vocab, int* __restrict__ out, int chunks) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  if (row_is_filtered(params + row * kParamWords, vocab)) return;   // written by sample_kernel
  ArgMax best{-INFINITY, 0x7fffffff};
  bool bad = false;
  for (int c = threadIdx.x; c < chunks; c += 32) {
    const int index = part_index[row * chunks + c];
    if (index < 0) bad = true;
    else best = better(best, ArgMax{part_value[row * chunks + c], index});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
    best = better(best, other);
  }
  bad = __any_sync(0xffffffffu, bad);
  if (threadIdx.x == 0) out[row] = bad ? -1 : best.index;
}

}  // namespace b200

extern "C" int b200_sample(const float* logits, int ld, int vocab, const int* params, int* out,
                           int rows, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || ld < vocab) return B200_ERR_BAD_SIZE;
  const int threads = vocab >= 8192 ? 1024 : (vocab >= 1024 ? 256 : 128);
  b200::launch(b200::sample_kernel, dim3(rows), dim3(threads), 0, stream, logits, ld, vocab, params, out, 0);
  return b200::launch_status();
}

// Two-stage variant.  `scratch` holds rows * chunks floats followed by rows * chunks ints;
// `any_filtered` tells whether some row uses top_k / top_p (then the single-CTA kernel also
// runs, for those rows only).
extern "C" int b200_sample_chunked(const float* logits, int ld, int vocab, const int* params, int* out, int rows,
                                   int chunks, void* scratch, int any_filtered, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || ld < vocab || chunks <= 0 || rows > 65535) return B200_ERR_BAD_SIZE;
  float* part_value = static_cast<float*>(scratch);
  int* part_index = reinterpret_cast<int*>(part_value + static_cast<size_t>(rows) * chunks);
  dim3 grid(chunks, rows);
  b200::launch(b200::sample_partial_kernel, dim3(grid), dim3(256), 0, stream, logits, ld, vocab, params, part_value, part_index, chunks);
  b200::launch(b200::sample_final_kernel, dim3(rows), dim3(32), 0, stream, part_value, part_index, params, vocab, out, chunks);
  if (any_filtered) {
    const int threads = vocab >= 8192 ? 1024 : (vocab >= 1024 ? 256 : 128);
    b200::launch(b200::sample_kernel, dim3(rows), dim3(threads), 0, stream, logits, ld, vocab, params, out, 1);
  }
  return b200::launch_status();
}
