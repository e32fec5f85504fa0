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
// are found by a search over the 32 bits of an order-preserving integer key of x, four
// bits a pass (fifteen candidate thresholds are counted at once), which needs no sort and
// no scratch memory; the passes over the row use 16-byte loads, two in flight per thread.
// Every sum is taken in an order fixed by the launch shape: the same bits every run.
//
// The per-row parameters are six words [temperature bits, top_k, top_p bits, seed low, seed high,
// counter].  They come either as an array [rows][6], or out of the per-request slot records on the
// device (slots.cu): then `row_slots[row]` names the record, and the kernel that settles a row also
// writes the chosen token and the advanced counter back into it, so that the next decode step and
// the next draw need nothing from the host.
#include "common.cuh"
#include "slots.h"

namespace b200 {

constexpr int kParamWords = 6;   // per row: [temperature bits, top_k, top_p bits, seed low, seed high, counter]

// Where a row's six parameter words are, and (slot records only) where its result goes.
struct RowParams {
  int* base;              // [rows][6], or the slot table
  const int* row_slots;   // nullptr: row i uses base + 6 i; else base + kSlotWords * row_slots[i] + kSlotSampling
  __device__ __forceinline__ const int* of(int row) const {
    return row_slots ? base + static_cast<size_t>(row_slots[row]) * kSlotWords + kSlotSampling : base + row * kParamWords;
  }
  // The draw for this row is settled: remember it in the request's record and advance its counter.
  __device__ __forceinline__ void settle(int row, int token, int counter) const {
    if (!row_slots) return;
    int* rec = base + static_cast<size_t>(row_slots[row]) * kSlotWords;
    rec[kSlotLastToken] = token;
    rec[kSlotCounter] = counter + 1;
  }
};

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

// A CTA's share of a row: elements [begin, end), begin a multiple of four.
struct Slice {
  const float* x;      // the row
  int begin, end;
};

// Calls f(x[i] / temperature, i) for every i of the slice: 16-byte loads, two in flight per thread,
// then the ragged end.  The order in which a thread sees its elements is fixed by the block size.
template <typename F>
__device__ __forceinline__ void for_each_scaled(const Slice& sl, float temperature, F&& f) {
  const bool aligned = (reinterpret_cast<uintptr_t>(sl.x) & 15) == 0;
  const int first = sl.begin >> 2;
  const int vec = aligned ? sl.end >> 2 : first;          // whole groups of four up to here
  const float4* x4 = reinterpret_cast<const float4*>(sl.x);
  const float* x = sl.x;
  const int step = blockDim.x;
  int i = first + threadIdx.x;
  for (; i + step < vec; i += 2 * step) {
    const float4 a = x4[i], b = x4[i + step];
    f(a.x / temperature, 4 * i);
    f(a.y / temperature, 4 * i + 1);
    f(a.z / temperature, 4 * i + 2);
    f(a.w / temperature, 4 * i + 3);
    f(b.x / temperature, 4 * (i + step));
    f(b.y / temperature, 4 * (i + step) + 1);
    f(b.z / temperature, 4 * (i + step) + 2);
    f(b.w / temperature, 4 * (i + step) + 3);
  }
  for (; i < vec; i += step) {
    const float4 a = x4[i];
    f(a.x / temperature, 4 * i);
    f(a.y / temperature, 4 * i + 1);
    f(a.z / temperature, 4 * i + 2);
    f(a.w / temperature, 4 * i + 3);
  }
  for (int j = 4 * vec + threadIdx.x; j < sl.end; j += step) f(x[j] / temperature, j);
}

// ---- reductions over the CTAs of a cluster (a cluster of one is the plain block) ----
// Each CTA puts its block-wide result into a slot of its own shared memory; after a cluster barrier every
// CTA reads the slots of all ranks in rank order, so all of them hold the same bits.  Two sets of slots
// alternate, which makes one barrier per reduction enough.
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t n;
  asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(n));
  return n;
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float load_from_rank(const float* local, uint32_t rank) {
  uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(local)), remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(address), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
struct ClusterSlots {
  float (*slots)[16];      // [2][16] in shared memory: what this CTA contributes
  float (*gathered)[16];   // [16 ranks][16]: the contributions of all ranks, fetched by one thread each
  int which;
};
constexpr int kMaxClusterRanks = 16;
template <int N>
__device__ void cluster_sum_n(float (&v)[N], ClusterSlots& cs, uint32_t ranks) {
  static_assert(N <= 16, "slots hold sixteen values");
  if (ranks == 1) return;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int n = 0; n < N; ++n) cs.slots[cs.which][n] = v[n];
  }
  cluster_barrier();
  // one remote load per thread, all in flight together; then every thread adds them up in rank order
  if (threadIdx.x < ranks * N) {
    const uint32_t r = threadIdx.x / N, n = threadIdx.x % N;
    cs.gathered[r][n] = load_from_rank(&cs.slots[cs.which][n], r);
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < N; ++n) {
    float total = 0.f;
    for (uint32_t r = 0; r < ranks; ++r) total += cs.gathered[r][n];
    v[n] = total;
  }
  __syncthreads();          // the gathered values are read before the next reduction overwrites them
  cs.which ^= 1;
}

// Sums of N per-thread values over the block, in a fixed order; every thread gets all N results.
template <int N>
__device__ void block_sum_n(float (&v)[N], float (*scratch)[32]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int n = 0; n < N; ++n) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[n] += __shfl_xor_sync(0xffffffffu, v[n], o);
  }
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int n = 0; n < N; ++n) scratch[n][warp] = v[n];
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < N; ++n) {
    float t = lane < nwarps ? scratch[n][lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    v[n] = t;
  }
}

// The largest key k such that weight(keys >= k) >= target, searched four bits a pass over the whole row
// (every CTA of the cluster scans its slice; the partial weights are added in rank order).  The weight of
// an element is 1 (MASS = false: a count) or exp(v - mx) (MASS = true); elements below `floor_key`
// weigh nothing.  0 when even the whole row does not reach the target.
template <bool MASS>
__device__ uint32_t find_threshold(const Slice& sl, float temperature, uint32_t floor_key, float mx, float target,
                                   float (*scratch)[32], ClusterSlots& cs, uint32_t ranks) {
  uint32_t k = 0;
  for (int shift = 28; shift >= 0; shift -= 4) {
    float w[15];
#pragma unroll
    for (int j = 0; j < 15; ++j) w[j] = 0.f;
    for_each_scaled(sl, temperature, [&](float v, int) {
      const uint32_t key = ordered_key(v);
      if (key < floor_key || key < k) return;
      // among the keys that share the bits found so far, the next four bits say how many candidates it reaches
      const uint32_t reach = (key >> shift) >= (k >> shift) + 16u ? 15u : ((key >> shift) & 15u);
      const float weight = MASS ? expf(v - mx) : 1.f;
#pragma unroll
      for (int j = 0; j < 15; ++j) w[j] += static_cast<uint32_t>(j) < reach ? weight : 0.f;
    });
    block_sum_n<15>(w, scratch);
    cluster_sum_n<15>(w, cs, ranks);
    uint32_t best = 0;
#pragma unroll
    for (int j = 0; j < 15; ++j)
      if (w[j] >= target) best = j + 1;       // weights fall with j: the last one that still reaches the target
    k |= best << shift;
  }
  return k;
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

// One cluster of CTAs per row (gridDim.x = rows * cluster size): each CTA scans its slice of the row and
// the CTAs combine their results through distributed shared memory.
__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, RowParams params,
              int* __restrict__ out, int filtered_only) {
  __shared__ ArgMax arg_scratch[32];
  __shared__ float sum_scratch[32];
  __shared__ float multi_scratch[15][32];
  __shared__ float slot_memory[2][16];
  __shared__ float gathered_memory[kMaxClusterRanks][16];
  pdl_trigger();
  pdl_wait();
  const uint32_t ranks = cluster_size(), rank = cluster_rank();
  const int row = blockIdx.x / ranks;
  const int* p = params.of(row);
  // the whole cluster leaves together: no CTA may wait at a cluster barrier for one that has returned
  if (filtered_only && !(__int_as_float(p[0]) != 0.f && ((p[1] > 0 && p[1] < vocab) || __int_as_float(p[2]) < 1.f))) return;
  const float temperature = __int_as_float(p[0]);
  const int top_k = p[1];
  const float top_p = __int_as_float(p[2]);
  const uint64_t seed = (static_cast<uint64_t>(static_cast<uint32_t>(p[4])) << 32) | static_cast<uint32_t>(p[3]);
  const uint32_t counter = static_cast<uint32_t>(p[5]);
  const int per = ((vocab + static_cast<int>(ranks) - 1) / static_cast<int>(ranks) + 3) & ~3;
  Slice sl{logits + static_cast<size_t>(row) * ld, min(vocab, static_cast<int>(rank) * per), min(vocab, static_cast<int>(rank + 1) * per)};
  ClusterSlots cs{slot_memory, gathered_memory, 0};
  auto cluster_sum = [&](float v) {
    float one[1] = {block_sum(v, sum_scratch)};
    cluster_sum_n<1>(one, cs, ranks);
    return one[0];
  };
  auto cluster_argmax = [&](ArgMax v) {
    v = block_argmax(v, arg_scratch);
    if (ranks == 1) return v;
    if (threadIdx.x == 0) {
      cs.slots[cs.which][0] = v.value;
      cs.slots[cs.which][1] = __int_as_float(v.index);
    }
    cluster_barrier();
    if (threadIdx.x < ranks * 2) {
      const uint32_t r = threadIdx.x >> 1, n = threadIdx.x & 1;
      cs.gathered[r][n] = load_from_rank(&cs.slots[cs.which][n], r);
    }
    __syncthreads();
    ArgMax best{-INFINITY, 0x7fffffff};
    for (uint32_t r = 0; r < ranks; ++r) best = better(best, ArgMax{cs.gathered[r][0], __float_as_int(cs.gathered[r][1])});
    __syncthreads();
    cs.which ^= 1;
    return best;
  };

  // non-finite logits are an error (mini_llm/sampling.py:104-113): report -1
  float bad = 0.f;
  for_each_scaled(sl, 1.f, [&](float v, int) { bad += isfinite(v) ? 0.f : 1.f; });
  const bool any_bad = cluster_sum(bad) > 0.f;
  int result = -1;
  if (!any_bad && temperature == 0.f) {
    ArgMax best{-INFINITY, 0x7fffffff};
    for_each_scaled(sl, 1.f, [&](float v, int i) { best = better(best, ArgMax{v, i}); });
    result = cluster_argmax(best).index;
  } else if (!any_bad) {
    uint32_t low_key = 0;  // tokens with key >= low_key stay
    if (top_k > 0 && top_k < vocab)
      low_key = find_threshold<false>(sl, temperature, 0u, 0.f, static_cast<float>(top_k), multi_scratch, cs, ranks);
    if (top_p < 1.f) {
      float mx = -INFINITY;
      for_each_scaled(sl, temperature, [&](float v, int) { mx = fmaxf(mx, v); });
      mx = cluster_argmax(ArgMax{mx, 0}).value;
      float z = 0.f;
      for_each_scaled(sl, temperature, [&](float v, int) {
        if (ordered_key(v) >= low_key) z += expf(v - mx);
      });
      const float target = top_p * cluster_sum(z);
      low_key = max(low_key, find_threshold<true>(sl, temperature, low_key, mx, target, multi_scratch, cs, ranks));
    }
    const uint64_t stream = splitmix64(seed ^ splitmix64(static_cast<uint64_t>(counter)));
    ArgMax best{-INFINITY, 0x7fffffff};
    for_each_scaled(sl, temperature, [&](float v, int i) {
      if (ordered_key(v) < low_key) return;
      const float u = uniform23(stream, static_cast<uint32_t>(i));
      best = better(best, ArgMax{v - logf(-logf(u)), i});
    });
    result = cluster_argmax(best).index;
  }
  // every CTA of the cluster has read the row's parameters by now (the reductions above are barriers)
  if (rank == 0 && threadIdx.x == 0) {
    out[row] = result;
    params.settle(row, result, static_cast<int>(counter));
  }
  if (ranks > 1) cluster_barrier();        // nobody leaves while its slots may still be read
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
sample_partial_kernel(const float* __restrict__ logits, int ld, int vocab, RowParams params,
                      float* __restrict__ part_value, int* __restrict__ part_index, int chunks) {
  __shared__ ArgMax arg_scratch[32];
  __shared__ float sum_scratch[32];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.y, chunk = blockIdx.x;
  const int* p = params.of(row);
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
                                    RowParams params, int vocab, int* __restrict__ out, int chunks) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int* p = params.of(row);
  if (row_is_filtered(p, vocab)) return;   // written by sample_kernel
  const int counter = p[5];
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
  if (threadIdx.x == 0) {
    out[row] = bad ? -1 : best.index;
    params.settle(row, bad ? -1 : best.index, counter);
  }
}

}  // namespace b200

// The single-kernel path: a cluster of up to eight CTAs per row for vocabularies of 32,768 entries and
// more, one CTA otherwise.
static int launch_sample(const float* logits, int ld, int vocab, b200::RowParams params, int* out, int rows, int filtered_only,
                         cudaStream_t stream) {
  const int threads = vocab >= 8192 ? 1024 : (vocab >= 1024 ? 256 : 128);
  // a cluster of CTAs per row for large vocabularies, as long as all clusters fit on the GPU at once
  const int cluster = vocab < 32768 ? 1 : (rows <= 16 ? 8 : (rows <= 32 ? 4 : (rows <= 64 ? 2 : 1)));
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(rows * cluster);
  config.blockDim = dim3(threads);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = b200::pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&config, b200::sample_kernel, logits, ld, vocab, params, out, filtered_only);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

extern "C" int b200_sample(const float* logits, int ld, int vocab, const int* params, int* out,
                           int rows, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || ld < vocab) return B200_ERR_BAD_SIZE;
  return launch_sample(logits, ld, vocab, b200::RowParams{const_cast<int*>(params), nullptr}, out, rows, 0, stream);
}

// Two-stage variant.  `scratch` holds rows * chunks floats followed by rows * chunks ints;
// `any_filtered` tells whether some row uses top_k / top_p (then the single-CTA kernel also
// runs, for those rows only).
static int sample_chunked(const float* logits, int ld, int vocab, b200::RowParams params, int* out, int rows,
                          int chunks, void* scratch, int any_filtered, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || ld < vocab || chunks <= 0 || rows > 65535) return B200_ERR_BAD_SIZE;
  float* part_value = static_cast<float*>(scratch);
  int* part_index = reinterpret_cast<int*>(part_value + static_cast<size_t>(rows) * chunks);
  dim3 grid(chunks, rows);
  b200::launch(b200::sample_partial_kernel, dim3(grid), dim3(256), 0, stream, logits, ld, vocab, params, part_value, part_index, chunks);
  b200::launch(b200::sample_final_kernel, dim3(rows), dim3(32), 0, stream, part_value, part_index, params, vocab, out, chunks);
  if (int e = b200::launch_status()) return e;
  if (any_filtered) return launch_sample(logits, ld, vocab, params, out, rows, 1, stream);
  return 0;
}

extern "C" int b200_sample_chunked(const float* logits, int ld, int vocab, const int* params, int* out, int rows,
                                   int chunks, void* scratch, int any_filtered, cudaStream_t stream) {
  return sample_chunked(logits, ld, vocab, b200::RowParams{const_cast<int*>(params), nullptr}, out, rows, chunks, scratch,
                        any_filtered, stream);
}

// The same selection with the rows' parameters taken from the slot records (`records`: the table,
// `row_slots[i]`: the record of row i): the chosen token and the advanced counter are written back
// into the record as well as into `out`.
extern "C" int b200_sample_slots(const float* logits, int ld, int vocab, int* records, const int* row_slots, int* out,
                                 int rows, int chunks, void* scratch, int any_filtered, cudaStream_t stream) {
  if (records == nullptr || row_slots == nullptr) return B200_ERR_BAD_SIZE;
  return sample_chunked(logits, ld, vocab, b200::RowParams{records, row_slots}, out, rows, chunks, scratch, any_filtered, stream);
}
