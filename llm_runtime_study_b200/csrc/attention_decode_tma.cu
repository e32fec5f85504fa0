// Decode attention over the paged cache with the pages streamed by TMA (sm_100a).
//
// One query token per request.  A CTA owns one (request, KV head, part of the sequence) and up to
// eight query heads of that KV head's group; its four warps take the 16-key blocks of the part in
// turn.  Every warp runs its own ring of DEPTH stages: lane 0 asks the TMA unit for the K and V
// rows of a block (two or four 2 KB boxes, 128-byte swizzle, found through the block table) and the
// warp waits on the stage's mbarrier, so the bytes in flight do not cost registers or instructions.
// The products are the transposed ones: S^T = K Q^T (keys on the 16-row side of mma.sync m16n8k16,
// query heads on the 8-column side) and O^T += V^T P^T, with softmax statistics in float32.
// When the sequence is cut into parts, each CTA writes (max, sum, unnormalised output) of its part
// and takes a ticket; the CTA that draws the last ticket of its (request, KV head) adds the parts
// in their fixed order, so no second launch is needed and the result does not depend on which CTA
// came last.
//
// The kernel can also do what otherwise a kernel before it does for the one new token of every
// request (mini_llm/nn/attention.py:174-187: per-head RMS norm of q and k before the rotation,
// mini_llm/nn/norm.py:90; rotation of the pairs (i, i + d/2) by position * inv_freq[i],
// mini_llm/nn/rope.py:110-146; write of k and v at the token's position,
// mini_llm/cache/paged/store.py:51-60): given the raw rows of the stacked q/k/v projection, every CTA
// normalises and rotates its own query heads in registers, and the warp whose block of keys holds the
// new position computes the new key, patches it (and the new value) into the block in shared memory once
// the block has arrived, and stores both rows into the cache pages for the steps to come.  No block then
// depends on the kernel before, so all of a part's first blocks are asked for before the dependency wait.
//
// Sizes: head sizes that are multiples of 64 (HEAD_DIM at compile time), pages of a multiple of 16
// tokens, any number of heads and groups, no window.  Other shapes use the kernels of
// attention_mma.cu.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 64>"
#endif
#ifndef DECODE_DEPTH
#define DECODE_DEPTH 3
#endif

namespace b200 {

using bf16 = __nv_bfloat16;

constexpr int D = HEAD_DIM;
static_assert(D % 64 == 0 && D >= 64 && D <= 256, "head size must be a multiple of 64, at most 256");
constexpr int BOXES = D / 64;                 // 64-column TMA boxes per row of K or V
constexpr int KEYS = 16;                      // keys per block
constexpr int BOX_BYTES = KEYS * 128;         // 2 KB
constexpr int TENSOR_BYTES = BOXES * BOX_BYTES;
constexpr int STAGE_BYTES = 2 * TENSOR_BYTES; // K then V
constexpr int DEPTH = DECODE_DEPTH;
constexpr int WARPS = 4;
constexpr int RING_BYTES = WARPS * DEPTH * STAGE_BYTES;
constexpr int HEADS = 8;                      // query heads per CTA (the n side of the mma)
constexpr int MAX_SPLITS = 64;
constexpr int COMBINE_FLOATS = 2 * WARPS * HEADS + WARPS * HEADS * D;
static_assert(COMBINE_FLOATS * 4 <= RING_BYTES, "the combine buffers reuse the ring");
constexpr int SMEM_BYTES = RING_BYTES + 1024 /* alignment */ + 256 /* barriers */;

struct DecodeParams {
  const bf16* q;
  bf16* out;
  const int* kv_len;
  const int* block_table;
  int table_stride, page_size, page_shift;
  int nq, nkv, group, gs, slices;
  float scale_log2;
  int num_splits;
  float* part_o;        // [requests][nq][num_splits][D]
  float* part_ml;       // [requests][nq][num_splits][2]
  unsigned* tickets;    // [requests][nkv][slices], zero between launches
  int* error;
  // the new token's raw projections, when this kernel also prepares them (else nullptr and q is ready-made)
  const bf16* qkv;      // [requests][qkv_stride]: query heads, then key heads, then value heads, D columns each
  int qkv_stride;
  const float* q_weight;   // [D] or nullptr: RMS-norm weight of the query heads
  const float* k_weight;   // [D] or nullptr
  float eps;
  const float* inv_freq;   // [D / 2] or nullptr: no rotation
  bf16* k_pool;            // [pages][nkv][page_size][D], written at the new position
  bf16* v_pool;
  // A launch recorded into a CUDA graph has its grid fixed for good, sized (num_splits) for the longest sequence
  // the engine may ever hold.  How many of those parts a replay uses the host says before every replay, in
  // *live_parts (what it would choose for the batch's longest sequence); the CTAs of the parts beyond leave at once.
  const int* live_parts;   // nullptr: every launch uses num_splits parts
};

__device__ int g_decode_error = 0;

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void ldmatrix_x4_addr(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans_addr(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__global__ void __launch_bounds__(128) decode_attention_tma_kernel(const __grid_constant__ CUtensorMap kmap,
                                                                   const __grid_constant__ CUtensorMap vmap,
                                                                   DecodeParams p) {
  constexpr int KS = D / 16;                  // k-steps of S^T = K Q^T
  constexpr int MT = D / 16;                  // 16-row tiles of O^T
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + RING_BYTES);
  __shared__ float sm_pm[HEADS][MAX_SPLITS], sm_pl[HEADS][MAX_SPLITS];
  __shared__ int sm_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  if (threadIdx.x == 0) {
    for (int i = 0; i < WARPS * DEPTH; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
  }
  const int split = blockIdx.x, b = blockIdx.z;
  const int kvh = blockIdx.y / p.slices, slice = blockIdx.y % p.slices;
  const int head0 = kvh * p.group + slice * p.gs;
  const int heads_here = min(p.gs, p.group - slice * p.gs);
  const int* table = p.block_table + static_cast<size_t>(b) * p.table_stride;
  __syncthreads();

  // Lengths and block tables are uploaded before the step's first kernel; the pages of all keys but
  // the newest were written by earlier steps.  Only q, the newest key and the outputs depend on the
  // kernel before this one, so the first blocks can be asked for before the dependency wait.
  const int len = p.kv_len[b];
  int splits = p.num_splits;     // parts in use: all of the grid's, or as many as the host says this batch needs
  if (p.live_parts != nullptr) splits = max(1, min(*p.live_parts, p.num_splits));
  if (split >= splits) return;   // the whole CTA: nothing of it has touched a barrier or a ticket
  int chunk = (len + splits - 1) / splits;
  chunk = ((chunk + 63) / 64) * 64;
  const int c0 = split * chunk;
  const int c1 = min(c0 + chunk, len) - 1;    // last key of this CTA's part (c1 < c0: nothing to do)
  const int nblocks = c1 >= c0 ? (c1 - c0) / KEYS + 1 : 0;
  const int my_count = nblocks > warp ? (nblocks - warp + WARPS - 1) / WARPS : 0;
  unsigned char* ring = base + warp * DEPTH * STAGE_BYTES;
  uint64_t* full = bars + warp * DEPTH;

  // Page ids of this warp's blocks: lane l holds the id of block (32 r + l) of the warp for the
  // current round r of 32 blocks, read from the block table in one go instead of one dependent
  // global load per block; a block's id then comes out of a shuffle.
  auto load_round = [&](int round) -> int {
    const int i = 32 * round + lane;
    if (i >= my_count) return -1;
    const int t0 = c0 + (warp + WARPS * i) * KEYS;
    return table[p.page_shift >= 0 ? t0 >> p.page_shift : t0 / p.page_size];
  };
  auto row_of = [&](int i, int page) -> int {   // row of block i's first key in the pool seen as [rows][D]; -1: no page
    const int t0 = c0 + (warp + WARPS * i) * KEYS;
    const int slot = p.page_shift >= 0 ? t0 & (p.page_size - 1) : t0 % p.page_size;
    return page < 0 ? -1 : (page * p.nkv + kvh) * p.page_size + slot;
  };
  auto issue = [&](int i, int page) {         // one lane: ask for the K and V rows of this warp's i-th block
    const int row = row_of(i, page);
    unsigned char* stage = ring + (i % DEPTH) * STAGE_BYTES;
    uint64_t* bar = &full[i % DEPTH];
    if (row < 0) {                            // no page (never the case for a live sequence): complete the phase empty-handed
      mbar_arrive(bar);
      return;
    }
    mbar_expect_tx(bar, STAGE_BYTES);
#pragma unroll
    for (int box = 0; box < BOXES; ++box) {
      tma_load_2d(stage + box * BOX_BYTES, &kmap, bar, box * 64, row);
      tma_load_2d(stage + TENSOR_BYTES + box * BOX_BYTES, &vmap, bar, box * 64, row);
    }
  };
  int ids = load_round(0), ids_round = 0;     // ids of blocks 32 ids_round .. + 31
  auto page_of = [&](int i) -> int {          // all lanes call this together, i uniform and rising
    if (i >= 32 * (ids_round + 1)) {
      ++ids_round;
      ids = load_round(ids_round);
    }
    return __shfl_sync(0xffffffffu, ids, i & 31);
  };
  // blocks that cannot hold the newest key (index len - 1) go out before the wait
  const int newest_block = (len - 1 - c0) / KEYS;            // block of this part holding key len - 1, if it is here
  const bool newest_here = len - 1 >= c0 && len - 1 <= c1;
  int issued = 0;
  unsigned valid = 0;                         // bit s: the block now in stage s has a page
  auto start = [&](int i) {                   // all lanes
    const int page = page_of(i);
    valid = (valid & ~(1u << (i % DEPTH))) | (page >= 0 ? 1u << (i % DEPTH) : 0u);
    if (elect_one()) issue(i, page);          // one lane, but from a converged warp: operands stay in uniform registers
  };
  const bool fused = p.qkv != nullptr;   // the newest key is made here, not read: no block waits for the kernel before
  while (issued < my_count && issued < DEPTH && (fused || !(newest_here && warp + WARPS * issued == newest_block))) start(issued++);
  pdl_wait();
  while (issued < my_count && issued < DEPTH) start(issued++);

  // cosines and sines of the new position, one copy per warp (no CTA-wide meeting before the main loop)
  __shared__ float sm_cos[WARPS][D / 2], sm_sin[WARPS][D / 2];
  const bool rotate = fused && p.inv_freq != nullptr;
  if (rotate) {
    for (int j = lane; j < D / 2; j += 32) sincosf(static_cast<float>(len - 1) * p.inv_freq[j], &sm_sin[warp][j], &sm_cos[warp][j]);
    __syncwarp();
  }
  // The new key and value, held by the warp whose block they fall into: lane l has the pairs (j, j + D/2), j = l, l + 32, ...
  constexpr int PAIRS = D / 64;
  const bool patcher = fused && newest_here && len > 0 && warp == newest_block % WARPS;
  float knew_lo[PAIRS], knew_hi[PAIRS];
  uint32_t vnew[PAIRS];       // bf16 pair: v[j], v[j + D/2]
  if (patcher) {
    const bf16* krow = p.qkv + static_cast<size_t>(b) * p.qkv_stride + static_cast<size_t>(p.nq + kvh) * D;
    const bf16* vrow = p.qkv + static_cast<size_t>(b) * p.qkv_stride + static_cast<size_t>(p.nq + p.nkv + kvh) * D;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PAIRS; ++i) {
      const int j = lane + 32 * i;
      knew_lo[i] = __bfloat162float(krow[j]);
      knew_hi[i] = __bfloat162float(krow[j + D / 2]);
      ss += knew_lo[i] * knew_lo[i] + knew_hi[i] * knew_hi[i];
      const uint16_t a = *reinterpret_cast<const uint16_t*>(vrow + j), c = *reinterpret_cast<const uint16_t*>(vrow + j + D / 2);
      vnew[i] = static_cast<uint32_t>(a) | (static_cast<uint32_t>(c) << 16);
    }
    const float r = p.k_weight ? rsqrtf(warp_sum(ss) / static_cast<float>(D) + p.eps) : 1.f;
#pragma unroll
    for (int i = 0; i < PAIRS; ++i) {
      const int j = lane + 32 * i;
      float a = knew_lo[i], c = knew_hi[i];
      if (p.k_weight) {
        a *= r * p.k_weight[j];
        c *= r * p.k_weight[j + D / 2];
      }
      if (rotate) {
        const float co = sm_cos[warp][j], si = sm_sin[warp][j];
        knew_lo[i] = a * co - c * si;
        knew_hi[i] = c * co + a * si;
      } else {
        knew_lo[i] = a;
        knew_hi[i] = c;
      }
    }
    if (slice == 0) {   // one CTA per (request, KV head) stores the rows for the steps to come
      const int pos = len - 1;
      const int page = table[p.page_shift >= 0 ? pos >> p.page_shift : pos / p.page_size];
      if (page >= 0) {
        const size_t row = (static_cast<size_t>(page) * p.nkv + kvh) * p.page_size + (p.page_shift >= 0 ? pos & (p.page_size - 1) : pos % p.page_size);
        bf16* kdst = p.k_pool + row * D;
        bf16* vdst = p.v_pool + row * D;
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
          const int j = lane + 32 * i;
          kdst[j] = __float2bfloat16_rn(knew_lo[i]);
          kdst[j + D / 2] = __float2bfloat16_rn(knew_hi[i]);
          *reinterpret_cast<uint16_t*>(vdst + j) = static_cast<uint16_t>(vnew[i] & 0xffffu);
          *reinterpret_cast<uint16_t*>(vdst + j + D / 2) = static_cast<uint16_t>(vnew[i] >> 16);
        }
      }
    }
  }

  // Q^T as B fragments: lane (g, t) holds Q[head g][16 ks + 2t, +1] and Q[head g][16 ks + 8 + 2t, +1]
  uint32_t qb[KS][2];
  {
    const bf16* qrow = fused ? p.qkv + static_cast<size_t>(b) * p.qkv_stride + static_cast<size_t>(head0 + g) * D
                             : p.q + (static_cast<size_t>(b) * p.nq + head0 + g) * D;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qb[ks][0] = qb[ks][1] = 0u;
      if (g < heads_here) {
        qb[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t);
        qb[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t + 8);
      }
    }
  }
  if (fused && (p.q_weight != nullptr || rotate)) {
    // this lane's 4 KS elements of head g: columns 16 ks + 2t, +1, +8, +9; the other half of a rotation pair
    // (column + D/2) is in the same lane, KS/2 steps on.  The sum of squares of a head is spread over the
    // four lanes of a quad.
    float v[KS][4];
    float ss = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qb[ks][0]));
      const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qb[ks][1]));
      v[ks][0] = a.x; v[ks][1] = a.y; v[ks][2] = c.x; v[ks][3] = c.y;
      ss += a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y;
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    if (p.q_weight) {
      const float r = rsqrtf(ss / static_cast<float>(D) + p.eps);
#pragma unroll
      for (int ks = 0; ks < KS; ++ks)
#pragma unroll
        for (int e = 0; e < 4; ++e) v[ks][e] *= r * p.q_weight[16 * ks + 2 * t + (e & 1) + (e >> 1) * 8];
    }
    if (rotate) {
#pragma unroll
      for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = 16 * ks + 2 * t + (e & 1) + (e >> 1) * 8;        // < D / 2
          const float co = sm_cos[warp][j], si = sm_sin[warp][j];
          const float a = v[ks][e], c = v[ks + KS / 2][e];
          v[ks][e] = a * co - c * si;
          v[ks + KS / 2][e] = c * co + a * si;
        }
    }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qb[ks][0] = g < heads_here ? pack_bf16(v[ks][0], v[ks][1]) : 0u;
      qb[ks][1] = g < heads_here ? pack_bf16(v[ks][2], v[ks][3]) : 0u;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};   // heads 2t and 2t + 1
  float o[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[mt][e] = 0.f;

  // ldmatrix lane roles: K (A operand, rows = keys): row (lane & 7) + 8 ((lane >> 3) & 1), 16-byte chunk 2 ks + (lane >> 4);
  // V^T (A operand through .trans, rows of the tile = keys): key (lane & 7) + 8 ((lane >> 4) & 1), chunk 2 mt + ((lane >> 3) & 1)
  const int k_row = (lane & 7) + ((lane >> 3) & 1) * 8, k_half = lane >> 4;
  const int v_key = (lane & 7) + ((lane >> 4) & 1) * 8, v_half = (lane >> 3) & 1;

  for (int i = 0; i < my_count; ++i) {
    const int t0 = c0 + (warp + WARPS * i) * KEYS;
    if (!mbar_wait(&full[i % DEPTH], (i / DEPTH) & 1)) {
      if (lane == 0) atomicExch(p.error, 1);
      break;
    }
    if ((valid >> (i % DEPTH)) & 1u) {        // else: no page, nothing was copied into the stage
      const uint32_t kbase = smem_addr(ring + (i % DEPTH) * STAGE_BYTES), vbase = kbase + TENSOR_BYTES;
      if (patcher && warp + WARPS * i == newest_block) {
        // the block that holds the new position: put the new key and value where the cache's (not yet written,
        // or being written right now) rows were copied to
        unsigned char* kst = ring + (i % DEPTH) * STAGE_BYTES;
        const int r = len - 1 - t0;
#pragma unroll
        for (int q = 0; q < PAIRS; ++q) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int col = lane + 32 * q + half * (D / 2);
            const int off = (col >> 6) * BOX_BYTES + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4) + (col & 7) * 2;
            *reinterpret_cast<bf16*>(kst + off) = __float2bfloat16_rn(half ? knew_hi[q] : knew_lo[q]);
            *reinterpret_cast<uint16_t*>(kst + TENSOR_BYTES + off) = static_cast<uint16_t>(half ? vnew[q] >> 16 : vnew[q] & 0xffffu);
          }
        }
        __syncwarp();
      }
      if (t0 + KEYS - 1 > c1) {
        // rows past the end of the sequence hold whatever the page held before: their scores are
        // masked below, their values are cleared here so that 0 x (stale) cannot become NaN
        const int first = c1 - t0 + 1;
        for (int c = lane; c < (KEYS - first) * (D / 8); c += 32) {
          const int r = first + c / (D / 8), ch = c % (D / 8);
          *reinterpret_cast<uint4*>(ring + (i % DEPTH) * STAGE_BYTES + TENSOR_BYTES + (ch >> 3) * BOX_BYTES + r * 128 + (ch & 7) * 16) =
              make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int chunk16 = 2 * ks + k_half;
        uint32_t a[4];
        ldmatrix_x4_addr(a, kbase + (chunk16 >> 3) * BOX_BYTES + k_row * 128 + (((chunk16 & 7) ^ (k_row & 7)) << 4));
        mma_bf16(c, a, qb[ks][0], qb[ks][1]);
      }
      // c0, c1: key t0 + g, heads 2t, 2t+1;  c2, c3: key t0 + g + 8
      const bool vis_a = t0 + g <= c1, vis_b = t0 + g + 8 <= c1;
      c[0] = vis_a ? c[0] * p.scale_log2 : -INFINITY;
      c[1] = vis_a ? c[1] * p.scale_log2 : -INFINITY;
      c[2] = vis_b ? c[2] * p.scale_log2 : -INFINITY;
      c[3] = vis_b ? c[3] * p.scale_log2 : -INFINITY;
      float mx[2] = {fmaxf(c[0], c[2]), fmaxf(c[1], c[3])};
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], off));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], off));
      }
      float corr[2], ref[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float m_new = fmaxf(m[h], mx[h]);
        ref[h] = m_new == -INFINITY ? 0.f : m_new;
        corr[h] = exp2f(m[h] - ref[h]);
        m[h] = m_new;
        l[h] *= corr[h];
      }
      const float p0 = exp2f(c[0] - ref[0]), p1 = exp2f(c[1] - ref[1]), p2 = exp2f(c[2] - ref[0]), p3 = exp2f(c[3] - ref[1]);
      l[0] += p0 + p2;
      l[1] += p1 + p3;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        o[mt][0] *= corr[0];
        o[mt][1] *= corr[1];
        o[mt][2] *= corr[0];
        o[mt][3] *= corr[1];
      }
      // P^T [keys x heads] -> B fragments [k = keys][n = heads]
      const uint32_t pb0 = movmatrix_trans(pack_bf16(p0, p1));
      const uint32_t pb1 = movmatrix_trans(pack_bf16(p2, p3));
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int chunk16 = 2 * mt + v_half;
        uint32_t vf[4];
        ldmatrix_x4_trans_addr(vf, vbase + (chunk16 >> 3) * BOX_BYTES + v_key * 128 + (((chunk16 & 7) ^ (v_key & 7)) << 4));
        mma_bf16(o[mt], vf, pb0, pb1);
      }
    }
    __syncwarp();
    if (i + DEPTH < my_count) {
      if (lane == 0) fence_async_shared();
      start(i + DEPTH);
    }
  }
  __syncthreads();

  // combine the four warps through shared memory (the ring is idle now)
  float* sm_m = reinterpret_cast<float*>(base);       // [4][8]
  float* sm_l = sm_m + WARPS * HEADS;                 // [4][8]
  float* sm_o = sm_l + WARPS * HEADS;                 // [4][8 heads][D]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float total = l[h];
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
    if (g == 0) {
      sm_m[warp * HEADS + 2 * t + h] = m[h];
      sm_l[warp * HEADS + 2 * t + h] = total;
    }
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    sm_o[(warp * HEADS + 2 * t) * D + mt * 16 + g] = o[mt][0];
    sm_o[(warp * HEADS + 2 * t + 1) * D + mt * 16 + g] = o[mt][1];
    sm_o[(warp * HEADS + 2 * t) * D + mt * 16 + g + 8] = o[mt][2];
    sm_o[(warp * HEADS + 2 * t + 1) * D + mt * 16 + g + 8] = o[mt][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < heads_here * D; idx += 128) {
    const int h = idx / D, col = idx - h * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_m[w * HEADS + h]);
    const float ref = M == -INFINITY ? 0.f : M;
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float f = exp2f(sm_m[w * HEADS + h] - ref);
      acc += sm_o[(w * HEADS + h) * D + col] * f;
      L += sm_l[w * HEADS + h] * f;
    }
    const int head = head0 + h;
    if (splits == 1) {
      p.out[(static_cast<long>(b) * p.nq + head) * D + col] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      const long slot = (static_cast<long>(b) * p.nq + head) * p.num_splits + split;
      p.part_o[slot * D + col] = acc;
      if (col == 0) {
        p.part_ml[slot * 2] = M;
        p.part_ml[slot * 2 + 1] = L;
      }
    }
  }
  if (splits == 1) return;

  // ticket: the CTA that finishes last among the parts of this (request, KV head, slice) adds them up
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned old = atomicInc(&p.tickets[(static_cast<size_t>(b) * p.nkv + kvh) * p.slices + slice], splits - 1);
    sm_last = old == static_cast<unsigned>(splits - 1);   // atomicInc wraps to zero: ready for the next launch
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < heads_here * splits; idx += 128) {
    const int h = idx / splits, s = idx - h * splits;
    const long slot = (static_cast<long>(b) * p.nq + head0 + h) * p.num_splits + s;
    sm_pm[h][s] = __ldcg(p.part_ml + slot * 2);
    sm_pl[h][s] = __ldcg(p.part_ml + slot * 2 + 1);
  }
  __syncthreads();
  // four neighbouring columns per thread, the loads of eight parts in flight at a time
  for (int idx = threadIdx.x; idx < heads_here * (D / 4); idx += 128) {
    const int h = idx / (D / 4), col = (idx - h * (D / 4)) * 4;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, sm_pm[h][s]);
    const float ref = M == -INFINITY ? 0.f : M;
    const float* part = p.part_o + (static_cast<long>(b) * p.nq + head0 + h) * p.num_splits * D + col;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float L = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < splits) v[u] = __ldcg(reinterpret_cast<const float4*>(part + static_cast<long>(s0 + u) * D));
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < splits) {           // parts are added in their order, whatever the order of arrival
          const float f = exp2f(sm_pm[h][s0 + u] - ref);
          acc[0] += v[u].x * f;
          acc[1] += v[u].y * f;
          acc[2] += v[u].z * f;
          acc[3] += v[u].w * f;
          L += sm_pl[h][s0 + u] * f;
        }
    }
    bf16* dst = p.out + (static_cast<long>(b) * p.nq + head0 + h) * D + col;
    uint2 packed;
    packed.x = pack_bf16(L > 0.f ? acc[0] / L : 0.f, L > 0.f ? acc[1] / L : 0.f);
    packed.y = pack_bf16(L > 0.f ? acc[2] / L : 0.f, L > 0.f ? acc[3] / L : 0.f);
    *reinterpret_cast<uint2*>(dst) = packed;
  }
}

// Tensor maps over a pool seen as [rows][D] bfloat16, boxes of 16 rows x 64 columns, 128-byte swizzle.
// Encoding costs a microsecond or two on the host, so the maps of the pools seen so far are kept.
struct CachedMap {
  const void* base;
  uint64_t rows;
  CUtensorMap map;
};
static int pool_map(const void* base, uint64_t rows, CUtensorMap* out) {
  constexpr int kSlots = 1024;
  static CachedMap cache[kSlots];
  static int used = 0;
  for (int i = 0; i < used; ++i)
    if (cache[i].base == base && cache[i].rows == rows) {
      *out = cache[i].map;
      return 0;
    }
  EncodeTiledFn fn = tensor_map_encoder();
  if (!fn) return 10005;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(D), rows};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(D) * 2};
  const cuuint32_t box[2] = {64, KEYS};
  const cuuint32_t elem[2] = {1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return 10006;
  if (used < kSlots) {
    cache[used].base = base;
    cache[used].rows = rows;
    cache[used].map = *out;
    ++used;
  }
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_attention_decode_tma_head_dim() { return HEAD_DIM; }
// CTAs of the kernel that fit on an SM: shared memory (ring, static arrays, 1 KB the system keeps per
// CTA) or registers (128 threads of up to 128 registers: four CTAs), whichever is less.
extern "C" int b200_attention_decode_tma_ctas_per_sm() {
  const int by_smem = (227 * 1024) / (SMEM_BYTES + 1024 + 2 * HEADS * MAX_SPLITS * 4 + 2 * WARPS * (D / 2) * 4);
  return by_smem < 4 ? by_smem : 4;
}

extern "C" long b200_attention_decode_tma_scratch_floats(int requests, int nq, int num_splits) {
  return num_splits <= 1 ? 0 : static_cast<long>(requests) * nq * num_splits * (D + 2);
}
// Tickets the caller keeps, zeroed once: one per (request, KV head, slice of the group).
extern "C" long b200_attention_decode_tma_tickets(int requests, int nq, int nkv) {
  if (nq <= 0 || nkv <= 0 || nq % nkv) return -1;
  const int group = nq / nkv, gs = group < HEADS ? group : HEADS;
  return static_cast<long>(requests) * nkv * ((group + gs - 1) / gs);
}

// 0: no wait of the kernel ever gave up; 1: a TMA copy did not arrive within the poll limit.
extern "C" int b200_attention_decode_tma_error() {
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, g_decode_error, sizeof(int)) != cudaSuccess) return -1;
  return value;
}

// What the fused form adds to a launch: the raw q/k/v rows and the constants of the norm and the rotation.
struct FusedInputs {
  const void* qkv = nullptr;
  int qkv_stride = 0;
  const float* q_weight = nullptr;
  const float* k_weight = nullptr;
  float eps = 0.f;
  const float* inv_freq = nullptr;
  const int* live_parts = nullptr;     // see DecodeParams
};

static int decode_tma(const void* q, const FusedInputs& fused, const void* k_pool, const void* v_pool, void* out, const int* kv_len,
                      const int* block_table, int table_stride, int page_size, int num_pages, int requests,
                      int nq, int nkv, float scale, int num_splits, float* scratch, long scratch_floats,
                      unsigned* tickets, long ticket_count, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || page_size % KEYS != 0 || table_stride <= 0 || num_pages <= 0)
    return B200_ERR_BAD_SIZE;
  if (num_splits < 1 || num_splits > MAX_SPLITS || requests > 65535) return B200_ERR_BAD_SIZE;
  const uint64_t rows = static_cast<uint64_t>(num_pages) * nkv * page_size;
  if (rows >= (1ull << 31)) return B200_ERR_TOO_LARGE;
  if (scratch_floats < b200_attention_decode_tma_scratch_floats(requests, nq, num_splits)) return 10004;
  if (num_splits > 1 && (tickets == nullptr || ticket_count < b200_attention_decode_tma_tickets(requests, nq, nkv))) return 10004;
  if (fused.qkv != nullptr && (fused.qkv_stride < (nq + 2 * nkv) * D || (reinterpret_cast<uintptr_t>(fused.qkv) & 3) || (fused.qkv_stride & 1)))
    return B200_ERR_BAD_SIZE;
  DecodeParams p{};
  p.q = static_cast<const bf16*>(q);
  p.qkv = static_cast<const bf16*>(fused.qkv);
  p.qkv_stride = fused.qkv_stride;
  p.q_weight = fused.q_weight;
  p.k_weight = fused.k_weight;
  p.eps = fused.eps;
  p.inv_freq = fused.inv_freq;
  p.live_parts = fused.live_parts;
  p.k_pool = static_cast<bf16*>(const_cast<void*>(k_pool));
  p.v_pool = static_cast<bf16*>(const_cast<void*>(v_pool));
  p.out = static_cast<bf16*>(out);
  p.kv_len = kv_len;
  p.block_table = block_table;
  p.table_stride = table_stride;
  p.page_size = page_size;
  p.page_shift = -1;
  for (int s = 0; s < 20; ++s)
    if ((1 << s) == page_size) p.page_shift = s;
  p.nq = nq;
  p.nkv = nkv;
  p.group = nq / nkv;
  p.gs = p.group < HEADS ? p.group : HEADS;
  p.slices = (p.group + p.gs - 1) / p.gs;
  if (static_cast<long>(nkv) * p.slices > 65535) return B200_ERR_TOO_LARGE;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_splits = num_splits;
  p.part_o = scratch;
  p.part_ml = scratch + static_cast<long>(requests) * nq * num_splits * D;
  p.tickets = tickets;
  static int* error_address[kMaxDevices] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 10007;
  if (!error_address[device] &&
      cudaGetSymbolAddress(reinterpret_cast<void**>(&error_address[device]), g_decode_error) != cudaSuccess)
    return 10007;
  p.error = error_address[device];
  CUtensorMap kmap, vmap;
  if (int e = pool_map(k_pool, rows, &kmap)) return e;
  if (int e = pool_map(v_pool, rows, &vmap)) return e;
  static DeviceOnce once;
  if (int e = configure_once(once, decode_attention_tma_kernel, SMEM_BYTES)) return e;
  dim3 grid(num_splits, nkv * p.slices, requests);
  launch(decode_attention_tma_kernel, grid, dim3(128), SMEM_BYTES, stream, kmap, vmap, p);
  return launch_status();
}

extern "C" int b200_attention_decode_tma(const void* q, const void* k_pool, const void* v_pool, void* out, const int* kv_len,
                                         const int* block_table, int table_stride, int page_size, int num_pages, int requests,
                                         int nq, int nkv, float scale, int num_splits, float* scratch, long scratch_floats,
                                         unsigned* tickets, long ticket_count, const int* live_parts, cudaStream_t stream) {
  FusedInputs plain;
  plain.live_parts = live_parts;
  return decode_tma(q, plain, k_pool, v_pool, out, kv_len, block_table, table_stride, page_size, num_pages, requests, nq,
                    nkv, scale, num_splits, scratch, scratch_floats, tickets, ticket_count, stream);
}

// The same attention for the one new token of every request, starting from the raw rows of the stacked q/k/v
// projection (`qkv`: [requests][qkv_stride], query heads, key heads, value heads): the kernel normalises
// (weights optional) and rotates (inv_freq optional, whole head) q and the new k itself, writes the new k and v
// into the pools at position kv_len - 1, and attends over all kv_len keys.
extern "C" int b200_attention_decode_tma_fused(const void* qkv, int qkv_stride, const float* q_weight, const float* k_weight,
                                               float eps, const float* inv_freq, void* k_pool, void* v_pool, void* out,
                                               const int* kv_len, const int* block_table, int table_stride, int page_size,
                                               int num_pages, int requests, int nq, int nkv, float scale, int num_splits,
                                               float* scratch, long scratch_floats, unsigned* tickets, long ticket_count,
                                               const int* live_parts, cudaStream_t stream) {
  if (qkv == nullptr) return B200_ERR_BAD_SIZE;
  FusedInputs fused;
  fused.live_parts = live_parts;
  fused.qkv = qkv;
  fused.qkv_stride = qkv_stride;
  fused.q_weight = q_weight;
  fused.k_weight = k_weight;
  fused.eps = eps;
  fused.inv_freq = inv_freq;
  return decode_tma(nullptr, fused, k_pool, v_pool, out, kv_len, block_table, table_stride, page_size, num_pages, requests, nq,
                    nkv, scale, num_splits, scratch, scratch_floats, tickets, ticket_count, stream);
}
