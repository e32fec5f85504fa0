// bfloat16 matrix product on the 5th-generation tensor cores: C[M,N] = A[M,K] * W[N,K]^T (+ bias)
// with float32 accumulation in tensor memory (TMEM).  Three kernels share the roles below and
// differ in how tiles are handed to SMs: one CTA per 128 x 256 tile (persistent), pairs of CTAs
// on 256 x 256 tiles (cta_group::2), and stream-K for products with few tiles.
//   warp 0   producer: one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the
//            operands' 64-wide K blocks into a ring of shared-memory stages, signalling a "full"
//            mbarrier per stage;
//   warp 1   allocates TMEM; one lane issues tcgen05.mma (K = 16, four per stage) and commits
//            each stage's completion to its "empty" mbarrier and each tile's to "acc_full";
//   warps 2-5  epilogue: tcgen05.ld of the accumulator (each warp its quarter of the 128 TMEM
//            lanes), bias, SwiGLU or residual sum where asked for, conversion, store.  The
//            accumulator is double buffered, so the epilogue of a tile runs under the products
//            of the next.
// Both operands are K-major ("row . row^T"), which is how nn.Linear stores its weight
// (mini_llm/nn/attention.py:102-111), so no transposition is needed anywhere.
//
// Every wait on an mbarrier or a flag is bounded: after its limit of polls the kernel records an
// error code, stops issuing work, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"

namespace b200 {

constexpr int BM = 128;   // rows of the row operand per CTA = TMEM lanes
constexpr int BK = 64;    // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kStreamKMaxCtas = 256;   // slots of the stream-K workspace the caller provides

__device__ int g_gemm_error = 0;

// ------------------------------------------------------------------ the shared wrappers, as this file names them
// (mbarrier, TMA, fences, descriptors and tcgen05.ld live in tcgen05.cuh, shared with the attention kernels)

// The wait as a converged warp runs it: every lane waits, and all lanes get the same answer.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity) ? 1 : 0) != 0;
}
// shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr) { return umma_desc_sw128(smem_byte_addr, 16, 1024); }
// instruction descriptor, kind::f16: D = f32, A = B = bf16, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t umma_idesc(int n) { return umma_idesc_bf16(BM, n, 0); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  umma_bf16_ss(tmem_d, adesc, bdesc, idesc, accumulate);
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) { umma_commit_to(bar); }
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  tmem_ld_32(taddr, r);
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  tmem_ld_16(taddr, r);
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

template <typename OutT> __device__ __forceinline__ void store_out(OutT* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void store_row_32(float* dst, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
}
__device__ __forceinline__ void store_row_32(__nv_bfloat16* dst, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 q;
    q.x = pack_bf16(v[j], v[j + 1]);
    q.y = pack_bf16(v[j + 2], v[j + 3]);
    q.z = pack_bf16(v[j + 4], v[j + 5]);
    q.w = pack_bf16(v[j + 6], v[j + 7]);
    *reinterpret_cast<uint4*>(dst + j) = q;
  }
}

__device__ __forceinline__ void store_row_8(float* dst, const float* v) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store_row_8(__nv_bfloat16* dst, const float* v) {
  uint4 q;
  q.x = pack_bf16(v[0], v[1]);
  q.y = pack_bf16(v[2], v[3]);
  q.z = pack_bf16(v[4], v[5]);
  q.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(dst) = q;
}

struct GemmParams {
  void* c;
  const float* bias;
  int M, N, K, ldc;
  int vector_ok;      // rows of C start on 16-byte boundaries
  int accumulate;     // float output only: C += A W^T + bias instead of C = ...
  float* partials;    // stream-K: [grid][128][256] partial accumulators
  unsigned* flags;    // stream-K: [grid], zero between launches
  int splits;         // split-K: CTAs (one cluster) that share the K range of a tile, at most 8
  int a_rows;         // split-K: rows of the row operand's box, a multiple of 8 up to 128
  int bn, stages;     // split-K: columns per tile (a multiple of 32, at most 256), stages of the operand ring
};

// What the epilogue does with 32 consecutive accumulator columns of one row, starting at column nb of
// the product: bias, then either SiLU(gate) * up on interleaved blocks of eight, or the optional sum
// with what C holds, then conversion and 16-byte stores where the row allows them.
template <bool SWIGLU, typename OutT>
__device__ __forceinline__ void finish_chunk(float (&v)[32], const GemmParams& p, OutT* crow, int nb) {
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += nb + j < p.N ? p.bias[nb + j] : 0.f;
  }
  if constexpr (SWIGLU) {
    // [g0..7 | u0..7 | g8..15 | u8..15] -> 16 outputs at column nb / 2 (N is a multiple of 16)
    float h[16];
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gate = v[b * 16 + j], up = v[b * 16 + 8 + j];
        h[b * 8 + j] = __fdividef(gate, 1.f + __expf(-gate)) * up;     // 2 ulp; for huge negative gates 0, as the limit is
      }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      if (nb + b * 16 + 16 > p.N) continue;
      OutT* dst = crow + (nb >> 1) + b * 8;
      if (p.vector_ok) {
        store_row_8(dst, h + b * 8);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) store_out<OutT>(dst + j, h[b * 8 + j]);
      }
    }
  } else {
    const bool whole = p.vector_ok && nb + 32 <= p.N;
    if constexpr (sizeof(OutT) == 4) {
      if (p.accumulate) {
        const float* have = reinterpret_cast<const float*>(crow) + nb;
        if (whole) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 e = *reinterpret_cast<const float4*>(have + j);
            v[j] += e.x; v[j + 1] += e.y; v[j + 2] += e.z; v[j + 3] += e.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (nb + j < p.N) v[j] += have[j];
        }
      }
    }
    if (whole) {
      store_row_32(crow + nb, v);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) store_out<OutT>(crow + nb + j, v[j]);
    }
  }
}

// ---------------------------------------------------------------------- persistent kernel
// One CTA per SM walks over the output tiles (tile, tile + gridDim.x, ...; the 128-row blocks
// of one 256-column panel are neighbours, so a wave of CTAs shares few weight panels in L2).
// The accumulator is double buffered in TMEM (2 x 256 columns): while the epilogue warps
// drain tile i, the tensor core already works on tile i + 1.
// SWIGLU: the weight holds gate and up rows interleaved in blocks of eight; the epilogue
// writes silu(gate) * up, N / 2 columns wide, and the [M, N] intermediate never exists.
template <int BN, int STAGES, bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
                               GemmParams p) {
  static_assert(BN == 64 || BN == 128 || BN == 256, "tile widths: 64, 128, 256");
  constexpr uint32_t ROW_BYTES = BM * BK * 2, COL_BYTES = BN * BK * 2, STAGE_BYTES = ROW_BYTES + COL_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;    // [2]
  uint64_t* acc_empty = acc_full + 2;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full + b, 1);
      mbar_init(acc_empty + b, 4);     // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                             // set-up above overlaps the kernel before; its results are read below

  // Producer and tensor-core warp run their loops as whole warps and issue under elect_one(): see there.
  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      const int row0 = (tile % m_tiles) * BM, col0 = (tile / m_tiles) * BN;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_warp(empty + s, phase ^ 1)) { atomicExch(&g_gemm_error, 1); ok = false; break; }
        unsigned char* stage = smem + s * STAGE_BYTES;
        if (elect_one()) {
          mbar_expect_tx(full + s, STAGE_BYTES);
          tma_load_2d(stage, &map_rows, full + s, kb * BK, row0);
          tma_load_2d(stage + ROW_BYTES, &map_cols, full + s, kb * BK, col0);
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- tensor-core issue
    constexpr uint32_t idesc = umma_idesc(BN);
    int s = 0, local = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait_warp(acc_empty + buf, acc_phase ^ 1)) { atomicExch(&g_gemm_error, 4); ok = false; break; }
      tcgen05_fence_after();
      const uint32_t tmem_d = tmem_base + buf * BN;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_warp(full + s, phase)) { atomicExch(&g_gemm_error, 2); ok = false; break; }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_addr(smem + s * STAGE_BYTES), b_addr = a_addr + ROW_BYTES;
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_d, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc, (kb | k) != 0);
          umma_commit(empty + s);
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; phase ^= 1; }
      }
      if (elect_one()) umma_commit(acc_full + buf);
      __syncwarp();
    }
  } else if (warp >= 2) {
    // -------------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    int local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int row0 = (tile % m_tiles) * BM, col0 = (tile / m_tiles) * BN;
      const bool ok = mbar_wait(acc_full + buf, acc_phase);
      if (!ok) atomicExch(&g_gemm_error, 3);
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
      const int m = row0 + row;
      OutT* crow = static_cast<OutT*>(p.c) + static_cast<size_t>(m) * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        float v[32];
        if (ok) {
          tmem_load_32(taddr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        if (m < p.M) finish_chunk<SWIGLU, OutT>(v, p, crow, col0 + c);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(acc_empty + buf)) : "memory");
      }
      if (!ok) break;
    }
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------ 2-CTA kernel
// A pair of CTAs (a cluster of two, on neighbouring SMs) computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA brings in 128 rows of A and 128 of the 256 weight rows per
// 64-wide K block (32 KB instead of the 48 KB a CTA of the one-CTA kernel needs for the same
// 128 x 256 outputs) and keeps its 128 x 256 half of the accumulator in its own TMEM; the tensor
// core of the pair reads both halves of B.  Only the even CTA (the leader) issues MMAs.  Protocol
// per stage: both CTAs' TMA copies complete on the leader's `full` barrier (armed by the leader
// for the bytes of both); the leader's commit arrives on `empty` in both CTAs.  Per tile: the
// leader's commit arrives on `acc_full` in both CTAs; the eight epilogue warps of the pair arrive
// on the leader's `acc_empty`.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_address, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"(smem_address), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// TMA copy into this CTA's shared memory whose bytes are counted on a barrier of the pair's leader
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
          smem_addr(dst)),
      "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives, once the MMAs issued so far have finished, on the barrier at this address in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(
                   smem_addr(bar)),
               "h"(both)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_address) : "memory");
}
// instruction descriptor for the pair: M = 256 (128 rows per CTA)
__host__ __device__ constexpr uint32_t umma_idesc_pair(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
}

template <int STAGES, bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols, GemmParams p) {
  constexpr int BN = 256, HALF_N = 128, PAIR_M = 256;
  constexpr uint32_t ROW_BYTES = BM * BK * 2, COL_BYTES = HALF_N * BK * 2, STAGE_BYTES = ROW_BYTES + COL_BYTES;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;    // [2]
  uint64_t* acc_empty = acc_full + 2;     // [2], used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_tiles = (p.M + PAIR_M - 1) / PAIR_M, n_tiles = (p.N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full + b, 1);
      mbar_init(acc_empty + b, 8);     // one arrival per epilogue warp of the pair
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                     // both CTAs' barriers exist before anything arrives on them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                             // set-up above overlaps the kernel before; its results are read below

  if (warp == 0) {
    // ---------------------------------------------------------------- producer (both CTAs)
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair; tile < tiles && ok; tile += pairs) {
      const int row0 = (tile % m_tiles) * PAIR_M + static_cast<int>(rank) * BM;
      const int col0 = (tile / m_tiles) * BN + static_cast<int>(rank) * HALF_N;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_warp(empty + s, phase ^ 1)) { atomicExch(&g_gemm_error, 1); ok = false; break; }
        const uint32_t leader_full = map_to_cta(smem_addr(full + s), 0);
        unsigned char* stage = smem + s * STAGE_BYTES;
        if (elect_one()) {
          if (leader) mbar_expect_tx(full + s, 2 * STAGE_BYTES);
          tma_load_2d_pair(stage, &map_rows, leader_full, kb * BK, row0);
          tma_load_2d_pair(stage + ROW_BYTES, &map_cols, leader_full, kb * BK, col0);
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1 && leader) {
    // ---------------------------------------------------------------- tensor-core issue (leader)
    constexpr uint32_t idesc = umma_idesc_pair(BN);
    int s = 0, local = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair; tile < tiles && ok; tile += pairs, ++local) {
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait_warp(acc_empty + buf, acc_phase ^ 1)) { atomicExch(&g_gemm_error, 4); ok = false; break; }
      tcgen05_fence_after();
      const uint32_t tmem_d = tmem_base + buf * BN;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_warp(full + s, phase)) { atomicExch(&g_gemm_error, 2); ok = false; break; }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_addr(smem + s * STAGE_BYTES), b_addr = a_addr + ROW_BYTES;
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_pair(tmem_d, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc, (kb | k) != 0);
          umma_commit_pair(empty + s);
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; phase ^= 1; }
      }
      if (elect_one()) umma_commit_pair(acc_full + buf);
      __syncwarp();
    }
  } else if (warp >= 2) {
    // -------------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    int local = 0;
    for (int tile = pair; tile < tiles; tile += pairs, ++local) {
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int row0 = (tile % m_tiles) * PAIR_M + static_cast<int>(rank) * BM, col0 = (tile / m_tiles) * BN;
      const bool ok = mbar_wait(acc_full + buf, acc_phase);
      if (!ok) atomicExch(&g_gemm_error, 3);
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
      const int m = row0 + row;
      OutT* crow = static_cast<OutT*>(p.c) + static_cast<size_t>(m) * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        float v[32];
        if (ok) {
          tmem_load_32(taddr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        if (m < p.M) finish_chunk<SWIGLU, OutT>(v, p, crow, col0 + c);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_addr(acc_empty + buf), 0));
      if (!ok) break;
    }
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                     // the leader's MMAs read this CTA's shared memory until its last commit
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------ stream-K kernel
// One CTA per SM.  The tiles that fill whole rounds of gridDim.x CTAs are computed whole, round
// by round (tile = round * gridDim.x + CTA, so the CTAs of a round share few weight panels in L2).
// The tiles that are left, fewer than gridDim.x, would keep only some SMs busy for a whole tile's
// time; instead their (tile, 64-wide K block) pairs, tile-major, are cut into equal contiguous
// ranges, one per CTA, so that every SM does the same number of tensor-core steps.  Such a range
// may begin in the middle of a tile and end in the middle of another.  The CTA that holds K block
// 0 of a tile owns it: it runs that piece last, then adds what the CTAs after it computed for the
// rest of the tile's K range, and writes the result.  Those CTAs ran their piece first (it is the
// head of their range), wrote the accumulator to `partials` and raised their flag; the owner
// lowers the flags again, so they are zero when the kernel ends.  Nobody waits for an owner, so
// no wait depends on a CTA that has not started; the owner's wait for a flag is bounded.
// The partial sums of a tile are added in the order of the CTAs: the result depends on the shape
// of the product only, never on timing.
__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_release(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

struct StreamKPlan {
  int num_kb, ctas, rounds, first_left, sharers;   // sharers: CTAs that take part in the left-over tiles
  long long left_units;
  __device__ long long begin_of(int cta) const { return cta >= sharers ? left_units : left_units * cta / sharers; }
  // Calls f(tile, kb0, kb1, last_partner): the K blocks [kb0, kb1) of `tile`; for an owned tile whose K range
  // continues in other CTAs, those are blockIdx.x + 1 .. last_partner (else last_partner == blockIdx.x).
  template <typename F> __device__ __forceinline__ void for_each_piece(int cta, F&& f) const {
    for (int r = 0; r < rounds; ++r) f(r * ctas + cta, 0, num_kb, cta);
    const long long begin = begin_of(cta), end = begin_of(cta + 1);
    for (long long u = begin; u < end;) {
      const int t = static_cast<int>(u / num_kb), kb0 = static_cast<int>(u - static_cast<long long>(t) * num_kb);
      const int kb1 = static_cast<int>(min(static_cast<long long>(num_kb), kb0 + (end - u)));
      int last = cta;
      if (kb0 == 0 && kb1 < num_kb) {
        const long long tile_end = static_cast<long long>(t + 1) * num_kb;
        while (last + 1 < sharers && begin_of(last + 1) < tile_end) ++last;
      }
      f(first_left + t, kb0, kb1, last);
      u += kb1 - kb0;
    }
  }
};

// Element (row, column c) of a partial accumulator: 16-byte groups of four columns, the 128 rows of a
// group next to each other, so that a warp (32 rows) moves 512 contiguous bytes.
__device__ __forceinline__ float4* partial_group(float* base, int cta, int group, int row) {
  return reinterpret_cast<float4*>(base) + (static_cast<size_t>(cta) * 64 + group) * BM + row;
}

template <int BN, int STAGES, bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_streamk_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
                            GemmParams p) {
  static_assert(BN == 64 || BN == 128 || BN == 256, "tile widths: 64, 128, 256");
  constexpr uint32_t ROW_BYTES = BM * BK * 2, COL_BYTES = BN * BK * 2, STAGE_BYTES = ROW_BYTES + COL_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t kFlagSpins = 1u << 22;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;    // [2]
  uint64_t* acc_empty = acc_full + 2;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  StreamKPlan plan;
  plan.num_kb = (p.K + BK - 1) / BK;
  plan.ctas = gridDim.x;
  plan.rounds = tiles / plan.ctas;
  plan.first_left = plan.rounds * plan.ctas;
  const int left = tiles - plan.first_left;
  plan.left_units = static_cast<long long>(left) * plan.num_kb;
  // at most three CTAs per left-over tile: each further one costs the owner a pass over 128 KB
  plan.sharers = static_cast<int>(min(static_cast<long long>(min(plan.ctas, 3 * left)), plan.left_units));
  const int cta = blockIdx.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full + b, 1);
      mbar_init(acc_empty + b, 4);     // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                             // set-up above overlaps the kernel before; its results are read below

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    plan.for_each_piece(cta, [&](int tile, int kb0, int kb1, int) {
      const int row0 = (tile % m_tiles) * BM, col0 = (tile / m_tiles) * BN;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (!mbar_wait_warp(empty + s, phase ^ 1)) { atomicExch(&g_gemm_error, 1); ok = false; break; }
        unsigned char* stage = smem + s * STAGE_BYTES;
        if (elect_one()) {
          mbar_expect_tx(full + s, STAGE_BYTES);
          tma_load_2d(stage, &map_rows, full + s, kb * BK, row0);
          tma_load_2d(stage + ROW_BYTES, &map_cols, full + s, kb * BK, col0);
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; phase ^= 1; }
      }
    });
  } else if (warp == 1) {
    // ---------------------------------------------------------------- tensor-core issue
    constexpr uint32_t idesc = umma_idesc(BN);
    int s = 0, local = 0;
    uint32_t phase = 0;
    bool ok = true;
    plan.for_each_piece(cta, [&](int, int kb0, int kb1, int) {
      if (!ok) return;
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ++local;
      if (!mbar_wait_warp(acc_empty + buf, acc_phase ^ 1)) { atomicExch(&g_gemm_error, 4); ok = false; return; }
      tcgen05_fence_after();
      const uint32_t tmem_d = tmem_base + buf * BN;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_warp(full + s, phase)) { atomicExch(&g_gemm_error, 2); ok = false; return; }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_addr(smem + s * STAGE_BYTES), b_addr = a_addr + ROW_BYTES;
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_d, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc, ((kb - kb0) | k) != 0);
          umma_commit(empty + s);
        }
        __syncwarp();
        if (++s == STAGES) { s = 0; phase ^= 1; }
      }
      if (elect_one()) umma_commit(acc_full + buf);
      __syncwarp();
    });
  } else if (warp >= 2) {
    // -------------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    int local = 0;
    bool alive = true;
    plan.for_each_piece(cta, [&](int tile, int kb0, int kb1, int last_partner) {
      if (!alive) return;
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ++local;
      const int row0 = (tile % m_tiles) * BM, col0 = (tile / m_tiles) * BN;
      const bool ok = mbar_wait(acc_full + buf, acc_phase);
      if (!ok) { atomicExch(&g_gemm_error, 3); alive = false; }
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
      if (kb0 > 0) {
        // the rest of a tile that an earlier CTA owns: hand the accumulator over
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          float v[32];
          if (ok) {
            tmem_load_32(taddr + c, v);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            __stcg(partial_group(p.partials, cta, (c + j) >> 2, row), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(acc_empty + buf)) : "memory");
        __threadfence();
        epilogue_barrier();
        if (warp == 2 && lane == 0) store_release(p.flags + cta, 1u);
        return;
      }
      // owner: the CTAs cta + 1 .. last_partner hold the rest of the tile's K range
      for (int q = cta + 1; q <= last_partner; ++q) {
        uint32_t spins = 0;
        while (load_acquire(p.flags + q) == 0u) {
          if (++spins > kFlagSpins) { atomicExch(&g_gemm_error, 5); break; }
          __nanosleep(32);
        }
      }
      const int m = row0 + row;
      OutT* crow = static_cast<OutT*>(p.c) + static_cast<size_t>(m) * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        float v[32];
        float4 t[2][8];
        const int partners = last_partner - cta;
        // the loads of up to two partners are in flight while the accumulator comes out of TMEM
#pragma unroll
        for (int q = 0; q < 2; ++q)
          if (q < partners) {
#pragma unroll
            for (int j = 0; j < 8; ++j) t[q][j] = __ldcg(partial_group(p.partials, cta + 1 + q, (c >> 2) + j, row));
          }
        if (ok) {
          tmem_load_32(taddr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int q = 0; q < 2; ++q)
          if (q < partners) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              v[4 * j] += t[q][j].x; v[4 * j + 1] += t[q][j].y; v[4 * j + 2] += t[q][j].z; v[4 * j + 3] += t[q][j].w;
            }
          }
        for (int q = cta + 3; q <= last_partner; ++q) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 e = __ldcg(partial_group(p.partials, q, (c >> 2) + j, row));
            v[4 * j] += e.x; v[4 * j + 1] += e.y; v[4 * j + 2] += e.z; v[4 * j + 3] += e.w;
          }
        }
        if (m < p.M) finish_chunk<SWIGLU, OutT>(v, p, crow, col0 + c);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(acc_empty + buf)) : "memory");
      if (last_partner > cta) {
        epilogue_barrier();      // every epilogue thread has read the partners' sums
        if (warp == 2 && lane == 0)
          for (int q = cta + 1; q <= last_partner; ++q) p.flags[q] = 0u;
      }
    });
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------ split-K
// Products with so few tiles that one CTA per tile would leave most SMs without work (decoding
// batches of 17 to 128 rows, short prompt portions).  A cluster of `splits` CTAs takes one
// 128 x `bn` tile together, each a contiguous share of its K blocks, so that the weights stream
// in through every SM.  Each CTA moves its accumulator from tensor memory into its own shared
// memory (over the operand stages, which are done by then), the cluster meets at its barrier, and
// every CTA finishes its share of the tile: 1/splits of the (row, 32-column) pieces, summed over
// the CTAs' partial accumulators through distributed shared memory in the order of the K ranges.
// The result depends on the shape of the product only.  The hardware starts the CTAs of a cluster
// together, so no wait here depends on a CTA that has not started.  `bn` (a multiple of 32, at most
// 256) and the number of stages are run-time values: the tile width is chosen so that tiles x splits
// comes close to the number of SMs.
__device__ __forceinline__ float4 load_cluster_float4(uint32_t cluster_address) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(cluster_address) : "memory");
  return v;
}

template <bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_splitk_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
                           GemmParams p) {
  constexpr uint32_t TMEM_COLS = 256;
  const int bn = p.bn, stages = p.stages, splits = p.splits;
  // The row operand's box holds a_rows <= 128 rows (a product with fewer rows brings in no more than it
  // has); the MMA still reads 128 rows from the start of the stage, the rest of them being whatever
  // follows in shared memory: those rows of the accumulator belong to no row of C and are never read.
  const uint32_t ROW_BYTES = static_cast<uint32_t>(p.a_rows) * BK * 2;
  const uint32_t stage_bytes = ROW_BYTES + static_cast<uint32_t>(bn) * BK * 2;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + stages * stage_bytes + BM * BK * 2);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM;
  const int tile = blockIdx.x / splits, part = static_cast<int>(cluster_rank());
  const int row0 = (tile % m_tiles) * BM, col0 = (tile / m_tiles) * bn;
  const int num_kb = (p.K + BK - 1) / BK;
  const int kb0 = static_cast<int>(static_cast<long long>(num_kb) * part / splits);
  const int kb1 = static_cast<int>(static_cast<long long>(num_kb) * (part + 1) / splits);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int rows = min(BM, p.M - row0);
  const int quarter = warp & 3;
  const int row = quarter * 32 + lane;
  bool ok = true;
  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    // The weights do not depend on the kernel before this one: the first ring of weight tiles is asked
    // for while that kernel is still finishing, the activations only after the wait.
    const int ahead = min(stages, kb1 - kb0);
    if (elect_one()) {
      for (int i = 0; i < ahead; ++i) {
        mbar_expect_tx(full + i, stage_bytes);
        tma_load_2d(smem + i * stage_bytes + ROW_BYTES, &map_cols, full + i, (kb0 + i) * BK, col0);
      }
    }
    __syncwarp();
    pdl_wait();
    if (elect_one()) {
      for (int i = 0; i < ahead; ++i) tma_load_2d(smem + i * stage_bytes, &map_rows, full + i, (kb0 + i) * BK, row0);
    }
    __syncwarp();
    uint32_t phase = ahead == stages ? 1 : 0;
    for (int kb = kb0 + ahead, s = ahead == stages ? 0 : ahead; kb < kb1; ++kb) {
      if (!mbar_wait_warp(empty + s, phase ^ 1)) { atomicExch(&g_gemm_error, 1); break; }
      unsigned char* stage = smem + s * stage_bytes;
      if (elect_one()) {
        mbar_expect_tx(full + s, stage_bytes);
        tma_load_2d(stage, &map_rows, full + s, kb * BK, row0);
        tma_load_2d(stage + ROW_BYTES, &map_cols, full + s, kb * BK, col0);
      }
      __syncwarp();
      if (++s == stages) { s = 0; phase ^= 1; }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- tensor-core issue
    const uint32_t idesc = umma_idesc(bn);
    uint32_t phase = 0;
    for (int kb = kb0, s = 0; kb < kb1; ++kb) {
      if (!mbar_wait_warp(full + s, phase)) { atomicExch(&g_gemm_error, 2); break; }
      tcgen05_fence_after();
      const uint32_t a_addr = smem_addr(smem + s * stage_bytes), b_addr = a_addr + ROW_BYTES;
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16(tmem_base, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc, ((kb - kb0) | k) != 0);
        umma_commit(empty + s);
      }
      __syncwarp();
      if (++s == stages) { s = 0; phase ^= 1; }
    }
    if (elect_one()) umma_commit(acc_full);
    __syncwarp();
  } else if (warp >= 2) {
    // ---------------------------------------------- epilogue, first half: the accumulator leaves tensor memory
    pdl_wait();                           // C and the bias may be the work of the kernel before
    ok = kb1 > kb0 && mbar_wait(acc_full, 0);
    if (!ok) atomicExch(&g_gemm_error, 3);
    tcgen05_fence_after();
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    if (splits == 1) {
      const int m = row0 + row;
      OutT* crow = static_cast<OutT*>(p.c) + static_cast<size_t>(m) * p.ldc;
      if (quarter * 32 < rows) {
#pragma unroll 1
        for (int c = 0; c < bn; c += 32) {
          float v[32];
          if (ok) {
            tmem_load_32(taddr + c, v);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
          if (m < p.M) finish_chunk<SWIGLU, OutT>(v, p, crow, col0 + c);
        }
      }
    } else if (quarter * 32 < rows) {     // warps whose 32 rows all lie below the matrix have nothing to hand over
      // 16-byte groups of four columns, the 128 rows of a group next to each other: no bank conflicts here,
      // 512 contiguous bytes per warp for the CTA that reads them
      float4* mine = reinterpret_cast<float4*>(smem);
#pragma unroll 1
      for (int c = 0; c < bn; c += 32) {
        float v[32];
        if (ok) {
          tmem_load_32(taddr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4) mine[((c + j) >> 2) * BM + row] = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
    }
  }
  if (splits > 1) {
    __syncwarp();
    cluster_sync_all();                   // every CTA's partial accumulator is in its shared memory
    if (warp >= 2) {
      const uint32_t base = smem_addr(smem);
      const int pieces = rows * (bn / 32);
      const int begin = static_cast<int>(static_cast<long long>(pieces) * part / splits);
      const int end = static_cast<int>(static_cast<long long>(pieces) * (part + 1) / splits);
#pragma unroll 1
      for (int u = begin + static_cast<int>(threadIdx.x) - 64; u < end; u += 128) {
        const int chunk = u / rows, r = u - chunk * rows;
        const uint32_t offset = base + static_cast<uint32_t>((chunk * 8 * BM + r) * 16);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
#pragma unroll 1
        for (int q = 0; q < splits; q += 4) {   // the loads of four CTAs' pieces are in flight together
          float4 t[4][8];
#pragma unroll
          for (int h = 0; h < 4; ++h)
            if (q + h < splits) {
              const uint32_t remote = map_to_cta(offset, static_cast<uint32_t>(q + h));
#pragma unroll
              for (int j = 0; j < 8; ++j) t[h][j] = load_cluster_float4(remote + j * BM * 16);
            }
#pragma unroll
          for (int h = 0; h < 4; ++h)
            if (q + h < splits) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                v[4 * j] += t[h][j].x; v[4 * j + 1] += t[h][j].y; v[4 * j + 2] += t[h][j].z; v[4 * j + 3] += t[h][j].w;
              }
            }
        }
        const int m = row0 + r;
        finish_chunk<SWIGLU, OutT>(v, p, static_cast<OutT*>(p.c) + static_cast<size_t>(m) * p.ldc, col0 + chunk * 32);
      }
    }
    __syncwarp();
    cluster_sync_all();                   // nobody leaves while another CTA still reads its shared memory
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------ host side
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(ptr);
  }
  return fn;
}

// 2-D bf16 row-major [rows, cols] matrix, box = [box_rows, 64 columns], 128-byte swizzle
static int make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
  EncodeTiled fn = encode_fn();
  if (!fn) return 10005;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 10006;
}

template <int BN, int STAGES, bool SWIGLU, typename OutT>
static int launch_persistent(const CUtensorMap& rows, const CUtensorMap& cols, const GemmParams& p, cudaStream_t stream) {
  constexpr size_t smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 256;
  auto kernel = gemm_tcgen05_persistent_kernel<BN, STAGES, SWIGLU, OutT>;
  static b200::DeviceOnce once;
  int sm_count = 0;
  if (int e = b200::configure_once(once, kernel, smem, &sm_count)) return e;
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count ? tiles : sm_count;
  b200::launch(kernel, dim3(grid), dim3(kThreads), smem, stream, rows, cols, p);
  return static_cast<int>(cudaGetLastError());
}

template <int BN, int STAGES, bool SWIGLU, typename OutT>
static int launch_streamk(const CUtensorMap& rows, const CUtensorMap& cols, const GemmParams& p, cudaStream_t stream) {
  constexpr size_t smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 256;
  auto kernel = gemm_tcgen05_streamk_kernel<BN, STAGES, SWIGLU, OutT>;
  static b200::DeviceOnce once;
  int sm_count = 0;
  if (int e = b200::configure_once(once, kernel, smem, &sm_count)) return e;
  const long long units = static_cast<long long>((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * ((p.K + BK - 1) / BK);
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int grid = sm_count < kStreamKMaxCtas ? sm_count : kStreamKMaxCtas;
  if (3 * tiles < grid) grid = 3 * tiles;              // at most three CTAs share a tile
  if (units < grid) grid = static_cast<int>(units);
  b200::launch(kernel, dim3(grid), dim3(kThreads), smem, stream, rows, cols, p);
  return static_cast<int>(cudaGetLastError());
}

// Split-K: `splits` = 0 and `bn` = 0 ask for the choice made here.  The width is the one whose tiles,
// times the largest cluster that still fits, fill the SMs best, weighed by how much of a stage is weights
// (every CTA brings the activations in again beside its weight tile, so narrow tiles cost more traffic
// per weight byte).  The choice depends on N and K only, so a row's result does not depend on how many
// rows came along.
static int splitk_cluster(int tiles, int num_kb, int sm_count) {
  int s = 1;                              // 1, 2 or 4: clusters of three or of eight such CTAs rarely find room (two to three times slower)
  while (s < 4 && tiles * s * 2 <= sm_count && s * 2 <= num_kb) s *= 2;
  return s;
}
static void splitk_shape(int m_tiles, int N, int num_kb, int sm_count, int* bn, int* splits) {
  if (*bn <= 0) {
    double best = -1.;
    for (int width = 256; width >= 96; width -= 32) {
      const int tiles = m_tiles * ((N + width - 1) / width);
      const long ctas = static_cast<long>(tiles) * splitk_cluster(tiles, num_kb, sm_count);
      const long waves = (ctas + sm_count - 1) / sm_count;
      const double fill = static_cast<double>(ctas) / static_cast<double>(waves * sm_count);
      const double score = fill * width / (width + 64.);
      if (score > best + 1e-9) { best = score; *bn = width; }
    }
  }
  if (*splits <= 0) *splits = splitk_cluster(m_tiles * ((N + *bn - 1) / *bn), num_kb, sm_count);
}

template <bool SWIGLU, typename OutT>
static int launch_splitk(const CUtensorMap& rows, const CUtensorMap& cols, GemmParams p, cudaStream_t stream) {
  constexpr size_t kRing = 196 * 1024;                 // operand stages in flight per SM
  constexpr size_t kTail = BM * BK * 2 + 1024 + 512;   // what an MMA may read past a short row operand; alignment; barriers
  auto kernel = gemm_tcgen05_splitk_kernel<SWIGLU, OutT>;
  static b200::DeviceOnce once;
  if (int e = b200::configure_once(once, kernel, kRing + kTail)) return e;
  const size_t stage = static_cast<size_t>(p.a_rows + p.bn) * BK * 2;
  if (p.stages <= 0) p.stages = static_cast<int>(kRing / stage);
  if (p.stages > 16) p.stages = 16;
  // the partial accumulator (bn x 128 floats) lies over the stages
  if (p.stages < 2 || static_cast<size_t>(p.stages) * stage > kRing ||
      (p.splits > 1 && static_cast<size_t>(p.stages) * stage + BM * BK * 2 < static_cast<size_t>(p.bn) * BM * 4))
    return B200_ERR_BAD_SIZE;
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + p.bn - 1) / p.bn);
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(tiles * p.splits);
  config.blockDim = dim3(kThreads);
  // never two of these CTAs on one SM: two CTAs that shared an SM's tensor core (in the prefill attention) gave
  // results that changed from launch to launch; more than half of the shared memory keeps an SM to one CTA
  constexpr size_t kOnePerSm = 120 * 1024;
  config.dynamicSmemBytes = static_cast<size_t>(p.stages) * stage + kTail;
  if (config.dynamicSmemBytes < kOnePerSm) config.dynamicSmemBytes = kOnePerSm;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, rows, cols, p);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

template <int STAGES, bool SWIGLU, typename OutT>
static int launch_pair(const CUtensorMap& rows, const CUtensorMap& cols, const GemmParams& p, cudaStream_t stream) {
  constexpr size_t smem = STAGES * (BM * BK * 2 + 128 * BK * 2) + 1024 + 256;
  auto kernel = gemm_tcgen05_pair_kernel<STAGES, SWIGLU, OutT>;
  static b200::DeviceOnce once;
  int sm_count = 0;
  if (int e = b200::configure_once(once, kernel, smem, &sm_count)) return e;
  const int tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
  int pairs = sm_count / 2;
  if (tiles < pairs) pairs = tiles;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, rows, cols, p);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

}  // namespace b200

using namespace b200;

// Read and clear the error flag set by a bounded wait that ran out (0: none; 1: producer,
// 2: tensor-core issue, 3: epilogue).  Synchronises the device.
extern "C" int b200_gemm_tcgen05_error() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int));
  cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  return v;
}

// C[M,N] (ldc) = A[M,K] * W[N,K]^T + bias; out_f32 selects float or bfloat16 output.
// K must be a multiple of 8 and both bases 16-byte aligned (TMA); refused otherwise.
//   swiglu      W holds gate and up rows interleaved in blocks of eight (N a multiple of 16);
//               C = silu(gate) * up with N / 2 columns (ldc >= N / 2)
//   accumulate  float output without swiglu: C += A W^T + bias (the residual sum done where the product is)
//   kind        0: one CTA per 128 x tile_n tile, persistent; 1: pairs of CTAs on 256 x 256 tiles
//               (cta_group::2); 2: stream-K (left-over tiles shared between CTAs); 3: split-K (every
//               128 x tile_n tile shared by a cluster of `splits` <= 8 CTAs; tile_n a multiple of 32 up to
//               256; 0 for either: chosen from N and K so that the SMs are filled once; `stages`: depth of
//               the operand ring, 0 = as deep as shared memory allows)
//   tile_n      128 or 256 columns per tile (kind 0; the others take 256): narrower tiles put a product
//               with few rows on more SMs
//   partials, flags  stream-K only: b200_gemm_tcgen05_streamk_partial_floats() floats and
//               b200_gemm_tcgen05_streamk_flags() 32-bit words that are zero before the first launch
//               (the kernel leaves them zero); launches that share them must not overlap
extern "C" long b200_gemm_tcgen05_streamk_partial_floats() { return static_cast<long>(kStreamKMaxCtas) * BM * 256; }
extern "C" int b200_gemm_tcgen05_streamk_flags() { return kStreamKMaxCtas; }

// The tile width and cluster size the split-K kernel chooses for a product of M x N x K on a GPU with
// `sm_count` SMs (host arithmetic only: callable without a GPU).
extern "C" int b200_gemm_tcgen05_splitk_shape(int M, int N, int K, int sm_count, int* tile_n, int* splits) {
  if (M <= 0 || N <= 0 || K <= 0 || sm_count <= 0 || !tile_n || !splits) return B200_ERR_BAD_SIZE;
  *tile_n = 0;
  *splits = 0;
  splitk_shape((M + BM - 1) / BM, N, (K + BK - 1) / BK, sm_count, tile_n, splits);
  return 0;
}

template <int KIND, int BN, bool SWIGLU, typename OutT>
static int launch_kind(const CUtensorMap& rows, const CUtensorMap& cols, const GemmParams& p, cudaStream_t stream) {
  constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);      // 192 KB of stages in every case
  if constexpr (KIND == 0) return launch_persistent<BN, STAGES, SWIGLU, OutT>(rows, cols, p, stream);
  else if constexpr (KIND == 1) return launch_pair<6, SWIGLU, OutT>(rows, cols, p, stream);
  else if constexpr (KIND == 3) return launch_splitk<SWIGLU, OutT>(rows, cols, p, stream);
  else return launch_streamk<BN, STAGES, SWIGLU, OutT>(rows, cols, p, stream);
}
template <int KIND, int BN>
static int launch_variant(const CUtensorMap& rows, const CUtensorMap& cols, const GemmParams& p, int out_f32, int swiglu,
                          cudaStream_t stream) {
  if (swiglu)
    return out_f32 ? launch_kind<KIND, BN, true, float>(rows, cols, p, stream)
                   : launch_kind<KIND, BN, true, __nv_bfloat16>(rows, cols, p, stream);
  return out_f32 ? launch_kind<KIND, BN, false, float>(rows, cols, p, stream)
                 : launch_kind<KIND, BN, false, __nv_bfloat16>(rows, cols, p, stream);
}

extern "C" int b200_gemm_tcgen05(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int ldc,
                                 int out_f32, int swiglu, int accumulate, int kind, int tile_n, int splits, int stages,
                                 float* partials, unsigned* flags, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ldc < (swiglu ? N / 2 : N) || (swiglu && N % 16 != 0) || kind < 0 || kind > 3) return B200_ERR_BAD_SIZE;
  if (kind == 1) tile_n = 256;
  if (kind != 3 && tile_n != 128 && tile_n != 256) return B200_ERR_BAD_SIZE;
  if (accumulate && (!out_f32 || swiglu)) return B200_ERR_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return B200_ERR_BAD_SIZE;
  if (kind == 2 && (!partials || !flags || (reinterpret_cast<uintptr_t>(partials) & 15))) return 10004;
  GemmParams p{C, bias, M, N, K, ldc, (ldc % 8 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0, accumulate, partials, flags, splits, BM, tile_n, 0};
  CUtensorMap rows, cols;
  if (int e = make_map(&rows, A, M, K, BM)) return e;
  if (kind != 3)
    if (int e = make_map(&cols, W, N, K, kind == 1 ? 128 : tile_n)) return e;
  if (kind == 1) return launch_variant<1, 256>(rows, cols, p, out_f32, swiglu, stream);
  if (kind == 3) {
    int device = 0, sm_count = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    splitk_shape((M + BM - 1) / BM, N, (K + BK - 1) / BK, sm_count, &p.bn, &p.splits);
    if (p.bn % 32 || p.bn < 32 || p.bn > 256 || p.splits < 1 || p.splits > 8 || p.splits > (K + BK - 1) / BK) return B200_ERR_BAD_SIZE;
    p.a_rows = M >= BM ? BM : (M + 7) / 8 * 8;
    p.stages = stages;
    if (int e = make_map(&rows, A, M, K, p.a_rows)) return e;
    if (int e = make_map(&cols, W, N, K, p.bn)) return e;
    return launch_variant<3, 256>(rows, cols, p, out_f32, swiglu, stream);
  }
  if (kind == 2) {                       // stream-K is built for 256 columns
    if (tile_n != 256) return B200_ERR_BAD_SIZE;
    return launch_variant<2, 256>(rows, cols, p, out_f32, swiglu, stream);
  }
  if (tile_n == 128) return launch_variant<0, 128>(rows, cols, p, out_f32, swiglu, stream);
  return launch_variant<0, 256>(rows, cols, p, out_f32, swiglu, stream);
}
