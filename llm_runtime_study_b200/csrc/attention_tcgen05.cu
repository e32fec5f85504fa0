// bfloat16 causal attention over the paged cache on the 5th-generation tensor cores, for
// batches that hold prompt portions.  Built once per head size (-DHEAD_DIM=64 or 128).
//
// One CTA owns 128 rows of S = Q K^T: up to 128 / gs consecutive query tokens of one request
// times the gs query heads that share one KV head.  Keys are taken 64 at a time:
//   warp 4     TMA loads: the Q tile once (3-D map over [token, head, d]), then for every key tile
//              the request's pages of K and V (rings of four or eight stages, running that far ahead), one box
//              per page and 64-column half, found through the block table, each lane issuing one;
//   warp 5     allocates TMEM; one lane issues tcgen05.mma: S = Q K^T (M 128, N 64, K = head size)
//              into one of two S buffers in TMEM - the product for the next tile is issued before
//              the softmax of the current one is awaited - and, once P is in tensor memory,
//              O += P V (M 128, N = head size, K 64) with P as the TMEM operand and V read from
//              shared memory as an MN-major operand (no transposition of the cache);
//   warps 0-3  softmax: thread r owns row r of S (tcgen05.ld gives a thread its whole row, so
//              the row maximum and sum need no shuffles); it masks, exponentiates in float32,
//              writes P as bfloat16 over its own row of S in tensor memory (tcgen05.st, two values
//              per column), and keeps the running maximum and sum.  O stays in TMEM; it is only
//              rescaled (tcgen05.ld / st) when a row's maximum has grown by more than 2^8, which
//              keeps the result exact (the final division uses the same reference maximum).
// One CTA per SM.  (Two used to share an SM, one's softmax overlapping the other's products; their results changed
// from launch to launch once tiles were started longest first, also with every hand-over below in place, and not
// with an SM to each CTA.  Two more faults showed on the way and are closed: a softmax warp that ran a tile ahead
// arrived on the barrier of the tile before - there is one P barrier per S buffer now - and S(j+1) was written
// over P(j-1) while P(j-1) V was still reading it.)
//
// Formula (mini_llm/nn/attention.py:95-99, 231-248): S = q.k^T * scale, key t visible iff
// t <= p, P = softmax(S), o = P.v; query head j reads KV head j / (nq / nkv).
// Every wait on an mbarrier is bounded; a wait that runs out records an error code, the CTA
// stops issuing work, frees its TMEM and returns.
#include "common.cuh"
#include "tcgen05.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=64 or 128"
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "this kernel is built for head sizes 64 and 128");

namespace b200 {

using bf16 = __nv_bfloat16;
constexpr int D = HEAD_DIM;
constexpr int BM = 128;                    // rows per CTA = TMEM lanes
constexpr int BN = 64;                     // keys per tile
constexpr int DSUB = D / 64;               // 64-column (128-byte) sub-tiles of the head size
constexpr uint32_t Q_SUB = BM * 128;       // bytes of one Q sub-tile
constexpr uint32_t KV_SUB = BN * 128;      // bytes of one K or V sub-tile
constexpr uint32_t Q_BYTES = DSUB * Q_SUB, KV_BYTES = DSUB * KV_SUB;
// One CTA per SM (the ring takes more than half of an SM's shared memory on purpose): two CTAs that share an SM's
// tensor core gave results that changed from launch to launch (see the note at the top), and a ring this deep keeps
// the copies of several key tiles in flight, which is what the second CTA was there to hide.
constexpr int KSTAGES = D == 128 ? 4 : 8;
constexpr uint32_t SMEM_TILES = Q_BYTES + 2 * KSTAGES * KV_BYTES;
static_assert(SMEM_TILES > 116 * 1024, "one CTA per SM");
constexpr uint32_t kBarrierBytes = 512;
static_assert((1 + 4 * KSTAGES + 2 + 2 + 1) * 8 + 4 <= kBarrierBytes, "barriers");
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t S_COL = 0, O_COL = 2 * BN;   // two S buffers of 64 columns, then O
constexpr int kTcThreads = 192;
constexpr float kRescaleStep = 8.f;        // log2 units a row maximum may lag behind

__device__ int g_attn_error = 0;

// 2^x for x <= 0 in one MUFU instruction (exp2f() adds range handling that is not needed here:
// results below the normal range may flush to zero, which is what a vanishing weight should do)
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

struct TcAttnParams {
  bf16* out;
  const int* positions;
  const int* block_table;
  int table_stride, page_size, page_shift;
  int nq, nkv, group, gs, slices;
  float scale_log2;
  const int* tile_entry;
  const int* tile_start;
  const int* tile_count;
};

__global__ void __launch_bounds__(kTcThreads)
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* q_smem = smem;
  unsigned char* k_smem = q_smem + Q_BYTES;                 // [KSTAGES]
  unsigned char* v_smem = k_smem + KSTAGES * KV_BYTES;      // [KSTAGES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_TILES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                 // [KSTAGES]
  uint64_t* k_empty = k_full + KSTAGES;
  uint64_t* v_full = k_empty + KSTAGES;
  uint64_t* v_empty = v_full + KSTAGES;
  uint64_t* s_full = v_empty + KSTAGES;        // [2]
  uint64_t* p_full = s_full + 2;               // [2]: one per S buffer, like s_full (see the softmax loop)
  uint64_t* o_done = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);

  pdl_wait();
  if ((smem_addr(smem) & 1023u) != 0) {      // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicExch(&g_attn_error, 9);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid (KV heads x slices, tiles): CTAs start in the order of the tile list, which the caller sorts by
  // falling length, whatever their KV head - the longest chains start first
  const int tile = blockIdx.y;
  const int kvh = blockIdx.x / p.slices, slice = blockIdx.x % p.slices;
  const int entry = p.tile_entry[tile], tok0 = p.tile_start[tile], ntok = p.tile_count[tile];
  const int* table = p.block_table + static_cast<size_t>(entry) * p.table_stride;
  const int p_first = p.positions[tok0], p_last = p_first + ntok - 1;   // an entry's positions are consecutive
  const int ntiles = p_last / BN + 1;
  const int head0 = kvh * p.group + slice * p.gs;
  const int tokens_per_cta = BM / p.gs;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KSTAGES; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
      mbar_init(v_full + s, 1);
      mbar_init(v_empty + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_full + s, 1);
      mbar_init(p_full + s, BM);
    }
    mbar_init(o_done, 1);
    fence_barrier_init();
  }
  if (warp == 5) tmem_alloc(tmem_slot, TMEM_COLS);
  // Rows of the V stages that no page is ever copied into must hold finite numbers: a masked
  // key has probability 0, and 0 * NaN would still be NaN.
  for (uint32_t i = threadIdx.x; i < KSTAGES * KV_BYTES / 16; i += kTcThreads)
    reinterpret_cast<uint4*>(v_smem)[i] = make_uint4(0, 0, 0, 0);
  fence_async_shared();
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer (one warp)
    if (lane == 0) {
      mbar_expect_tx(q_full, DSUB * 128u * p.gs * tokens_per_cta);
      for (int sub = 0; sub < DSUB; ++sub) tma_load_3d(q_smem + sub * Q_SUB, &map_q, q_full, sub * 64, head0, tok0);
    }
    // A key tile is pages_per_tile pages of K and as many of V, DSUB boxes (64 columns) each.  Lane
    // i of the warp owns box i of a tensor: page i / DSUB, half i % DSUB.  All lanes issue their
    // copies at once, so a tile of small pages costs the time of one copy instruction, not sixteen.
    const int pages_per_tile = BN / p.page_size;
    const int boxes = pages_per_tile * DSUB;
    const int my_page = lane / DSUB, my_sub = lane % DSUB;
    const bool has_box = lane < boxes;
    // the page id of tile j for this lane, fetched one tile ahead of its use
    auto fetch_id = [&](int j) -> int {
      const int t0 = j * BN + my_page * p.page_size;
      return (has_box && t0 <= p_last) ? table[t0 >> p.page_shift] : -1;
    };
    auto load_boxes = [&](unsigned char* dst, const CUtensorMap* map, uint64_t* bar, int id) {
      const unsigned valid = __ballot_sync(0xffffffffu, id >= 0);
      if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(__popc(valid)) * p.page_size * 128u);
      __syncwarp();
      if (id >= 0)
        tma_load_2d(dst + my_sub * KV_SUB + my_page * p.page_size * 128, map, bar, my_sub * 64, (id * p.nkv + kvh) * p.page_size);
    };
    // K and V of tile j go to stage j % KSTAGES; a stage is free again when the product that read it
    // has completed (S(j-2) for K, P.V(j-2) for V): the first two tiles find their stages free.
    int id = fetch_id(0);
    for (int j = 0; j < ntiles; ++j) {
      const int s = j % KSTAGES;
      const uint32_t parity = ((j / KSTAGES) & 1) ^ 1;
      const int next_id = j + 1 < ntiles ? fetch_id(j + 1) : -1;
      bool free_k = mbar_wait(k_empty + s, parity);
      if (!__all_sync(0xffffffffu, free_k)) { if (lane == 0) atomicExch(&g_attn_error, 1); break; }
      load_boxes(k_smem + s * KV_BYTES, &map_k, k_full + s, id);
      bool free_v = mbar_wait(v_empty + s, parity);
      if (!__all_sync(0xffffffffu, free_v)) { if (lane == 0) atomicExch(&g_attn_error, 1); break; }
      load_boxes(v_smem + s * KV_BYTES, &map_v, v_full + s, id);
      id = next_id;
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ tensor-core issue
    // The whole warp runs the loop and waits; one elected lane issues (see elect_one()).
    constexpr uint32_t idesc_s = umma_idesc_bf16(BM, BN, 0);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(BM, D, 1);
    auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity) ? 1 : 0) != 0; };
    bool ok = wait_all(q_full, 0);
    if (!ok) atomicExch(&g_attn_error, 2);
    const uint32_t q_addr = smem_addr(q_smem);
    auto issue_s = [&](int j) -> bool {        // S(j) = Q K_j^T into S buffer j & 1
      const int s = j % KSTAGES, buf = j & 1;
      if (!wait_all(k_full + s, (j / KSTAGES) & 1)) return false;
      tcgen05_fence_after();
      const uint32_t k_addr = smem_addr(k_smem + s * KV_BYTES);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16_ss(tmem_base + S_COL + buf * BN, umma_desc_sw128(q_addr + (k >> 2) * Q_SUB + (k & 3) * 32, 16, 1024),
                       umma_desc_sw128(k_addr + (k >> 2) * KV_SUB + (k & 3) * 32, 16, 1024), idesc_s, k != 0);
        umma_commit_to(s_full + buf);
        umma_commit_to(k_empty + s);
      }
      __syncwarp();
      return true;
    };
    if (ok && !issue_s(0)) { atomicExch(&g_attn_error, 2); ok = false; }
    for (int j = 0; j < ntiles && ok; ++j) {
      const int s = j % KSTAGES, buf = j & 1;
      // S of the next tile first, so that the tensor core has work while the softmax of tile j runs.  Its
      // buffer holds P(j - 1): the product P(j - 1) V must have completed (not just been issued before:
      // products into different accumulators are not ordered among themselves by their order of issue).
      if (j >= 1 && j + 1 < ntiles && !wait_all(o_done, (j - 1) & 1)) { atomicExch(&g_attn_error, 6); break; }
      if (j + 1 < ntiles && !issue_s(j + 1)) { atomicExch(&g_attn_error, 2); break; }
      if (!wait_all(p_full + buf, (j >> 1) & 1) || !wait_all(v_full + s, (j / KSTAGES) & 1)) { atomicExch(&g_attn_error, 3); break; }
      tcgen05_fence_after();
      const uint32_t v_addr = smem_addr(v_smem + s * KV_BYTES);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)       // P of this tile lies where its S was: 8 columns per 16 keys
          umma_bf16_ts(tmem_base + O_COL, tmem_base + S_COL + buf * BN + k * 8,
                       umma_desc_sw128(v_addr + k * 2048, KV_SUB, 1024), idesc_pv, (j | k) != 0);
        umma_commit_to(o_done);
        umma_commit_to(v_empty + s);
      }
      __syncwarp();
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ softmax, one row per thread
    const int row = threadIdx.x;
    const int tl = row / p.gs, g = row - tl * p.gs;
    const bool row_ok = tl < ntok && slice * p.gs + g < p.group;
    const int row_hi = p_first + tl;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    float m_used = -INFINITY, l = 0.f;       // m_used in units of log2, after scaling
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      if (!mbar_wait(s_full + (j & 1), (j >> 1) & 1)) { atomicExch(&g_attn_error, 4); ok = false; break; }
      tcgen05_fence_after();
      float sv[BN];
      {
        uint32_t r0[32], r1[32];            // both halves in flight, one wait
        tmem_ld_32_nowait(lane_base + S_COL + (j & 1) * BN, r0);
        tmem_ld_32_nowait(lane_base + S_COL + (j & 1) * BN + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          sv[i] = __uint_as_float(r0[i]);
          sv[32 + i] = __uint_as_float(r1[i]);
        }
      }
      const int t0 = j * BN;
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (t0 + BN - 1 <= p_first) {          // every key of the tile is visible to every row of this CTA
#pragma unroll
        for (int i = 0; i < BN; ++i) mx[i & 3] = fmaxf(mx[i & 3], sv[i]);
      } else {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          sv[i] = t0 + i <= row_hi ? sv[i] : -INFINITY;
          mx[i & 3] = fmaxf(mx[i & 3], sv[i]);
        }
      }
      const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      const float m_new = fmaxf(m_used, m_tile * p.scale_log2);   // the scale is positive
      const bool grow = m_new > m_used + kRescaleStep;            // also true on the first tile (m_used = -inf)
      if (j == 0) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        // O must hold every product issued so far and no later one: P.V(j-1) has been issued
        // (it follows S(j), which is complete) and P.V(j) waits for this thread's arrival.
        if (!mbar_wait(o_done, (j - 1) & 1)) { atomicExch(&g_attn_error, 5); ok = false; break; }
        tcgen05_fence_after();
        const float factor = grow ? exp2f(m_used - m_new) : 1.f;
        if (grow) m_used = m_new;
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld_32(lane_base + O_COL + c * 32, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
          tmem_st_32(lane_base + O_COL + c * 32, r);
        }
        l *= factor;
      }
      const float neg_ref = m_used == -INFINITY ? 0.f : -m_used;
      uint4 packed[BN / 8];
      float lsum[4] = {0.f, 0.f, 0.f, 0.f};      // four chains instead of one long dependent sum
#pragma unroll
      for (int c = 0; c < BN / 8; ++c) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = exp2_fast(fmaf(sv[c * 8 + i], p.scale_log2, neg_ref));
          lsum[i & 3] += e[i];
        }
        packed[c].x = pack_bf16(e[0], e[1]);
        packed[c].y = pack_bf16(e[2], e[3]);
        packed[c].z = pack_bf16(e[4], e[5]);
        packed[c].w = pack_bf16(e[6], e[7]);
      }
      l += (lsum[0] + lsum[1]) + (lsum[2] + lsum[3]);
      // P goes where this thread's row of S was (it has been read into registers above): 32 columns of
      // two bfloat16 each.  The product that read the P before the last one there has completed, since
      // the S that followed it into this buffer has.
      {
        uint32_t words[32];
#pragma unroll
        for (int c = 0; c < BN / 8; ++c) {
          words[4 * c] = packed[c].x;
          words[4 * c + 1] = packed[c].y;
          words[4 * c + 2] = packed[c].z;
          words[4 * c + 3] = packed[c].w;
        }
        tmem_st_32(lane_base + S_COL + (j & 1) * BN, words);
      }
      // One barrier per S buffer: S(j+1) is ready before this tile's P is handed over, so a warp that is done
      // with tile j may be through tile j + 1 and arrive for it while another warp still works on tile j;
      // on a single barrier that arrival would be counted for tile j and let P(j) V start on a P that is not
      // all written.  No warp gets two tiles ahead: S(j+2) is issued behind P(j) V.
      tcgen05_fence_before();
      mbar_arrive(p_full + (j & 1));
    }
    if (ok) {
      if (!mbar_wait(o_done, (ntiles - 1) & 1)) {
        atomicExch(&g_attn_error, 7);
      } else {
        tcgen05_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* dst = p.out + (static_cast<size_t>(tok0 + tl) * p.nq + head0 + g) * D;
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld_32(lane_base + O_COL + c * 32, r);   // warp-collective: every lane takes part
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 q;
              q.x = pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
              q.y = pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
              q.z = pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
              q.w = pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = q;
            }
          }
        }
      }
    }
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------
// The same attention with two row tiles per CTA, for portions long enough to fill both.
//
// One CTA owns 256 rows of S: two tiles of 128 (consecutive tokens of one request times the query heads
// of one KV head) that share one stream of K and V.  Keys are taken 128 at a time (a product over 64 keys
// is too short for the time it takes to issue); the whole of tensor memory belongs to the CTA (S of both
// row tiles, 128 columns each, and O of both), one CTA per SM.
//   warps 0-3 / 4-7  softmax of row tile 0 / 1, one row per thread
//   warp 8           TMA loads: both Q tiles once, then K and V tile by tile through the block table
//   warp 9           tensor-core issue, in the order  P_0(j) V, S_0(j+1), P_1(j) V, S_1(j+1):  while the
//                    threads of one row tile turn S into P, the tensor core works for the other, and both
//                    read every K and V stage (half the shared-memory and L2 traffic of the one-tile kernel)
//   warps 10, 11     nothing: warps 8-11 are a warpgroup that gives most of its registers to the softmax
//                    warps (setmaxnreg), which hold a row of 128 scores each.
// S_t(j+1) overwrites the columns that hold P_t(j): it is issued when P_t(j) V has completed.
//
// What shortens the chain S -> P -> P V -> next S, which is what a row tile's time is made of:
//  * the exponentials of a tile start from the reference maximum of the tiles before it, without a pass for
//    the tile's own maximum: a weight 2^(s - reference) may be any size that float32 holds (the final
//    division uses the same reference), so only when a row's weights of one tile add up to more than
//    kSpeculationLimit is the maximum found, O rescaled and the tile redone;
//  * P is handed over in two halves of 64 keys, so the product of the first half runs while the second
//    half is exponentiated;
//  * one lane of each warp arrives on the barrier, not 128 threads one after the other.
constexpr int PBN = 128;                             // keys per tile
constexpr uint32_t PKV_SUB = PBN * 128;              // bytes of one 64-column sub-tile of a K or V stage
constexpr uint32_t PKV_BYTES = DSUB * PKV_SUB;
constexpr int KSTAGES_P = 3, VSTAGES_P = D == 128 ? 2 : 3;   // more than half of an SM's shared memory either way: one CTA per SM
constexpr uint32_t PAIR_SMEM_TILES = 2 * Q_BYTES + (KSTAGES_P + VSTAGES_P) * PKV_BYTES;
constexpr uint32_t PAIR_BARRIER_BYTES = 512;
constexpr uint32_t PAIR_TMEM_COLS = 512;
constexpr uint32_t PAIR_O_COL = 2 * PBN;
constexpr int kPairThreads = 384;                    // three warpgroups: every quarter of the SM holds two softmax warps and one other
constexpr int kPairSoftmaxRegs = 216, kPairOtherRegs = 72;   // 2 * 216 + 72 = 3 * 168, what the launch gives each quarter
constexpr float kSpeculationLimit = 1099511627776.f;  // 2^40
static_assert(PAIR_SMEM_TILES > 116 * 1024, "two of these CTAs on one SM would wait for each other's tensor memory");
static_assert((1 + 2 * (KSTAGES_P + VSTAGES_P) + 2 + 4 + 2 + 2) * 8 + 4 <= PAIR_BARRIER_BYTES, "barriers");

__global__ void __launch_bounds__(kPairThreads, 1)
prefill_attention_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* q_smem = smem;                               // [2]
  unsigned char* k_smem = q_smem + 2 * Q_BYTES;               // [KSTAGES_P]
  unsigned char* v_smem = k_smem + KSTAGES_P * PKV_BYTES;     // [VSTAGES_P]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PAIR_SMEM_TILES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                  // [KSTAGES_P]
  uint64_t* k_empty = k_full + KSTAGES_P;
  uint64_t* v_full = k_empty + KSTAGES_P;       // [VSTAGES_P]
  uint64_t* v_empty = v_full + VSTAGES_P;
  uint64_t* s_full = v_empty + VSTAGES_P;       // [2]: per row tile
  uint64_t* p_full = s_full + 2;                // [2 row tiles][2 halves]
  uint64_t* o_done = p_full + 4;                // [2]: all of P_t(j) V is in O
  uint64_t* o_half = o_done + 2;                // [2]: the first half of P_t(j) V is in O
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_half + 2);

  pdl_wait();
  if ((smem_addr(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(&g_attn_error, 9);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.y;
  const int kvh = blockIdx.x / p.slices, slice = blockIdx.x % p.slices;
  const int entry = p.tile_entry[tile], tok0 = p.tile_start[tile], ntok = p.tile_count[tile];
  const int* table = p.block_table + static_cast<size_t>(entry) * p.table_stride;
  const int tpc = BM / p.gs;                                  // tokens of one row tile
  const int p_first = p.positions[tok0], p_last = p_first + ntok - 1;
  const int ntok1 = ntok > tpc ? ntok - tpc : 0;              // tokens of the second row tile
  const int nt0 = (p_first + min(ntok, tpc) - 1) / PBN + 1;   // key tiles that row tile 0 can see
  const int nt1 = ntok1 > 0 ? p_last / PBN + 1 : 0;           // nt1 >= nt0 unless tile 1 is empty
  const int ntiles = max(nt0, nt1);
  const int head0 = kvh * p.group + slice * p.gs;
  if (ntok > 2 * tpc) {                                       // the caller cut its tiles for another kernel
    if (threadIdx.x == 0) atomicExch(&g_attn_error, 18);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KSTAGES_P; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
    }
    for (int s = 0; s < VSTAGES_P; ++s) {
      mbar_init(v_full + s, 1);
      mbar_init(v_empty + s, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full + t, 1);
      mbar_init(p_full + 2 * t, 4);             // one arrival per softmax warp
      mbar_init(p_full + 2 * t + 1, 4);
      mbar_init(o_done + t, 1);
      mbar_init(o_half + t, 1);
    }
    fence_barrier_init();
  }
  if (warp == 9) tmem_alloc(tmem_slot, PAIR_TMEM_COLS);
  for (uint32_t i = threadIdx.x; i < VSTAGES_P * PKV_BYTES / 16; i += kPairThreads)   // see the one-tile kernel
    reinterpret_cast<uint4*>(v_smem)[i] = make_uint4(0, 0, 0, 0);
  // rows of the Q tiles past the last (token, head) pair (a group size that does not divide 128) are copied by nobody
  for (uint32_t i = threadIdx.x; i < 2 * DSUB * (BM - tpc * p.gs) * 8; i += kPairThreads) {
    const uint32_t sub = i / ((BM - tpc * p.gs) * 8), rest = i % ((BM - tpc * p.gs) * 8);
    reinterpret_cast<uint4*>(q_smem + sub * Q_SUB + (tpc * p.gs + rest / 8) * 128)[rest % 8] = make_uint4(0, 0, 0, 0);
  }
  fence_async_shared();
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // All four warps of a warpgroup execute the same setmaxnreg instruction, as it demands.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kPairOtherRegs));
    if (warp == 8) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        const uint32_t tile_bytes = DSUB * 128u * p.gs * tpc;
        mbar_expect_tx(q_full, ntok1 > 0 ? 2 * tile_bytes : tile_bytes);
        for (int t = 0; t < (ntok1 > 0 ? 2 : 1); ++t)
          for (int sub = 0; sub < DSUB; ++sub)
            tma_load_3d(q_smem + t * Q_BYTES + sub * Q_SUB, &map_q, q_full, sub * 64, head0, tok0 + t * tpc);
      }
      const int pages_per_tile = PBN / p.page_size;
      const int boxes = pages_per_tile * DSUB;             // at most 32: pages of 8 tokens, head size 128
      const int my_page = lane / DSUB, my_sub = lane % DSUB;
      const bool has_box = lane < boxes;
      auto fetch_id = [&](int j) -> int {
        const int t0 = j * PBN + my_page * p.page_size;
        return (has_box && t0 <= p_last) ? table[t0 >> p.page_shift] : -1;
      };
      auto load_boxes = [&](unsigned char* dst, const CUtensorMap* map, uint64_t* bar, int id) {
        const unsigned valid = __ballot_sync(0xffffffffu, id >= 0);
        if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(__popc(valid)) * p.page_size * 128u);
        __syncwarp();
        if (id >= 0)
          tma_load_2d(dst + my_sub * PKV_SUB + my_page * p.page_size * 128, map, bar, my_sub * 64, (id * p.nkv + kvh) * p.page_size);
      };
      // K of tile j + 1 is asked for before V of tile j: S_t(j+1) is issued ahead of P_t(j+1) V, and the K ring
      // is the deeper one.
      int id_k = fetch_id(0), id_v = -1;
      for (int j = 0; j <= ntiles; ++j) {
        int next_id = -1;
        if (j < ntiles) {
          const int s = j % KSTAGES_P;
          if (j + 1 < ntiles) next_id = fetch_id(j + 1);
          bool free_k = mbar_wait(k_empty + s, ((j / KSTAGES_P) & 1) ^ 1);
          if (!__all_sync(0xffffffffu, free_k)) { if (lane == 0) atomicExch(&g_attn_error, 11); break; }
          load_boxes(k_smem + s * PKV_BYTES, &map_k, k_full + s, id_k);
        }
        if (j > 0) {
          const int jv = j - 1, s = jv % VSTAGES_P;
          bool free_v = mbar_wait(v_empty + s, ((jv / VSTAGES_P) & 1) ^ 1);
          if (!__all_sync(0xffffffffu, free_v)) { if (lane == 0) atomicExch(&g_attn_error, 11); break; }
          load_boxes(v_smem + s * PKV_BYTES, &map_v, v_full + s, id_v);
        }
        id_v = id_k;
        id_k = next_id;
      }
    } else if (warp == 9) {
      // ---------------------------------------------------------------- tensor-core issue
      constexpr uint32_t idesc_s = umma_idesc_bf16(BM, PBN, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(BM, D, 1);
      auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, mbar_wait(bar, parity) ? 1 : 0) != 0; };
      const int nt[2] = {nt0, nt1};
      bool ok = wait_all(q_full, 0);
      if (!ok) atomicExch(&g_attn_error, 12);
      const uint32_t q_addr = smem_addr(q_smem);
      // S_t(j) = Q_t K_j^T; the caller has waited for K_j.  `last`: no other row tile reads K_j after this one.
      auto issue_s = [&](int t, int j, bool last) {
        const int s = j % KSTAGES_P;
        const uint32_t k_addr = smem_addr(k_smem + s * PKV_BYTES);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_bf16_ss(tmem_base + t * PBN, umma_desc_sw128(q_addr + t * Q_BYTES + (k >> 2) * Q_SUB + (k & 3) * 32, 16, 1024),
                         umma_desc_sw128(k_addr + (k >> 2) * PKV_SUB + (k & 3) * 32, 16, 1024), idesc_s, k != 0);
          umma_commit_to(s_full + t);
          if (last) umma_commit_to(k_empty + s);
        }
        __syncwarp();
      };
      if (ok) {
        ok = wait_all(k_full, 0);
        if (!ok) atomicExch(&g_attn_error, 12);
      }
      if (ok) {
        tcgen05_fence_after();
        issue_s(0, 0, nt1 == 0);
        if (nt1 > 0) issue_s(1, 0, true);
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j % VSTAGES_P;
        bool have_v = false, have_k = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= nt[t]) continue;
          const uint32_t v_addr = smem_addr(v_smem + s * PKV_BYTES);
          const bool last_pv = t == 1 || j >= nt[1];
          for (int half = 0; half < 2 && ok; ++half) {    // P_t(j) arrives in two halves of 64 keys
            if (!wait_all(p_full + 2 * t + half, j & 1)) { atomicExch(&g_attn_error, 13); ok = false; break; }
            if (!have_v) {
              if (!wait_all(v_full + s, (j / VSTAGES_P) & 1)) { atomicExch(&g_attn_error, 13); ok = false; break; }
              have_v = true;
            }
            tcgen05_fence_after();
            if (elect_one()) {
#pragma unroll
              for (int k = 4 * half; k < 4 * half + 4; ++k)     // P_t lies where S_t was: 8 columns per 16 keys
                umma_bf16_ts(tmem_base + PAIR_O_COL + t * D, tmem_base + t * PBN + k * 8,
                             umma_desc_sw128(v_addr + k * 2048, PKV_SUB, 1024), idesc_pv, (j | k) != 0);
              if (half == 0) {
                umma_commit_to(o_half + t);
              } else {
                umma_commit_to(o_done + t);
                if (last_pv) umma_commit_to(v_empty + s);
              }
            }
            __syncwarp();
          }
          if (ok && j + 1 < nt[t]) {
            // S_t(j+1) goes where P_t(j) lies: P_t(j) V must have completed, not just been issued before
            // (products into different accumulators are not ordered among themselves by their order of issue)
            if (!wait_all(o_done + t, j & 1)) { atomicExch(&g_attn_error, 19); ok = false; break; }
            if (!have_k) {
              if (!wait_all(k_full + (j + 1) % KSTAGES_P, ((j + 1) / KSTAGES_P) & 1)) { atomicExch(&g_attn_error, 12); ok = false; break; }
              have_k = true;
              tcgen05_fence_after();
            }
            issue_s(t, j + 1, t == 1 || j + 1 >= nt[1]);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: warps 0-3 row tile 0, warps 4-7 row tile 1
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(kPairSoftmaxRegs));
    const int t = warp >> 2;
    const int my_tiles = t == 0 ? nt0 : nt1;
    const int row = threadIdx.x & (BM - 1);
    const int tl = row / p.gs, g = row - tl * p.gs;
    const int ntok_t = t == 0 ? min(ntok, tpc) : ntok1;
    const bool row_ok = tl < ntok_t && slice * p.gs + g < p.group;
    const int first_pos = p_first + t * tpc;             // position of the tile's first row
    const int row_hi = first_pos + tl;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t s_col = lane_base + t * PBN, o_col = lane_base + PAIR_O_COL + t * D;
    float m_used = -INFINITY, l = 0.f;       // m_used: the reference maximum, in units of log2 after scaling
    bool ok = true;
    for (int j = 0; j < my_tiles; ++j) {
      if (!mbar_wait(s_full + t, j & 1)) { atomicExch(&g_attn_error, 14); ok = false; break; }
      tcgen05_fence_after();
      float sv[PBN];
      {
        uint32_t r[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32_nowait(s_col + c * 32, r[c]);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) sv[c * 32 + i] = __uint_as_float(r[c][i]);
      }
      const int t0 = j * PBN;
      if (t0 + PBN - 1 > first_pos) {        // some key of the tile is hidden from some row
#pragma unroll
        for (int i = 0; i < PBN; ++i) sv[i] = t0 + i <= row_hi ? sv[i] : -INFINITY;
      }
      // weights of one half (64 keys) from the current reference, handed to the tensor core; returns their sum
      auto half_weights = [&](int half) -> float {
        const float neg_ref = -m_used;
        float lsum[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t words[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float e0 = exp2_fast(fmaf(sv[half * 64 + 2 * c], p.scale_log2, neg_ref));
          const float e1 = exp2_fast(fmaf(sv[half * 64 + 2 * c + 1], p.scale_log2, neg_ref));
          lsum[(2 * c) & 3] += e0;
          lsum[(2 * c + 1) & 3] += e1;
          words[c] = pack_bf16(e0, e1);
        }
        tmem_st_32(s_col + half * 32, words);
        return (lsum[0] + lsum[1]) + (lsum[2] + lsum[3]);
      };
      auto hand_over = [&](int half) {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + 2 * t + half);
      };
      // Every row sees key 0, so from the second tile on the reference is finite.  Speculate on it:
      float first_half = 0.f;
      bool redo = j == 0;
      if (j > 0) {
        first_half = half_weights(0);
        redo = !(first_half < kSpeculationLimit);
      }
      // rescale what O and l hold by 2^(old reference - new reference); every lane takes part
      auto move_reference = [&](float m_new) {
        const float factor = exp2f(m_used - m_new);
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld_32(o_col + c * 32, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
          tmem_st_32(o_col + c * 32, r);
        }
        l *= factor;
        first_half *= factor;
        m_used = m_new;
      };
      if (!__any_sync(0xffffffffu, redo)) {
        hand_over(0);
        float second_half = half_weights(1);
        const bool grow = !(second_half < kSpeculationLimit);
        if (__any_sync(0xffffffffu, grow)) {
          // The first half is with the tensor core already.  Once its product is in O, move the reference
          // to the maximum of the second half and redo that half.
          if (!mbar_wait(o_half + t, j & 1)) { atomicExch(&g_attn_error, 16); ok = false; break; }
          tcgen05_fence_after();
          float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int i = PBN / 2; i < PBN; ++i) mx[i & 3] = fmaxf(mx[i & 3], sv[i]);
          const float m_half = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
          move_reference(grow ? fmaxf(m_used, m_half) : m_used);
          second_half = half_weights(1);
        }
        hand_over(1);
        l += first_half + second_half;
        continue;
      }
      // The tile's own maximum: on the first tile, and when a row's weights outgrew the reference.
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < PBN; ++i) mx[i & 3] = fmaxf(mx[i & 3], sv[i]);
      const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      // Only a row that needs it moves its reference: what a row comes to must not depend on the rows that share
      // its warp (on whose account it may be here), least of all on rows that belong to no token.
      const float m_new = (j == 0 || redo) ? fmaxf(m_used, m_tile * p.scale_log2) : m_used;
      if (j > 0) {
        // O must hold every product issued so far and no later one: P_t(j-1) V has been issued and
        // P_t(j) V waits for this warp's arrival.
        if (!mbar_wait(o_done + t, (j - 1) & 1)) { atomicExch(&g_attn_error, 15); ok = false; break; }
        tcgen05_fence_after();
        move_reference(m_new);
      }
      m_used = m_new;
      const float a = half_weights(0);
      hand_over(0);
      const float b = half_weights(1);
      hand_over(1);
      l += a + b;
    }
    if (ok && my_tiles > 0) {
      if (!mbar_wait(o_done + t, (my_tiles - 1) & 1)) {
        atomicExch(&g_attn_error, 17);
      } else {
        tcgen05_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* dst = p.out + (static_cast<size_t>(tok0 + t * tpc + tl) * p.nq + head0 + g) * D;
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld_32(o_col + c * 32, r);
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 q;
              q.x = pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
              q.y = pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
              q.z = pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
              q.w = pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = q;
            }
          }
        }
      }
    }
  }
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tmem_dealloc(tmem_base, PAIR_TMEM_COLS);
  }
}

// rows x cols bf16 matrix with `row_bytes` between rows; box = [box_rows, 64 columns], 128-byte swizzle
static int make_map_2d(CUtensorMap* map, const void* base, uint64_t rows, int cols, int box_rows) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (!fn) return 10005;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), rows};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : 10006;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_attention_tcgen05_error() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int));
  cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
  return v;
}

// Tokens per CTA for a group of `group` query heads per KV head: the caller cuts entries into
// tiles of that many consecutive tokens.
extern "C" int b200_attention_tcgen05_tokens_per_tile(int group) {
  const int gs = group < 16 ? group : 16;
  return BM / gs;
}

// Tokens per CTA of the two-tile kernel.
extern "C" int b200_attention_tcgen05_tokens_per_pair(int group) { return 2 * b200_attention_tcgen05_tokens_per_tile(group); }

// q, out: [tokens, nq, D]; pools: [pages, nkv, page_size, D].  page_size must be 8, 16, 32 or 64.
// `pair` != 0: the two-tile kernel; the tiles of the list then hold up to twice as many tokens.
static int prefill_tcgen05(const void* q, const void* k_pool, const void* v_pool, void* out, const int* positions,
                           const int* block_table, int table_stride, int page_size, int num_pages, int tokens, int nq,
                           int nkv, float scale, const int* tile_entry, const int* tile_start, const int* tile_count,
                           int num_tiles, bool pair, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || table_stride <= 0 || tokens <= 0) return B200_ERR_BAD_SIZE;
  if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return B200_ERR_BAD_SIZE;
  TcAttnParams p{};
  p.out = static_cast<bf16*>(out);
  p.positions = positions;
  p.block_table = block_table;
  p.table_stride = table_stride;
  p.page_size = page_size;
  p.page_shift = page_size == 8 ? 3 : (page_size == 16 ? 4 : (page_size == 32 ? 5 : 6));
  p.nq = nq;
  p.nkv = nkv;
  p.group = nq / nkv;
  p.gs = p.group < 16 ? p.group : 16;
  p.slices = (p.group + p.gs - 1) / p.gs;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.tile_entry = tile_entry;
  p.tile_start = tile_start;
  p.tile_count = tile_count;

  CUtensorMap map_q, map_k, map_v;
  {
    EncodeTiledFn fn = tensor_map_encoder();
    if (!fn) return 10005;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(nq), static_cast<cuuint64_t>(tokens)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(nq) * D * 2};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(p.gs), static_cast<cuuint32_t>(BM / p.gs)};
    const cuuint32_t elem[3] = {1, 1, 1};
    if (fn(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return 10006;
  }
  const uint64_t pool_rows = static_cast<uint64_t>(num_pages) * nkv * page_size;
  if (int e = make_map_2d(&map_k, k_pool, pool_rows, D, page_size)) return e;
  if (int e = make_map_2d(&map_v, v_pool, pool_rows, D, page_size)) return e;

  dim3 grid(nkv * p.slices, num_tiles);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  if (pair) {
    constexpr size_t smem = PAIR_SMEM_TILES + PAIR_BARRIER_BYTES;
    static DeviceOnce once;
    if (int e = configure_once(once, prefill_attention_pair_kernel, smem)) return e;
    launch(prefill_attention_pair_kernel, grid, dim3(kPairThreads), smem, stream, map_q, map_k, map_v, p);
  } else {
    constexpr size_t smem = SMEM_TILES + kBarrierBytes;
    static DeviceOnce once;
    if (int e = configure_once(once, prefill_attention_tcgen05_kernel, smem)) return e;
    launch(prefill_attention_tcgen05_kernel, grid, dim3(kTcThreads), smem, stream, map_q, map_k, map_v, p);
  }
  return launch_status();
}

extern "C" int b200_attention_prefill_tcgen05(const void* q, const void* k_pool, const void* v_pool, void* out,
                                              const int* positions, const int* block_table, int table_stride,
                                              int page_size, int num_pages, int tokens, int nq, int nkv, float scale,
                                              const int* tile_entry, const int* tile_start, const int* tile_count,
                                              int num_tiles, cudaStream_t stream) {
  return prefill_tcgen05(q, k_pool, v_pool, out, positions, block_table, table_stride, page_size, num_pages, tokens, nq, nkv,
                         scale, tile_entry, tile_start, tile_count, num_tiles, false, stream);
}

extern "C" int b200_attention_prefill_tcgen05_pair(const void* q, const void* k_pool, const void* v_pool, void* out,
                                                   const int* positions, const int* block_table, int table_stride,
                                                   int page_size, int num_pages, int tokens, int nq, int nkv, float scale,
                                                   const int* tile_entry, const int* tile_start, const int* tile_count,
                                                   int num_tiles, cudaStream_t stream) {
  return prefill_tcgen05(q, k_pool, v_pool, out, positions, block_table, table_stride, page_size, num_pages, tokens, nq, nkv,
                         scale, tile_entry, tile_start, tile_count, num_tiles, true, stream);
}
