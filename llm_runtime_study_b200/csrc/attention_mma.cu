// bfloat16 tensor-core attention over the paged cache, built once per head size
// (-DHEAD_DIM=<multiple of 16, at most 256>).
//
//   prefill kernel  a tile of up to TM consecutive query tokens of one request times the
//                   query heads that share one KV head forms the rows of S = Q K^T; keys
//                   are streamed in tiles of 64 through shared memory (cp.async, double
//                   buffered) from the request's pages; online softmax in float32.
//                   Serves prompt portions cut anywhere and single tokens alike.
//   decode kernel   one query token per request: the sequence is split over CTAs (and
//                   inside a CTA over its four warps); partial (max, sum, output) triples
//                   go to scratch memory and a merge kernel combines them.
//
// Formula (mini_llm/nn/attention.py:95-99, 231-248): S = q.k^T * scale, key t visible iff
// t <= p (and t > p - window with a window), P = softmax(S), o = P.v; query head j reads KV
// head j / (nq / nkv).  Scores, maxima, exponentials, sums and the output accumulate in
// float32; P is rounded to bfloat16 for the P.V product, as the operands of Q.K^T are.
#include "common.cuh"
#include "mma.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size must be 16..256 in steps of 16");

namespace b200 {

using bf16 = __nv_bfloat16;
constexpr int D = HEAD_DIM;
constexpr int BN = 64;            // keys per shared-memory tile
constexpr int LDS = D + 8;        // padded row length: ldmatrix rows fall into different banks
constexpr int KSTEPS = D / 16;    // 16-wide steps over the head size in Q K^T
constexpr int DTILES = D / 8;     // 8-wide column tiles of the output
constexpr int kSmemBytes = 2 * 2 * BN * LDS * 2;

struct AttnParams {
  const bf16* q;
  const bf16* k_pool;
  const bf16* v_pool;
  bf16* out;
  const int* positions;
  const int* block_table;
  int table_stride, page_size;
  int page_shift;                  // log2(page_size) when it is a power of two, else -1
  int nq, nkv, group, gs, slices;  // group = nq / nkv; gs = heads of a group per CTA; slices = ceil(group / gs)
  float scale_log2;
  int window;
  // prefill
  const int* tile_entry;
  const int* tile_start;
  const int* tile_count;
  // decode
  const int* kv_len;
  int num_splits;
  float* part_o;   // [B][nq][splits][D]
  float* part_ml;  // [B][nq][splits][2]
};

// Copy keys t0 .. t0+BN-1 of one KV head into shared memory; rows outside [lo, hi] or on a
// page that has been given back are zero-filled (a masked key must never contribute NaN).
template <int NT>
__device__ __forceinline__ void load_kv_tile(bf16* ks, bf16* vs, const AttnParams& p, const int* table,
                                             int kvh, int t0, int lo, int hi) {
  constexpr int CH = D / 8;
  for (int c = threadIdx.x; c < BN * CH; c += NT) {
    const int r = c / CH, ch = c - r * CH;
    const int t = t0 + r;
    const bf16* ksrc = p.k_pool;
    const bf16* vsrc = p.v_pool;
    int bytes = 0;
    if (t >= lo && t <= hi) {
      const int index = p.page_shift >= 0 ? t >> p.page_shift : t / p.page_size;
      const int slot = p.page_shift >= 0 ? t & (p.page_size - 1) : t - index * p.page_size;
      const int page = table[index];
      if (page >= 0) {
        const size_t off = ((static_cast<size_t>(page) * p.nkv + kvh) * p.page_size + slot) * D + ch * 8;
        ksrc += off;
        vsrc += off;
        bytes = 16;
      }
    }
    cp_async_16(ks + r * LDS + ch * 8, ksrc, bytes);
    cp_async_16(vs + r * LDS + ch * 8, vsrc, bytes);
  }
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// One warp: NT8 tiles of 8 keys (rows key0.. of the shared tile) against its 16 query rows.
// Updates the running maximum m, the per-thread partial sum l and the output o.
template <int NT8>
__device__ __forceinline__ void warp_attend(const bf16* kbuf, const bf16* vbuf, int key0, int t_first,
                                            const uint32_t (&qf)[KSTEPS][4], const bool (&row_ok)[2],
                                            const int (&row_hi)[2], const int (&row_lo)[2],
                                            float scale_log2, float (&m)[2], float (&l)[2],
                                            float (&o)[DTILES][4]) {
  const int lane = threadIdx.x & 31, tig = lane & 3;
  float s[NT8][4];
#pragma unroll
  for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
    for (int ntp = 0; ntp < NT8 / 2; ++ntp) {
      uint32_t kf[4];
      ldmatrix_x4(kf, kbuf + (key0 + ntp * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LDS + ks * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[2 * ntp], qf[ks], kf[0], kf[1]);
      mma_bf16(s[2 * ntp + 1], qf[ks], kf[2], kf[3]);
    }
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < NT8; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1;
      const int t = t_first + key0 + nt * 8 + tig * 2 + (e & 1);
      const bool visible = row_ok[i] && t <= row_hi[i] && t >= row_lo[i];
      s[nt][e] = visible ? s[nt][e] * scale_log2 : -INFINITY;
      mx[i] = fmaxf(mx[i], s[nt][e]);
    }
  }
  float m_use[2], corr[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float m_new = fmaxf(m[i], quad_max(mx[i]));
    m_use[i] = m_new == -INFINITY ? 0.f : m_new;
    corr[i] = exp2f(m[i] - m_use[i]);
    m[i] = m_new;
    l[i] *= corr[i];
  }
#pragma unroll
  for (int nt = 0; nt < NT8; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float pv = exp2f(s[nt][e] - m_use[e >> 1]);
      s[nt][e] = pv;
      l[e >> 1] += pv;
    }
  }
#pragma unroll
  for (int dt = 0; dt < DTILES; ++dt) {
    o[dt][0] *= corr[0];
    o[dt][1] *= corr[0];
    o[dt][2] *= corr[1];
    o[dt][3] *= corr[1];
  }
#pragma unroll
  for (int kk = 0; kk < NT8 / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dtp = 0; dtp < DTILES / 2; ++dtp) {
      uint32_t vf[4];
      ldmatrix_x4_trans(vf, vbuf + (key0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + dtp * 16 + ((lane >> 4) & 1) * 8);
      mma_bf16(o[2 * dtp], a, vf[0], vf[1]);
      mma_bf16(o[2 * dtp + 1], a, vf[2], vf[3]);
    }
  }
}

__device__ __forceinline__ void load_q_fragments(uint32_t (&qf)[KSTEPS][4], const bf16* q, const long (&row_off)[2],
                                                 const bool (&row_ok)[2]) {
  const int tig = threadIdx.x & 3;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 2; ++i)
        qf[ks][i + 2 * h] = row_ok[i] ? *reinterpret_cast<const uint32_t*>(q + row_off[i] + ks * 16 + h * 8 + tig * 2) : 0u;
}

// ------------------------------------------------------------------ prefill / mixed batches
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) prefill_attention_kernel(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* ks = reinterpret_cast<bf16*>(smem_raw);
  bf16* vs = ks + 2 * BN * LDS;
  pdl_trigger();
  pdl_wait();
  // grid (KV heads x slices, tiles): CTAs start in the order of the caller's tile list (longest first)
  const int tile = blockIdx.y;
  const int kvh = blockIdx.x / p.slices, slice = blockIdx.x % p.slices;
  const int entry = p.tile_entry[tile], tok0 = p.tile_start[tile], ntok = p.tile_count[tile];
  const int* table = p.block_table + static_cast<size_t>(entry) * p.table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int p_first = p.positions[tok0], p_last = p_first + ntok - 1;  // an entry's positions are consecutive

  bool row_ok[2];
  int row_hi[2], row_lo[2];
  long row_off[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int R = warp * 16 + gid + i * 8;
    const int tl = R / p.gs, g = slice * p.gs + R % p.gs;
    row_ok[i] = tl < ntok && g < p.group;
    row_hi[i] = p_first + tl;
    row_lo[i] = p.window > 0 ? max(0, row_hi[i] - p.window + 1) : 0;
    row_off[i] = (static_cast<long>(tok0 + tl) * p.nq + kvh * p.group + g) * D;
  }
  uint32_t qf[KSTEPS][4];
  load_q_fragments(qf, p.q, row_off, row_ok);

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DTILES][4];
#pragma unroll
  for (int dt = 0; dt < DTILES; ++dt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dt][e] = 0.f;

  const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
  const int t_begin = (lo / BN) * BN;
  const int ntiles = (p_last - t_begin) / BN + 1;
  load_kv_tile<WARPS * 32>(ks, vs, p, table, kvh, t_begin, lo, p_last);
  cp_async_commit();
  for (int j = 0; j < ntiles; ++j) {
    const int buf = j & 1;
    if (j + 1 < ntiles) {
      load_kv_tile<WARPS * 32>(ks + (buf ^ 1) * BN * LDS, vs + (buf ^ 1) * BN * LDS, p, table, kvh,
                               t_begin + (j + 1) * BN, lo, p_last);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    warp_attend<BN / 8>(ks + buf * BN * LDS, vs + buf * BN * LDS, 0, t_begin + j * BN, qf, row_ok, row_hi, row_lo,
                        p.scale_log2, m, l, o);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!row_ok[i]) continue;
    const float total = quad_sum(l[i]);
    const float inv = total > 0.f ? 1.f / total : 0.f;
    bf16* dst = p.out + row_off[i];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt)
      *reinterpret_cast<uint32_t*>(dst + dt * 8 + tig * 2) = pack_bf16(o[dt][2 * i] * inv, o[dt][2 * i + 1] * inv);
  }
}

// --------------------------------------------------------------------------- decode
// grid (splits, nkv * slices, requests); 4 warps, each takes 16 keys of every 64-key tile.
__global__ void __launch_bounds__(128) decode_attention_kernel(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* ks = reinterpret_cast<bf16*>(smem_raw);
  bf16* vs = ks + 2 * BN * LDS;
  pdl_trigger();
  pdl_wait();
  const int split = blockIdx.x, b = blockIdx.z;
  const int kvh = blockIdx.y / p.slices, slice = blockIdx.y % p.slices;
  const int* table = p.block_table + static_cast<size_t>(b) * p.table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int len = p.kv_len[b];
  const int lo = p.window > 0 ? max(0, len - p.window) : 0;
  int chunk = (len - lo + p.num_splits - 1) / p.num_splits;
  chunk = ((chunk + BN - 1) / BN) * BN;
  const int c0 = lo + split * chunk;
  const int c1 = min(c0 + chunk, len) - 1;  // last key of this CTA's part (c1 < c0: nothing to do)

  bool row_ok[2];
  int row_hi[2], row_lo[2];
  long row_off[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int R = gid + i * 8;
    const int g = slice * p.gs + R;
    row_ok[i] = R < p.gs && g < p.group;
    row_hi[i] = len - 1;
    row_lo[i] = lo;
    row_off[i] = (static_cast<long>(b) * p.nq + kvh * p.group + g) * D;
  }
  uint32_t qf[KSTEPS][4];
  load_q_fragments(qf, p.q, row_off, row_ok);
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DTILES][4];
#pragma unroll
  for (int dt = 0; dt < DTILES; ++dt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dt][e] = 0.f;

  // Each warp runs a pipeline of its own over 16-key blocks (block w, w + 4, ... of this
  // CTA's part), with a private pair of shared-memory buffers: no CTA-wide barrier inside
  // the loop, so the warps drift apart and cover each other's waits.
  constexpr int WB = 16;                                  // keys per warp block
  bf16* wk = ks + warp * (2 * WB * LDS);                  // [2][WB][LDS] keys
  bf16* wv = vs + warp * (2 * WB * LDS);                  // [2][WB][LDS] values
  const int nblocks = c1 >= c0 ? (c1 - c0) / WB + 1 : 0;  // 16-key blocks in this CTA's part
  const int hi_here[2] = {min(row_hi[0], c1), min(row_hi[1], c1)};
  auto load_block = [&](int block, int buf) {
    constexpr int CH = D / 8;
    const int t0 = c0 + block * WB;
#pragma unroll
    for (int c = lane; c < WB * CH; c += 32) {
      const int r = c / CH, ch = c - r * CH;
      const int t = t0 + r;
      const bf16* ksrc = p.k_pool;
      const bf16* vsrc = p.v_pool;
      int bytes = 0;
      if (t <= c1) {
        const int index = p.page_shift >= 0 ? t >> p.page_shift : t / p.page_size;
        const int slot = p.page_shift >= 0 ? t & (p.page_size - 1) : t - index * p.page_size;
        const int page = table[index];
        if (page >= 0) {
          const size_t off = ((static_cast<size_t>(page) * p.nkv + kvh) * p.page_size + slot) * D + ch * 8;
          ksrc += off;
          vsrc += off;
          bytes = 16;
        }
      }
      cp_async_16(wk + (buf * WB + r) * LDS + ch * 8, ksrc, bytes);
      cp_async_16(wv + (buf * WB + r) * LDS + ch * 8, vsrc, bytes);
    }
  };
  if (warp < nblocks) {
    load_block(warp, 0);
    cp_async_commit();
  }
  int buf = 0;
  for (int block = warp; block < nblocks; block += 4, buf ^= 1) {
    if (block + 4 < nblocks) {
      load_block(block + 4, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncwarp();
    warp_attend<2>(wk + buf * WB * LDS, wv + buf * WB * LDS, 0, c0 + block * WB, qf, row_ok, hi_here, row_lo,
                   p.scale_log2, m, l, o);
    __syncwarp();
  }
  __syncthreads();

  // combine the four warps through shared memory (the K/V buffers are free now)
  float* sm_m = reinterpret_cast<float*>(smem_raw);  // [4][16]
  float* sm_l = sm_m + 64;                           // [4][16]
  float* sm_o = sm_l + 64;                           // [4][16][D]
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int R = gid + i * 8;
    const float total = quad_sum(l[i]);
    if (tig == 0) {
      sm_m[warp * 16 + R] = m[i];
      sm_l[warp * 16 + R] = total;
    }
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) {
      sm_o[(warp * 16 + R) * D + dt * 8 + tig * 2] = o[dt][2 * i];
      sm_o[(warp * 16 + R) * D + dt * 8 + tig * 2 + 1] = o[dt][2 * i + 1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.gs * D; idx += 128) {
    const int R = idx / D, col = idx - R * D;
    const int g = slice * p.gs + R;
    if (g >= p.group) continue;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + R]);
    const float base = M == -INFINITY ? 0.f : M;
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(sm_m[w * 16 + R] - base);
      acc += sm_o[(w * 16 + R) * D + col] * f;
      L += sm_l[w * 16 + R] * f;
    }
    const int head = kvh * p.group + g;
    if (p.num_splits == 1) {
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
}

// --------------------------------------------------------------------------- decode, transposed
// The same split-sequence scheme with the roles of the matrix dimensions exchanged, which
// suits a handful of query heads much better: keys are the 16-row (M) side and the query
// heads of the group the 8-wide (N) side,
//     S^T[16 keys x 8 heads]  = K[16 keys x d]   . Q^T[d x 8 heads]
//     O^T[d x 8 heads]       += V^T[d x 16 keys] . P^T[16 keys x 8 heads]
// so that half of an accumulator is real work instead of a quarter (or less), the softmax
// touches 4 values per thread instead of 32, and K never goes through shared memory: like
// the weight-streaming projection, each lane fetches 16 contiguous bytes of "its" key row
// straight into the A fragments (the order of the head-size index inside a 32-wide slab is
// permuted identically in K and Q).  V goes through shared memory (cp.async, a private
// two-stage buffer per warp) and is read transposed by ldmatrix.trans; P^T reaches the
// B-fragment layout with movmatrix.trans.
// grid (splits, nkv * slices, requests); at most 8 query heads of a group per CTA.
#if HEAD_DIM % 32 == 0
constexpr int kTGs = 8;                       // query heads per CTA = the N side of one mma
constexpr int TLDS = D + 8;                   // padded V row
constexpr int kTSmemBytes = 4 * 2 * 16 * TLDS * 2 > (2 * 4 * 8 + 4 * 8 * D) * 4 ? 4 * 2 * 16 * TLDS * 2 : (2 * 4 * 8 + 4 * 8 * D) * 4;

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__global__ void __launch_bounds__(128) decode_attention_t_kernel(AttnParams p) {
  constexpr int SLABS = D / 32;               // 32-wide slabs of the head size (two k-steps each)
  constexpr int MT = D / 16;                  // 16-row tiles of O^T
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_trigger();
  pdl_wait();
  const int split = blockIdx.x, b = blockIdx.z;
  const int kvh = blockIdx.y / p.slices, slice = blockIdx.y % p.slices;
  const int* table = p.block_table + static_cast<size_t>(b) * p.table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int len = p.kv_len[b];
  const int lo = p.window > 0 ? max(0, len - p.window) : 0;
  int chunk = (len - lo + p.num_splits - 1) / p.num_splits;
  chunk = ((chunk + 63) / 64) * 64;
  const int c0 = lo + split * chunk;
  const int c1 = min(c0 + chunk, len) - 1;    // last key of this CTA's part (c1 < c0: nothing to do)
  const int head0 = kvh * p.group + slice * p.gs;
  const int heads_here = min(p.gs, p.group - slice * p.gs);

  // Q^T fragments: lane (g, t) holds Q[head g][32 s + 8 t .. + 7] for every slab s
  uint4 qv[SLABS];
#pragma unroll
  for (int s = 0; s < SLABS; ++s) {
    qv[s] = make_uint4(0, 0, 0, 0);
    if (g < heads_here)
      qv[s] = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(b) * p.nq + head0 + g) * D + 32 * s + 8 * t);
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};   // heads 2t and 2t + 1
  float o[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[mt][e] = 0.f;

  bf16* wv = reinterpret_cast<bf16*>(smem_raw) + warp * (2 * 16 * TLDS);   // [2][16][TLDS] values of this warp
  const int nblocks = c1 >= c0 ? (c1 - c0) / 16 + 1 : 0;
  auto key_offset = [&](int key) -> long {          // element offset of a key's row in the pools; -1: none
    if (key > c1) return -1;
    const int index = p.page_shift >= 0 ? key >> p.page_shift : key / p.page_size;
    const int slot = p.page_shift >= 0 ? key & (p.page_size - 1) : key - index * p.page_size;
    const int page = table[index];
    if (page < 0) return -1;
    return ((static_cast<long>(page) * p.nkv + kvh) * p.page_size + slot) * D;
  };
  auto load_values = [&](int block, int buf) {
    constexpr int CH = D / 8;
    const int t0 = c0 + block * 16;
#pragma unroll
    for (int c = lane; c < 16 * CH; c += 32) {
      const int r = c / CH, ch = c - r * CH;
      const long off = key_offset(t0 + r);
      cp_async_16(wv + (buf * 16 + r) * TLDS + ch * 8, off >= 0 ? p.v_pool + off + ch * 8 : p.v_pool, off >= 0 ? 16 : 0);
    }
  };
  if (warp < nblocks) {
    load_values(warp, 0);
    cp_async_commit();
  }
  int buf = 0;
  for (int block = warp; block < nblocks; block += 4, buf ^= 1) {
    const int t0 = c0 + block * 16;
    // keys of this block straight into the A fragments
    uint4 ka[SLABS], kb[SLABS];
    {
      const long offa = key_offset(t0 + g), offb = key_offset(t0 + g + 8);
#pragma unroll
      for (int s = 0; s < SLABS; ++s) {
        ka[s] = offa >= 0 ? ldg_stream16(p.k_pool + offa + 32 * s + 8 * t) : make_uint4(0, 0, 0, 0);
        kb[s] = offb >= 0 ? ldg_stream16(p.k_pool + offb + 32 * s + 8 * t) : make_uint4(0, 0, 0, 0);
      }
    }
    if (block + 4 < nblocks) {
      load_values(block + 4, buf ^ 1);
      cp_async_commit();
    }
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < SLABS; ++s) {
      const uint32_t a_lo[4] = {ka[s].x, kb[s].x, ka[s].y, kb[s].y};
      const uint32_t a_hi[4] = {ka[s].z, kb[s].z, ka[s].w, kb[s].w};
      mma_bf16(c, a_lo, qv[s].x, qv[s].y);
      mma_bf16(c, a_hi, qv[s].z, qv[s].w);
    }
    // c0, c1: key t0 + g, heads 2t, 2t+1;  c2, c3: key t0 + g + 8
    const bool vis_a = t0 + g <= c1, vis_b = t0 + g + 8 <= c1;     // the whole part lies inside [lo, len)
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
    if (block + 4 < nblocks) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncwarp();
    const bf16* vbuf = wv + buf * 16 * TLDS;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      uint32_t vf[4];
      ldmatrix_x4_trans(vf, vbuf + ((lane & 7) + ((lane >> 4) & 1) * 8) * TLDS + mt * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(o[mt], vf, pb0, pb1);
    }
    __syncwarp();
  }
  __syncthreads();

  // combine the four warps through shared memory
  float* sm_m = reinterpret_cast<float*>(smem_raw);   // [4][8]
  float* sm_l = sm_m + 32;                            // [4][8]
  float* sm_o = sm_l + 32;                            // [4][8 heads][D]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float total = l[h];
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
    if (g == 0) {
      sm_m[warp * 8 + 2 * t + h] = m[h];
      sm_l[warp * 8 + 2 * t + h] = total;
    }
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    sm_o[(warp * 8 + 2 * t) * D + mt * 16 + g] = o[mt][0];
    sm_o[(warp * 8 + 2 * t + 1) * D + mt * 16 + g] = o[mt][1];
    sm_o[(warp * 8 + 2 * t) * D + mt * 16 + g + 8] = o[mt][2];
    sm_o[(warp * 8 + 2 * t + 1) * D + mt * 16 + g + 8] = o[mt][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < heads_here * D; idx += 128) {
    const int h = idx / D, col = idx - h * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 8 + h]);
    const float base = M == -INFINITY ? 0.f : M;
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(sm_m[w * 8 + h] - base);
      acc += sm_o[(w * 8 + h) * D + col] * f;
      L += sm_l[w * 8 + h] * f;
    }
    const int head = head0 + h;
    if (p.num_splits == 1) {
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
}

#endif  // HEAD_DIM % 32 == 0

// grid (nq, requests), D threads: combine the splits of one (request, head)
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, int nq, int num_splits) {
  pdl_trigger();
  pdl_wait();
  const long base = (static_cast<long>(blockIdx.y) * nq + blockIdx.x) * num_splits;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  const float ref = M == -INFINITY ? 0.f : M;
  for (int col = threadIdx.x; col < D; col += blockDim.x) {
    float acc = 0.f, L = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float f = exp2f(part_ml[(base + s) * 2] - ref);
      acc += part_o[(base + s) * D + col] * f;
      L += part_ml[(base + s) * 2 + 1] * f;
    }
    out[(static_cast<long>(blockIdx.y) * nq + blockIdx.x) * D + col] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  }
}

constexpr int kMergeThreads = D < 128 ? D : 128;
static int heads_per_cta(int group) { return group < 16 ? group : 16; }

}  // namespace b200

using namespace b200;

static int fill_common(AttnParams& p, const void* q, const void* k_pool, const void* v_pool, void* out,
                       const int* positions, const int* block_table, int table_stride, int page_size, int nq,
                       int nkv, float scale, int window) {
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || table_stride <= 0) return B200_ERR_BAD_SIZE;
  p.q = static_cast<const bf16*>(q);
  p.k_pool = static_cast<const bf16*>(k_pool);
  p.v_pool = static_cast<const bf16*>(v_pool);
  p.out = static_cast<bf16*>(out);
  p.positions = positions;
  p.block_table = block_table;
  p.table_stride = table_stride;
  p.page_size = page_size;
  p.page_shift = -1;
  for (int b = 0; b < 20; ++b)
    if ((1 << b) == page_size) p.page_shift = b;
  p.nq = nq;
  p.nkv = nkv;
  p.group = nq / nkv;
  p.gs = heads_per_cta(p.group);
  p.slices = (p.group + p.gs - 1) / p.gs;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  return 0;
}

extern "C" int b200_attention_head_dim() { return HEAD_DIM; }

// Rows per CTA of the prefill kernel: the caller cuts entries into tiles of
// tokens_per_tile = rows / heads_per_cta consecutive tokens.
extern "C" int b200_attention_prefill_rows() { return 64; }

extern "C" int b200_attention_prefill_bf16(const void* q, const void* k_pool, const void* v_pool, void* out,
                                           const int* positions, const int* block_table, int table_stride,
                                           int page_size, int nq, int nkv, float scale, int window,
                                           const int* tile_entry, const int* tile_start, const int* tile_count,
                                           int num_tiles, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  AttnParams p{};
  if (int e = fill_common(p, q, k_pool, v_pool, out, positions, block_table, table_stride, page_size, nq, nkv, scale, window)) return e;
  p.tile_entry = tile_entry;
  p.tile_start = tile_start;
  p.tile_count = tile_count;
  static DeviceOnce once;
  if (int e = configure_once(once, prefill_attention_kernel<4>, kSmemBytes)) return e;
  dim3 grid(nkv * p.slices, num_tiles);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  launch(prefill_attention_kernel<4>, dim3(grid), dim3(128), kSmemBytes, stream, p);
  return launch_status();
}

extern "C" long b200_attention_decode_scratch_floats(int requests, int nq, int num_splits) {
  return num_splits <= 1 ? 0 : static_cast<long>(requests) * nq * num_splits * (D + 2);
}

extern "C" int b200_attention_decode_bf16(const void* q, const void* k_pool, const void* v_pool, void* out,
                                          const int* kv_len, const int* block_table, int table_stride,
                                          int page_size, int requests, int nq, int nkv, float scale, int window,
                                          int num_splits, float* scratch, long scratch_floats, cudaStream_t stream) {
  if (requests <= 0) return 0;
  AttnParams p{};
  if (int e = fill_common(p, q, k_pool, v_pool, out, nullptr, block_table, table_stride, page_size, nq, nkv, scale, window)) return e;
  if (num_splits < 1 || requests > 65535) return B200_ERR_BAD_SIZE;
  if (scratch_floats < b200_attention_decode_scratch_floats(requests, nq, num_splits)) return 10004;
  p.kv_len = kv_len;
  p.num_splits = num_splits;
  p.part_o = scratch;
  p.part_ml = scratch + static_cast<long>(requests) * nq * num_splits * D;
#if HEAD_DIM % 32 == 0
  // The transposed kernel, unless LLM_RUNTIME_STUDY_B200_DECODE_ATTENTION=rows asks for the
  // older one with the query heads on the 16-row side (kept for head sizes like 48 and 80).
  static int use_rows = -1;
  if (use_rows < 0) {
    const char* e = getenv("LLM_RUNTIME_STUDY_B200_DECODE_ATTENTION");
    use_rows = (e && e[0] == 'r') ? 1 : 0;
  }
  if (!use_rows) {
    p.gs = p.group < kTGs ? p.group : kTGs;
    p.slices = (p.group + p.gs - 1) / p.gs;
    static DeviceOnce once_t;
    if (int e = configure_once(once_t, decode_attention_t_kernel, kTSmemBytes)) return e;
    dim3 tgrid(num_splits, nkv * p.slices, requests);
    launch(decode_attention_t_kernel, tgrid, dim3(128), kTSmemBytes, stream, p);
  } else
#endif
  {
    static DeviceOnce once;
    if (int e = configure_once(once, decode_attention_kernel, kSmemBytes)) return e;
    dim3 grid(num_splits, nkv * p.slices, requests);
    launch(decode_attention_kernel, dim3(grid), dim3(128), kSmemBytes, stream, p);
  }
  if (int e = launch_status()) return e;
  if (num_splits > 1) {
    dim3 mgrid(nq, requests);
    launch(decode_merge_kernel, dim3(mgrid), dim3(kMergeThreads), 0, stream, p.part_o, p.part_ml, p.out, nq, num_splits);
  }
  return launch_status();
}

// --------------------------------------------------------------------------------------
// Allocation-free variant of the decode entry point (see attention_noalloc.h for the
// contract and for who needs it).  The scratch that b200_attention_decode_bf16 takes from
// its caller lives here, in the library image.
#include "attention_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[B200_NOALLOC_SCRATCH_FLOATS];

// `g_noalloc_scratch` in host code is only a handle for the runtime, not an address a
// kernel could use; the device address is asked for once per device and kept.
static float* noalloc_scratch_address(int* status) {
  constexpr int kMaxDevices = 64;
  static float* address[kMaxDevices] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
    *status = e != cudaSuccess ? static_cast<int>(e) : B200_ERR_NOALLOC_SETUP;
    return nullptr;
  }
  if (address[device] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *status = e != cudaSuccess ? static_cast<int>(e) : B200_ERR_NOALLOC_SETUP;
      return nullptr;
    }
    address[device] = p;
  }
  *status = 0;
  return address[device];
}

extern "C" int b200_attention_decode_bf16_noalloc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                                  const int* kv_len, const int* block_table, int table_stride,
                                                  int page_size, int requests, int nq, int nkv, float scale,
                                                  int window, int num_splits, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (num_splits < 1) return B200_ERR_BAD_SIZE;
  const long needed = b200_attention_decode_scratch_floats(requests, nq, num_splits);
  if (needed > B200_NOALLOC_SCRATCH_FLOATS) return B200_ERR_NOALLOC_TOO_LARGE;
  int status = 0;
  float* scratch = noalloc_scratch_address(&status);
  if (scratch == nullptr) return status;
  return b200_attention_decode_bf16(q, k_pool, v_pool, out, kv_len, block_table, table_stride, page_size, requests,
                                    nq, nkv, scale, window, num_splits, scratch, B200_NOALLOC_SCRATCH_FLOATS, stream);
}
