// The decode-side W4A16 kernel for sm_100a: one persistent kernel serves the
// M=1 GEMV, the skinny GEMM of a speculative-verify block (M <= 16) and the
// lm_head GEMV with the argmax fused into its epilogue.
//
// Replaces k_prep + k_gemv + k_reduce, k_prep_m + k_gemm_small + k_reduce_bf16_m
// and k_gemm_mma of the reference (src/kernels/gemv_w4a16.cu:74-279,673-865) and,
// for lm_head, the separate argmax kernels (src/kernels/elementwise.cu:96-194).
//
// The path is HBM-bound (every weight byte is read exactly once); what limits a
// straightforward port is instruction issue, and on this part the legacy
// mma.sync pipe in particular (measured: ~3 TB/s ceiling). So the multiply runs
// on the 5th-generation tensor core with the weights as the TMEM-resident A
// operand:
//   * persistent grid, two CTAs per SM. The (128-row tile, k group) units of the
//     matrix are dealt out as equal contiguous ranges, so every CTA streams the same
//     number of bytes whatever N and K are. A row tile whose K range is shared by
//     several CTAs is finished by the last CTA to arrive, which adds the partial tiles
//     in a fixed order (bitwise reproducible, no float atomics). Shared tiles are
//     processed FIRST, so that reduction overlaps everybody's main loop.
//   * warp roles: a weight producer streams the CTA's contiguous share of the weight
//     stream through a ring of shared-memory stages with 1-D bulk async copies
//     (cp.async.bulk + mbarrier); it does not wait for the previous kernel
//     (programmatic dependent launch), so one layer's weights start flowing while the
//     previous layer drains. An activation warp stages x as the K-major B operand.
//     Four consumer warps own one output row per thread: 16 bytes of packed int4 ->
//     bf16 (128+q) pairs with one LOP3 per two weights, an exact packed bf16 subtract
//     of (128+zp), then tcgen05.st into tensor memory. One thread issues
//     tcgen05.mma (M=128 rows, N=16 tokens, K=16) per 16-k slab with A from TMEM and
//     commits to an mbarrier; the consumers read the fp32 group sums back with
//     tcgen05.ld and apply the group scale:  y += s * sum((q - zp) x).
#include <cfloat>
#include <climits>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace w4a16 {
namespace {

constexpr int CW = 8;                                 // consumer warps: 128 rows x 2 k-halves, one row per thread
constexpr int kWarps = CW + 4;                        // + weight producer, 2 MMA issuers, activation warp
constexpr int NCT = CW * 32;                          // consumer threads
constexpr int kRowWarps = 4;                          // warps per k-half = TMEM lane quadrants
constexpr int kItemGroups = 2;                        // k groups per weight ring stage
constexpr int kStageBytes = kItemGroups * kTileGroupBytes;  // 17152
static_assert(kStageBytes % 128 == 0, "ring stages must stay 128-byte aligned");
constexpr int kXBufs = 3;                             // activation chunk buffers
constexpr int kXGroupBytes = 4096;                    // B operand of one k group: 16 slabs(8 k) x 16 tokens x 16 B
constexpr int kFirstChunk = 2;                        // groups in a CTA's first activation chunk (short start-up)
constexpr int kMaxChunkGroups = 8;
constexpr int kTokens = 16;                           // N of the MMA
#ifndef W4A16_NB
#define W4A16_NB 3
#endif
constexpr int NB = W4A16_NB;                          // groups in flight in tensor memory
constexpr uint32_t kTmemCols = NB <= 3 ? 256 : 512;   // allocation: A NB x 64 columns, D NB x 16 columns
constexpr uint32_t kTmemA = 0, kTmemD = NB * 64;
static_assert(NB * 80 <= 512, "tensor memory budget");
constexpr int kMinCtas = NB <= 3 ? 2 : 1;
constexpr uint32_t kSpinLimit = 1u << 20;             // polls before a wait gives up
constexpr uint32_t kMagic = 0x43004300u;              // bf16 pair (128.0, 128.0)
constexpr uint32_t kNibMask = 0x000F000Fu;
constexpr int kConsumerBar = 1;                       // named barrier of the consumer warps

struct SkinnyParams {
  const uint8_t* stream;  // weight stream, kTileGroupBytes per (row tile, group)
  const uint16_t* x;      // [M][K] bf16
  void* y;                // bf16 or fp32 [M][ldy], may be null in argmax mode
  int y_f32;
  long long ldy;  // elements between rows of y
  int y_col0;     // first column of this launch's rows inside y
  int M, N, K, G, tiles;
  int chunk_groups;  // k groups per activation chunk (even)
  float* partial;
  unsigned* counters;  // [tiles * 4 + 1], zero between launches
  int argmax;
  int32_t* ids;
  void* pairs_out;  // M x {float,int}
  int row_offset;
  void* cta_pairs;  // [grid][16] x {float,int}
  int* status;
  unsigned long long* dbg;  // TEMP: per-CTA timestamps
  int debug_skip;           // TEMP
  int npeers;  // extra destinations for y (fused all-gather), 0 = none
  uint16_t* y_peers[8];
};

struct Pair {
  float v;
  int i;
};

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

// ---- the order in which a CTA walks its unit range [u0,u1) -------------------------------
// Row tiles that this CTA shares with a neighbour come first (the piece at the end of the
// range, then the piece at its start), whole tiles after, so the cross-CTA reduction of the
// shared tiles overlaps everybody's main loop instead of sitting at the end of the kernel.
// Every role (weight producer, activation warp, MMA issuer, consumers) runs the same iterator.
struct Chunk {
  int tile, g, n;      // row tile, first group, number of groups (<= chunk_groups)
  int seg_g0, seg_g1;  // the segment this chunk belongs to: groups [seg_g0, seg_g1) of `tile`
  bool seg_last;       // last chunk of its segment
};

struct WorkIter {
  int G, CG, t_first, t_last, head_g0, tail_g1;
  bool single, head_partial, tail_partial, first;
  int phase, t;
  int s_tile, s_g0, s_g1, g;  // current segment and cursor
  bool have;

  __device__ void init(int u0, int u1, int G_, int CG_) {
    G = G_;
    CG = CG_;
    t_first = u0 / G;
    t_last = (u1 - 1) / G;
    head_g0 = u0 - t_first * G;
    tail_g1 = u1 - t_last * G;
    single = (t_first == t_last);
    head_partial = single ? !(head_g0 == 0 && tail_g1 == G) : (head_g0 != 0);
    tail_partial = single ? false : (tail_g1 != G);
    phase = 0;
    t = t_first;
    have = false;
    first = true;
    s_tile = s_g0 = s_g1 = g = 0;
  }
  __device__ bool next_segment() {
    if (phase == 0) {
      phase = 1;
      if (tail_partial) {
        s_tile = t_last; s_g0 = 0; s_g1 = tail_g1;
        return true;
      }
    }
    if (phase == 1) {
      phase = 2;
      if (head_partial) {
        s_tile = t_first; s_g0 = head_g0; s_g1 = single ? tail_g1 : G;
        return true;
      }
    }
    while (t <= t_last) {
      const int tt = t++;
      if (tt == t_first && head_partial) continue;
      if (tt == t_last && tail_partial) continue;
      s_tile = tt; s_g0 = 0; s_g1 = G;
      return true;
    }
    return false;
  }
  __device__ bool next(Chunk& c) {
    if (!have || g >= s_g1) {
      if (!next_segment()) return false;
      have = true;
      g = s_g0;
    }
    int n = first ? kFirstChunk : CG;
    first = false;
    if (s_g1 - g < n) n = s_g1 - g;
    c.tile = s_tile; c.g = g; c.n = n; c.seg_g0 = s_g0; c.seg_g1 = s_g1;
    g += n;
    c.seg_last = (g == s_g1);
    return true;
  }
};

// dynamic shared memory:
//   [weight ring D stages][x buffers kXBufs x chunk_groups x 4 KB][half sums 128 x 16 fp32]
//   [mbarriers][tmem base][flag]
constexpr int kHalfSumBytes = kTileRows * kTokens * 4 + NB * NCT * 4;  // + per-thread scale of each group in flight
template <int D>
__host__ __device__ constexpr int skinny_bar_count() { return 2 * D + 2 * NB + 2 * kXBufs + 1; }
template <int D>
__host__ __device__ constexpr int skinny_fixed_smem() {
  return D * kStageBytes + kHalfSumBytes + skinny_bar_count<D>() * 8 + 16;
}

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define TRACE(role, grp, ev) do { if (p.dbg && blockIdx.x == 7 && lane == 0 && (grp) < 24) p.dbg[4096 + ((role) * 24 + (grp)) * 4 + (ev)] = clock64(); } while (0)
#define DBG_T(i) do { if (p.dbg && tid == 0) p.dbg[blockIdx.x * 8 + (i)] = gtime(); } while (0)

// MC = token columns each consumer thread reads back (power of two >= M)
template <int MC, int D>
__global__ void __launch_bounds__(kWarps * 32, kMinCtas) k_skinny(const SkinnyParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int SLOT = kTileRows * kTokens;  // floats per partial tile

  const int XB = p.chunk_groups * kXGroupBytes;
  uint8_t* ring = smem;
  uint8_t* xbuf = ring + D * kStageBytes;
  float* halfsum = reinterpret_cast<float*>(xbuf + kXBufs * XB);  // [MC][128]: sums of the odd groups
  float* scs = halfsum + kTileRows * kTokens;  // [NB][consumer thread]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(halfsum) + kHalfSumBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + skinny_bar_count<D>());
  int* sflag = reinterpret_cast<int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, M = p.M;
  const int U = p.tiles * G;
  const int u0 = static_cast<int>(static_cast<long long>(U) * blockIdx.x / gridDim.x);
  const int u1 = static_cast<int>(static_cast<long long>(U) * (blockIdx.x + 1) / gridDim.x);

  const uint32_t ring_a = smem_u32(ring);
  const uint32_t xbuf_a = smem_u32(xbuf);
  const uint32_t wfull_a = smem_u32(bars);            // [D]  weights landed
  const uint32_t wempty_a = wfull_a + D * 8;          // [D]  stage free again (8 consumer warps)
  const uint32_t afull_a = wempty_a + D * 8;          // [NB] A operand of a group is in TMEM (8 consumer warps)
  const uint32_t mdone_a = afull_a + NB * 8;          // [NB] the group's MMAs have completed: D readable, A reusable
  const uint32_t xfull_a = mdone_a + NB * 8;          // [kXBufs] activation chunk staged
  const uint32_t xempty_a = xfull_a + kXBufs * 8;     // [kXBufs] both issuers are done with the chunk
  const uint32_t alldone_a = xempty_a + kXBufs * 8;   // [1]  consumers are finished with tensor memory

  DBG_T(0);
  // token rows >= M of every B-operand buffer stay zero for the whole kernel
  for (int i = tid; i < kXBufs * XB / 16; i += kWarps * 32) reinterpret_cast<uint4*>(xbuf)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async();  // the tensor core reads these buffers through the async proxy
  if (tid == 0) {
    for (int i = 0; i < D; ++i) {
      mbar_init(wfull_a + i * 8, 1);
      mbar_init(wempty_a + i * 8, CW);
    }
    for (int i = 0; i < NB; ++i) {
      mbar_init(afull_a + i * 8, CW);
      mbar_init(mdone_a + i * 8, 1);
    }
    for (int i = 0; i < kXBufs; ++i) {
      mbar_init(xfull_a + i * 8, 1);
      mbar_init(xempty_a + i * 8, 2);
    }
    mbar_init(alldone_a, CW);
    fence_mbar_init();
  }
  if (warp == CW + 1) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();

  // ================================================================ weight producer
  // One thread streams this CTA's share of the weight stream, one stage (two k groups of the
  // 128-row tile, 17 KB, contiguous in memory) per bulk copy. It does not wait for the
  // previous kernel: weights never depend on it.
  if (warp == CW) {
    if (lane == 0) {
      WorkIter it;
      it.init(u0, u1, G, p.chunk_groups);
      Chunk c;
      int st = 0;
      uint32_t ph = 1;  // a fresh "empty" barrier reads as already released
      bool ok = true;
      while (ok && it.next(c)) {
        for (int gi = 0; gi < c.n; gi += kItemGroups) {
          const int ng = (c.n - gi < kItemGroups) ? c.n - gi : kItemGroups;
          if (!mbar_wait_bounded_relaxed(wempty_a + st * 8, ph, kSpinLimit)) {
            atomicExch(p.status, W4A16_ETIMEOUT);
            ok = false;
            break;
          }
          mbar_expect_tx(wfull_a + st * 8, ng * kTileGroupBytes);
          bulk_g2s(ring_a + st * kStageBytes,
                   p.stream + (static_cast<size_t>(c.tile) * G + c.g + gi) * kTileGroupBytes, ng * kTileGroupBytes,
                   wfull_a + st * 8);
          if (++st == D) {
            st = 0;
            ph ^= 1;
          }
        }
      }
    }
    return;
  }

  // ================================================================ MMA issuers
  // Two threads (one per warp) take the k groups alternately. Per group: 8 x tcgen05.mma
  // (128 rows x 16 tokens x 16 k) with A from tensor memory and B (activations) from shared
  // memory, then a commit that tells the consumers the group's fp32 sums are ready and its A
  // columns may be overwritten.
  if (warp == CW + 1 || warp == CW + 2) {
    const int me = warp - (CW + 1);
    if (lane == 0) {
      WorkIter it;
      it.init(u0, u1, G, p.chunk_groups);
      Chunk c;
      constexpr uint32_t idesc = umma_idesc_bf16(kTileRows, kTokens);
      int xb = 0, b = 0, par = 0, tg = 0;
      uint32_t xph = 0, bph = 0;
      bool ok = true;
      while (ok && it.next(c)) {
        if (!mbar_wait_bounded(xfull_a + xb * 8, xph, kSpinLimit)) {
          atomicExch(p.status, W4A16_ETIMEOUT);
          break;
        }
        // descriptor of the chunk's first 16-k slab: 8-k core-matrix columns 256 B apart, token
        // groups 128 B apart; each following slab starts 512 B (32 descriptor units) later
        uint64_t bdesc = umma_desc_kmajor(xbuf_a + xb * XB, 256, 128);
        bool issued = false;
        for (int gi = 0; gi < c.n; ++gi) {
          if (par == me) {
            if (!mbar_wait_bounded(afull_a + b * 8, bph, kSpinLimit)) {
              atomicExch(p.status, W4A16_ETIMEOUT);
              ok = false;
              break;
            }
            TRACE(2 + me, tg, 0);
            tc_fence_after();
            const uint32_t d_t = tmem + kTmemD + b * kTokens, a_t = tmem + kTmemA + b * 64;
#ifndef EXP_NOMMA
            umma_bf16_ts(d_t, a_t, bdesc, idesc, 0);
#pragma unroll
            for (int s = 1; s < 8; ++s) umma_bf16_ts(d_t, a_t + s * 8, bdesc + s * 32, idesc, 1);
#endif
            umma_commit(mdone_a + b * 8);
            TRACE(2 + me, tg, 1);
            issued = true;
          }
          ++tg;
          bdesc += 8 * 32;
          par ^= 1;
          if (++b == NB) {
            b = 0;
            bph ^= 1;
          }
        }
        // the chunk buffer is free once both issuers' MMAs on it have completed
        if (issued) umma_commit(xempty_a + xb * 8);
        else mbar_arrive(xempty_a + xb * 8);
        if (++xb == kXBufs) {
          xb = 0;
          xph ^= 1;
        }
      }
    }
    __syncwarp();
    if (me == 0) {
      // tensor memory goes back only after every consumer has read its last sums
      mbar_wait_bounded_relaxed(alldone_a, 0, kSpinLimit);
      tc_fence_after();
      tmem_dealloc(tmem, kTmemCols);
    }
    return;
  }

  // ================================================================ activation warp
  // Waits for the previous kernel (it produced x), then stages x chunk by chunk as the
  // K-major B operand: core matrices of 8 tokens x 8 k (16 B per token row), laid out
  // [8-k slab][token group of 8][token][16 B].
  if (warp == CW + 3) {
    pdl_wait();
    WorkIter it;
    it.init(u0, u1, G, p.chunk_groups);
    Chunk c;
    int xb = 0;
    uint32_t eph = 1;
    while (it.next(c)) {
      if (!mbar_wait_bounded_relaxed(xempty_a + xb * 8, eph, kSpinLimit)) {
        atomicExch(p.status, W4A16_ETIMEOUT);
        break;
      }
      const int pieces = c.n * 16 * M;  // 16-byte pieces: (8-k slab, token)
      for (int i = lane; i < pieces; i += 32) {
        const int m = i % M, kc = i / M;
        cp_async16(xbuf_a + xb * XB + kc * 256 + (m >> 3) * 128 + (m & 7) * 16,
                   p.x + static_cast<size_t>(m) * p.K + c.g * kGroup + kc * 8);
      }
      cp_async_commit();
      cp_async_wait_all();
      fence_proxy_async();  // generic-proxy writes -> visible to the tensor core's async-proxy reads
      __syncwarp();
      if (lane == 0) mbar_arrive(xfull_a + xb * 8);
      if (++xb == kXBufs) {
        xb = 0;
        eph ^= 1;
      }
    }
    return;
  }

  // ================================================================ consumer warps
  // thread = one output row of the 128-row tile (TMEM lane 32 * (warp % 4) + lane) and one half
  // of every k group: warps 0-3 unpack k 0..63, warps 4-7 k 64..127. The fp32 sums of a group
  // are folded by the half whose index equals the group's parity, so both halves carry a partial
  // sum that is combined once per row tile.
  const int q = warp & (kRowWarps - 1), h = warp / kRowWarps;
  const int row = q * 32 + lane;
  const uint32_t tlane = static_cast<uint32_t>(q * 32) << 16;

  float fin[MC];
#pragma unroll
  for (int m = 0; m < MC; ++m) fin[m] = 0.f;
  float best_v[MC];
  int best_i[MC];
#pragma unroll
  for (int m = 0; m < MC; ++m) {
    best_v[m] = -FLT_MAX;
    best_i[m] = INT_MAX;
  }

  // Final values of one row tile are in registers: write them out / fold into the argmax.
  auto finalize = [&](int tile, const float (&v)[MC]) {
    const int r = tile * kTileRows + row;
    if (r >= p.N) return;
#pragma unroll
    for (int m = 0; m < MC; ++m) {
      if (m >= M) continue;
      const uint16_t hb = float_to_bf16_bits(v[m]);
      if (p.y) {
        const size_t o = static_cast<size_t>(m) * p.ldy + p.y_col0 + r;
        if (p.y_f32) static_cast<float*>(p.y)[o] = v[m];
        else static_cast<uint16_t*>(p.y)[o] = hb;
        for (int qq = 0; qq < p.npeers; ++qq) p.y_peers[qq][o] = hb;
      }
      if (p.argmax) {
        const float lv = bf16_bits_to_float(hb);
        if (better(lv, r, best_v[m], best_i[m])) {
          best_v[m] = lv;
          best_i[m] = r;
        }
      }
    }
  };

  bool dead = false;
  // Groups in flight in tensor memory: buffers are used round-robin, `ob` is the oldest one.
  // sc0..sc2 = this row's scale of the group in each buffer, par0..2 = that group's parity.
  int npend = 0, b = 0, ob = 0, gpar = 0, opar = 0;
  uint32_t oph = 0;
  // The oldest group in flight has completed: its A columns may be overwritten, and the half
  // responsible for it folds its sums: y += s * sum((q-zp) x).
  auto retire_oldest = [&]() {
    if (!dead && !mbar_wait_bounded(mdone_a + ob * 8, oph, kSpinLimit)) {
      dead = true;
      atomicExch(p.status, W4A16_ETIMEOUT);
    }
    if (opar == h) {
      tc_fence_after();
      float d[MC];
      tmem_ld<MC>(tmem + tlane + kTmemD + ob * kTokens, d);
      tmem_wait_ld();
      const float sc = scs[ob * NCT + tid];
#pragma unroll
      for (int m = 0; m < MC; ++m) fin[m] = fmaf(sc, d[m], fin[m]);
    }
    --npend;
    opar ^= 1;
    if (++ob == NB) {
      ob = 0;
      oph ^= 1;
    }
  };

  // Split tiles: each row-warp publishes its 32 rows on its own and moves on; whichever warp
  // turns out to be the last contributor of its rows adds the pieces up at the end of the kernel.
  // (tile, first/last contributing CTA, arrival ticket) of up to two split tiles, in lane 0.
  int sp_n = 0, sp_tile0 = 0, sp_cf0 = 0, sp_cl0 = 0, sp_tile1 = 0, sp_cf1 = 0, sp_cl1 = 0;
  unsigned sp_old0 = 0, sp_old1 = 0;
  bool waited_pdl = false;
  auto before_global_write = [&]() {
    if (!waited_pdl) {
      pdl_wait();  // outputs and the shared scratch belong to the previous kernel until now
      waited_pdl = true;
    }
  };

  WorkIter it;
  it.init(u0, u1, G, p.chunk_groups);
  Chunk c;
  int wst = 0, tg = 0;
  uint32_t wph = 0;
  bool first_chunk = true;

  while (it.next(c)) {
    for (int gi = 0; gi < c.n; ++gi) {
      if ((gi & 1) == 0) {
        if (!dead && !mbar_wait_bounded(wfull_a + wst * 8, wph, kSpinLimit)) {
          dead = true;
          atomicExch(p.status, W4A16_ETIMEOUT);
        }
        if (first_chunk) DBG_T(2);
        first_chunk = false;
      }
      if (q == 0) TRACE(h, tg, 0);
      const uint8_t* blk = ring + wst * kStageBytes + (gi & 1) * kTileGroupBytes;
      const uint32_t zp = blk[kTgZpOff + row];
      const uint32_t zpair = __byte_perm(zp, 0x43434343u, 0x4040);  // bf16 pair (128+zp, 128+zp)
      if (gpar == h) {
        scs[b * NCT + tid] = bf16_bits_to_float(reinterpret_cast<const uint16_t*>(blk + kTgScaleOff)[row]);
      }
      if (p.debug_skip != 1) {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int j = 2 * h + jj;  // 32-k chunk of the group
          const uint4 wq = *reinterpret_cast<const uint4*>(blk + j * kChunkBytes + row * 16);
          const uint32_t w[4] = {wq.x, wq.y, wq.z, wq.w};
          uint32_t a[16];
#ifdef EXP_NOUNPACK
#pragma unroll
          for (int i = 0; i < 16; ++i) a[i] = w[i & 3] ^ zpair;
#else
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            a[4 * i + 0] = sub_bf16x2((w[i] & kNibMask) | kMagic, zpair);
            a[4 * i + 1] = sub_bf16x2(((w[i] >> 4) & kNibMask) | kMagic, zpair);
            a[4 * i + 2] = sub_bf16x2(((w[i] >> 8) & kNibMask) | kMagic, zpair);
            a[4 * i + 3] = sub_bf16x2(((w[i] >> 12) & kNibMask) | kMagic, zpair);
          }
#endif
#ifdef EXP_NOST
#pragma unroll
          for (int i = 0; i < 16; ++i) asm volatile("" ::"r"(a[i]));
#else
          tmem_st16(tmem + tlane + kTmemA + b * 64 + j * 16, a);
#endif
        }
      }
      // While this group's stores drain into tensor memory, retire the oldest group that is
      // still in flight (its MMAs were issued two groups ago); that also frees the buffer the
      // next group will be written to.
      if (q == 0) TRACE(h, tg, 1);
      if (npend == NB - 1) retire_oldest();
      if (q == 0) TRACE(h, tg, 2);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(afull_a + b * 8);  // this warp's share of the A operand is in place
      if (q == 0) TRACE(h, tg, 3);
      ++tg;
      ++npend;
      gpar ^= 1;
      if (++b == NB) b = 0;
      if ((gi & 1) == 1 || gi == c.n - 1) {
        if (lane == 0) mbar_arrive(wempty_a + wst * 8);  // (ordered after every lane's reads by the __syncwarp)
        if (++wst == D) {
          wst = 0;
          wph ^= 1;
        }
      }
    }

    if (c.seg_last) {
      // ---- end of this CTA's segment of row tile c.tile: groups [seg_g0, seg_g1) ----
      while (npend) retire_oldest();
      // combine the two halves' sums: odd-group sums travel through shared memory
      if (h == 1) {
#pragma unroll
        for (int m = 0; m < MC; ++m) halfsum[m * kTileRows + row] = fin[m];
      }
      named_bar_sync(kConsumerBar, NCT);
      if (h == 0) {
#pragma unroll
        for (int m = 0; m < MC; ++m) fin[m] += halfsum[m * kTileRows + row];
      }
      named_bar_sync(kConsumerBar, NCT);  // halfsum may be rewritten by the next segment
      if (h == 0) {
        before_global_write();
        const int tile = c.tile;
        if (c.seg_g0 == 0 && c.seg_g1 == G) {
          finalize(tile, fin);
        } else {
          const long long X0 = static_cast<long long>(tile) * G;
          const int c_first = static_cast<int>(((X0 + 1) * gridDim.x - 1) / U);
          const int c_last = static_cast<int>(((X0 + G) * gridDim.x - 1) / U);
          const int which = (u0 / G == tile) ? 0 : 1;
          float* slot = p.partial + (static_cast<size_t>(blockIdx.x) * 2 + which) * SLOT;
#pragma unroll
          for (int m = 0; m < MC; ++m) slot[m * kTileRows + row] = fin[m];
          __syncwarp();
          if (lane == 0) {
            __threadfence();  // release: this warp's partial rows (ordered by the __syncwarp) before the ticket
            const unsigned old = atomicAdd(p.counters + tile * kRowWarps + q, 1u);
            if (sp_n == 0) {
              sp_tile0 = tile; sp_cf0 = c_first; sp_cl0 = c_last; sp_old0 = old;
            } else {
              sp_tile1 = tile; sp_cf1 = c_first; sp_cl1 = c_last; sp_old1 = old;
            }
            ++sp_n;
          }
        }
      }
#pragma unroll
      for (int m = 0; m < MC; ++m) fin[m] = 0.f;
    }
  }
  DBG_T(3);

  // tensor memory is no longer read by this warp
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(alldone_a);

  if (dead) {  // let whatever is still in flight land before the CTA exits
    for (int s = 0; s < D; ++s) mbar_wait_bounded(wfull_a + s * 8, 0, 1u << 16);
  }
  if (h == 1 && !p.argmax) return;

  // ---- split tiles: the warp that drew the last ticket for its rows adds the pieces up ----
  if (h == 0) {
    const int n = __shfl_sync(0xffffffffu, sp_n, 0);
    for (int i = 0; i < n; ++i) {
      const int tile = __shfl_sync(0xffffffffu, i ? sp_tile1 : sp_tile0, 0);
      const int c_first = __shfl_sync(0xffffffffu, i ? sp_cf1 : sp_cf0, 0);
      const int c_last = __shfl_sync(0xffffffffu, i ? sp_cl1 : sp_cl0, 0);
      const unsigned old = __shfl_sync(0xffffffffu, i ? sp_old1 : sp_old0, 0);
      if (old != static_cast<unsigned>(c_last - c_first)) continue;  // someone else finishes these rows
      if (lane == 0) {
        p.counters[tile * kRowWarps + q] = 0;  // every contributor has arrived: leave it clean
        __threadfence();                       // acquire side for the reads below
      }
      __syncwarp();
      float v[MC];
#pragma unroll
      for (int m = 0; m < MC; ++m) v[m] = 0.f;
      for (int cc = c_first; cc <= c_last; ++cc) {  // fixed order: bitwise reproducible
        const int cu0 = static_cast<int>(static_cast<long long>(U) * cc / gridDim.x);
        const int wc = (cu0 / G == tile) ? 0 : 1;
        const float* sl = p.partial + (static_cast<size_t>(cc) * 2 + wc) * SLOT;
#pragma unroll
        for (int m = 0; m < MC; ++m) v[m] += __ldcg(sl + m * kTileRows + row);
      }
      finalize(tile, v);
    }
  }

  if (p.argmax) {
    // ---- fused argmax: thread -> warp -> CTA -> grid, larger value then lower index ----
    // (only the h == 0 warps hold candidates; the others carry the neutral element)
    before_global_write();
#pragma unroll
    for (int m = 0; m < MC; ++m)
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_v[m], off);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i[m], off);
        if (better(ov, oi, best_v[m], best_i[m])) {
          best_v[m] = ov;
          best_i[m] = oi;
        }
      }
    named_bar_sync(kConsumerBar, NCT);
    // per-warp candidates go through the (now idle) weight ring: every stage was consumed
    Pair* cand = reinterpret_cast<Pair*>(ring);  // [CW][16]
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MC; ++m) cand[warp * 16 + m] = Pair{best_v[m], best_i[m]};
    }
    named_bar_sync(kConsumerBar, NCT);
    Pair* cta_pairs = static_cast<Pair*>(p.cta_pairs);
    if (tid < M) {
      Pair bb{-FLT_MAX, INT_MAX};
      for (int w = 0; w < CW; ++w) {
        const Pair qq = cand[w * 16 + tid];
        if (better(qq.v, qq.i, bb.v, bb.i)) bb = qq;
      }
      cta_pairs[blockIdx.x * 16 + tid] = bb;
    }
    named_bar_sync(kConsumerBar, NCT);
    if (tid == 0) {
      __threadfence();
      const unsigned old = atomicAdd(p.counters + p.tiles * kRowWarps, 1u);
      const int last = (old == gridDim.x - 1);
      if (last) {
        p.counters[p.tiles * kRowWarps] = 0;
        __threadfence();
      }
      *sflag = last;
    }
    named_bar_sync(kConsumerBar, NCT);
    if (*sflag && tid < M) {
      Pair bb{-FLT_MAX, INT_MAX};
      for (unsigned cc = 0; cc < gridDim.x; ++cc) {
        Pair qq;
        qq.v = __ldcg(&cta_pairs[cc * 16 + tid].v);
        qq.i = __ldcg(&cta_pairs[cc * 16 + tid].i);
        if (better(qq.v, qq.i, bb.v, bb.i)) bb = qq;
      }
      const int idx = (bb.i == INT_MAX) ? 0 : bb.i;  // nothing finite: index 0, as a plain scan gives
      if (p.ids) p.ids[tid] = idx + p.row_offset;
      if (p.pairs_out)
        static_cast<Pair*>(p.pairs_out)[tid] = Pair{bb.v, (bb.i == INT_MAX) ? INT_MAX : bb.i + p.row_offset};
    }
  }
}

__global__ void k_pairs_reduce(int32_t* ids, const Pair* pairs, int nranks, int M) {
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  Pair b{-FLT_MAX, INT_MAX};
  for (int r = 0; r < nranks; ++r) {
    const Pair q = pairs[r * M + m];
    if (better(q.v, q.i, b.v, b.i)) b = q;
  }
  ids[m] = (b.i == INT_MAX) ? 0 : b.i;
}

// ------------------------------------------------------------------ host side
}  // namespace
unsigned long long* g_dbg = nullptr;
namespace {
struct Config {
  int depth;         // weight ring stages (17 KB each)
  int ctas;          // CTAs per SM
  int chunk_groups;  // k groups per activation chunk
  int pdl;
};

const Config& config() {
  static Config c = [] {
    Config k{3, 2, 4, 1};
    if (const char* e = getenv("W4A16_DEPTH")) k.depth = atoi(e);
    if (const char* e = getenv("W4A16_CTAS")) k.ctas = atoi(e) >= 2 ? 2 : 1;
    if (kMinCtas == 1) k.ctas = 1;
    if (const char* e = getenv("W4A16_CHUNK")) k.chunk_groups = atoi(e);
    if (const char* e = getenv("W4A16_PDL")) k.pdl = atoi(e) != 0;
    if (k.depth != 2 && k.depth != 3 && k.depth != 4 && k.depth != 6) k.depth = 3;
    if (k.chunk_groups < 2) k.chunk_groups = 2;
    if (k.chunk_groups > kMaxChunkGroups) k.chunk_groups = kMaxChunkGroups;
    k.chunk_groups &= ~1;
    return k;
  }();
  return c;
}

constexpr int kMaxCtasPerSm = 2;

template <int MC, int D>
int launch_cfg(SkinnyParams& p, int grid, cudaStream_t st) {
  const int smem = skinny_fixed_smem<D>() + kXBufs * p.chunk_groups * kXGroupBytes;
  static int attr_set[64] = {};
  int dev = 0;
  W4_CUDA(cudaGetDevice(&dev));
  if (attr_set[dev & 63] < smem) {
    W4_CUDA(cudaFuncSetAttribute(k_skinny<MC, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[dev & 63] = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = config().pdl ? 1 : 0;
  W4_CUDA(cudaLaunchKernelEx(&cfg, k_skinny<MC, D>, p));
  return W4A16_OK;
}

template <int MC>
int launch_depth(SkinnyParams& p, int grid, cudaStream_t st) {
  switch (config().depth) {
    case 2: return launch_cfg<MC, 2>(p, grid, st);
    case 4: return launch_cfg<MC, 4>(p, grid, st);
    case 6: return launch_cfg<MC, 6>(p, grid, st);
    default: return launch_cfg<MC, 3>(p, grid, st);
  }
}

int tile_rows() { return kTileRows; }

int grid_for_shape(int out_f, int G, int sms) {
  const int tiles = (out_f + tile_rows() - 1) / tile_rows();
  const long long U = static_cast<long long>(tiles) * G;
  const long long want = static_cast<long long>(sms) * config().ctas;
  return static_cast<int>(U < want ? U : want);
}

int launch_skinny(SkinnyParams& p, const w4a16_weights_t* w, const uint16_t* x, int M, w4a16_scratch_t* s,
                  cudaStream_t st) {
  if (int rc = check_weights(w)) return rc;
  W4_REQUIRE(x != nullptr && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "x null or not 16-byte aligned");
  W4_REQUIRE(M >= 1 && M <= 16, "M = %d outside [1,16]", M);
  W4_REQUIRE(s != nullptr && s->xf && s->xgsum && s->partial, "scratch not allocated");
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  const int TR = tile_rows();
  p.stream = reinterpret_cast<const uint8_t*>(w->qweight);
  p.x = x;
  p.M = M;
  p.N = w->out_f;
  p.K = w->in_f;
  p.G = w->num_groups;
  p.tiles = (w->out_f + TR - 1) / TR;
  p.chunk_groups = config().chunk_groups;
  p.partial = s->partial;
  p.counters = reinterpret_cast<unsigned*>(s->xgsum);
  p.cta_pairs = s->xf;
  p.status = di->status;
  if (const char* e = getenv("W4A16_DEBUG_SKIP")) p.debug_skip = atoi(e);
  if (getenv("W4A16_DEBUG_TIME")) {
    static unsigned long long* dbg = nullptr;
    if (!dbg) cudaMalloc(&dbg, 4096 * 8 * 8);
    p.dbg = dbg;
    g_dbg = dbg;
  }
  const int grid = grid_for_shape(w->out_f, w->num_groups, di->sms);
  if (int rc = w4a16_scratch_check(s, w->out_f, M)) return rc;
  if (M == 1) return launch_depth<1>(p, grid, st);
  if (M == 2) return launch_depth<2>(p, grid, st);
  if (M <= 4) return launch_depth<4>(p, grid, st);
  if (M <= 8) return launch_depth<8>(p, grid, st);
  return launch_depth<16>(p, grid, st);
}

}  // namespace
}  // namespace w4a16

using namespace w4a16;

extern "C" {

int w4a16_scratch_alloc(w4a16_scratch_t* s, int max_in, int max_out, int min_group, int max_m) {
  W4_REQUIRE(s != nullptr, "scratch_alloc: null struct");
  W4_REQUIRE(max_in > 0 && max_out > 0 && min_group > 0 && max_m >= 1, "scratch_alloc: bad sizes");
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  memset(s, 0, sizeof *s);
  s->max_in = max_in;
  s->max_out = max_out;
  s->max_m = max_m;
  s->max_groups = max_in / min_group;
  s->max_splits = di->sms * kMaxCtasPerSm;  // CTAs of the persistent grid
  // two partial tiles per CTA (head and tail of its unit range), widest tile, 16 tokens
  s->partial_elems = static_cast<size_t>(s->max_splits) * 2 * kTileRows * kTokens;
  const size_t counters = ((static_cast<size_t>(max_out) / kTileRows + 2) * kRowWarps + 8) * sizeof(unsigned);
  const size_t pairs = static_cast<size_t>(s->max_splits) * 16 * sizeof(Pair);
  void *xf = nullptr, *cn = nullptr, *pa = nullptr;
  cudaError_t e = cudaMalloc(&xf, pairs);
  if (e == cudaSuccess) e = cudaMalloc(&cn, counters);
  if (e == cudaSuccess) e = cudaMalloc(&pa, s->partial_elems * sizeof(float));
  if (e == cudaSuccess) e = cudaMemset(cn, 0, counters);
  if (e != cudaSuccess) {
    cudaFree(xf);
    cudaFree(cn);
    cudaFree(pa);
    memset(s, 0, sizeof *s);
    return fail(W4A16_ECUDA, "scratch_alloc: %s", cudaGetErrorString(e));
  }
  s->xf = static_cast<float*>(xf);
  s->xgsum = static_cast<float*>(cn);
  s->partial = static_cast<float*>(pa);
  return W4A16_OK;
}

int w4a16_scratch_free(w4a16_scratch_t* s) {
  W4_REQUIRE(s != nullptr, "scratch_free: null struct");
  cudaFree(s->xf);
  cudaFree(s->xgsum);
  cudaFree(s->partial);
  memset(s, 0, sizeof *s);
  return W4A16_OK;
}

int w4a16_scratch_check(const w4a16_scratch_t* s, int out_f, int M) {
  W4_REQUIRE(s != nullptr, "scratch_check: null struct");
  (void)M;
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  const int ctas = di->sms * kMaxCtasPerSm;
  const size_t need = static_cast<size_t>(ctas) * 2 * kTileRows * kTokens;
  if (need > s->partial_elems)
    return fail(W4A16_ESCRATCH, "scratch: partial buffer holds %zu floats, %zu needed", s->partial_elems, need);
  if (out_f > s->max_out)
    return fail(W4A16_ESCRATCH, "scratch: sized for out_f <= %d, got %d", s->max_out, out_f);
  if (ctas > s->max_splits)
    return fail(W4A16_ESCRATCH, "scratch: sized for %d CTAs, this device runs %d", s->max_splits, ctas);
  return W4A16_OK;
}

int w4a16_choose_splits(int out_f, int num_groups) {
  const DeviceInfo* di = device_info();
  if (!di || out_f <= 0 || num_groups <= 0) return 1;
  const int tiles = (out_f + tile_rows() - 1) / tile_rows();
  const int grid = grid_for_shape(out_f, num_groups, di->sms);
  // CTAs per row tile under the equal-range schedule, rounded up
  const int s = (grid + tiles - 1) / tiles;
  return s < 1 ? 1 : s;
}

int w4a16_gemv(void* y, int y_is_f32, const w4a16_weights_t* w, const uint16_t* x, w4a16_scratch_t* s,
               void* stream) {
  W4_REQUIRE(y != nullptr, "gemv: y is null");
  SkinnyParams p = {};
  p.y = y;
  p.y_f32 = y_is_f32 ? 1 : 0;
  p.ldy = w ? w->out_f : 0;
  return launch_skinny(p, w, x, 1, s, static_cast<cudaStream_t>(stream));
}

int w4a16_gemm_skinny(uint16_t* y, const w4a16_weights_t* w, const uint16_t* x, int M, w4a16_scratch_t* s,
                      void* stream) {
  W4_REQUIRE(y != nullptr, "gemm_skinny: y is null");
  SkinnyParams p = {};
  p.y = y;
  p.ldy = w ? w->out_f : 0;
  return launch_skinny(p, w, x, M, s, static_cast<cudaStream_t>(stream));
}

int w4a16_lm_head_argmax(int32_t* ids, uint16_t* logits, void* pairs, int row_offset, const w4a16_weights_t* w,
                         const uint16_t* x, int M, w4a16_scratch_t* s, void* stream) {
  W4_REQUIRE(ids != nullptr || pairs != nullptr, "lm_head_argmax: both ids and pairs are null");
  SkinnyParams p = {};
  p.y = logits;
  p.ldy = w ? w->out_f : 0;
  p.argmax = 1;
  p.ids = ids;
  p.pairs_out = pairs;
  p.row_offset = row_offset;
  return launch_skinny(p, w, x, M, s, static_cast<cudaStream_t>(stream));
}

int w4a16_argmax_pairs_reduce(int32_t* ids, const void* pairs, int nranks, int M, void* stream) {
  W4_REQUIRE(ids && pairs, "argmax_pairs_reduce: null pointer");
  W4_REQUIRE(nranks >= 1 && M >= 1 && M <= 16, "argmax_pairs_reduce: nranks %d, M %d", nranks, M);
  k_pairs_reduce<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ids, static_cast<const Pair*>(pairs), nranks, M);
  W4_CUDA(cudaGetLastError());
  return W4A16_OK;
}

int w4a16_shard_rows(int out_f, int nranks, int rank, int* row_begin, int* row_end) {
  W4_REQUIRE(row_begin && row_end, "shard_rows: null output");
  if (nranks < 1 || rank < 0 || rank >= nranks)
    return fail(W4A16_ECOMM, "shard_rows: rank %d of %d", rank, nranks);
  if (out_f <= 0 || out_f % (kRowGranule * nranks) != 0)
    return fail(W4A16_ECOMM, "shard_rows: out_f %d does not split into %d shards of whole 16-row blocks", out_f,
                nranks);
  const int per = out_f / nranks;
  *row_begin = rank * per;
  *row_end = (rank + 1) * per;
  return W4A16_OK;
}

int w4a16_gemm_skinny_sharded(uint16_t* const* y_peers, int nranks, int rank, int out_f_total, int row_begin,
                              const w4a16_weights_t* w_shard, const uint16_t* x, int M, w4a16_scratch_t* s,
                              void* stream) {
  W4_REQUIRE(y_peers != nullptr, "gemm_skinny_sharded: null peer table");
  if (nranks < 1 || nranks > 8 || rank < 0 || rank >= nranks)
    return fail(W4A16_ECOMM, "gemm_skinny_sharded: rank %d of %d (1..8 ranks)", rank, nranks);
  W4_REQUIRE(w_shard != nullptr, "gemm_skinny_sharded: null weights");
  if (row_begin < 0 || row_begin % kRowGranule != 0 || row_begin + w_shard->out_f > out_f_total)
    return fail(W4A16_ECOMM, "gemm_skinny_sharded: rows [%d,%d) outside [0,%d)", row_begin,
                row_begin + w_shard->out_f, out_f_total);
  for (int r = 0; r < nranks; ++r) W4_REQUIRE(y_peers[r] != nullptr, "gemm_skinny_sharded: null peer %d", r);
  SkinnyParams p = {};
  p.y = y_peers[rank];
  p.ldy = out_f_total;
  p.y_col0 = row_begin;
  int q = 0;
  for (int r = 0; r < nranks; ++r)
    if (r != rank) p.y_peers[q++] = y_peers[r];
  p.npeers = q;
  return launch_skinny(p, w_shard, x, M, s, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

extern "C" __attribute__((visibility("default"))) int w4a16_debug_read(unsigned long long* host, int n) {
  if (!w4a16::g_dbg) return -1;
  cudaDeviceSynchronize();
  return cudaMemcpy(host, w4a16::g_dbg, size_t(n) * 8, cudaMemcpyDeviceToHost);
}
