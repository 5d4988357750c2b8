// The decode-side W4A16 kernel for sm_100a: one persistent kernel serves the
// M=1 GEMV, the skinny GEMM of a speculative-verify block (M <= 16) and the
// lm_head GEMV with the argmax fused into its epilogue.
//
// Replaces k_prep + k_gemv + k_reduce, k_prep_m + k_gemm_small + k_reduce_bf16_m
// and k_gemm_mma of the reference (src/kernels/gemv_w4a16.cu:74-279,673-865) and,
// for lm_head, the separate argmax kernels (src/kernels/elementwise.cu:96-194).
//
// Shape of the computation (HBM-bound: every weight byte is read exactly once):
//   * persistent grid, two CTAs per SM. The (128-row tile, k group) units of the
//     matrix are dealt out as equal contiguous ranges, so every CTA streams the same
//     number of bytes whatever N and K are. A row tile whose K range is shared by
//     several CTAs is finished by the last warp to arrive for its rows, which adds the
//     partial tiles in a fixed order (bitwise reproducible, no float atomics). Shared
//     tiles are processed FIRST and each warp publishes its rows without any CTA-wide
//     barrier, so that reduction overlaps everybody's main loop.
//   * warp roles: a weight producer streams the CTA's contiguous share of the weight
//     stream through a ring of shared-memory stages with 1-D bulk async copies
//     (cp.async.bulk + mbarrier full/empty pairs); it does not wait for the previous
//     kernel (programmatic dependent launch), so one layer's weights start flowing
//     while the previous layer drains. An activation warp bulk-copies the token rows
//     and reduces them to per-(group, token) sums on the tensor core. Eight consumer
//     warps own 16 output rows each: nibbles become bf16 (128+q) pairs with one LOP3
//     per two weights and go from registers into mma.sync m16n8k16 (bf16 x bf16 ->
//     fp32); per group  y += s * (sum((128+q) x) - (128+zp) * sum(x)).
//   * measured on B200: the legacy mma.sync pipe sustains about one m16n8k16 per 32
//     cycles per scheduler, which caps this formulation near 4.5 TB/s (M <= 8). The
//     same data path with the weights as a TMEM-resident tcgen05 operand removes that
//     cap but is sync-latency bound today (2.2 TB/s); it shares the weight stream
//     layout with the prefill kernel, so it can replace this loop once it is faster.
#include <cfloat>
#include <climits>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace w4a16 {
namespace {

constexpr int CW = 8;                                 // consumer warps per CTA: 16 rows of the 128-row tile each
constexpr int kWarps = CW + 2;                        // + weight producer warp + activation warp
constexpr int kItemGroups = 2;                        // k groups per weight ring stage
constexpr int kStageBytes = kItemGroups * kTileGroupBytes;  // 17152: two (tile, group) blocks
static_assert(kStageBytes % 128 == 0, "ring stages must stay 128-byte aligned");
constexpr int kXBufs = 3;                             // activation chunk buffers
constexpr int kFirstChunk = 2;                        // groups in a CTA's first activation chunk (short start-up)
constexpr int kMaxChunkGroups = 32;                   // bound on groups per activation chunk
constexpr uint32_t kSpinLimit = 1u << 20;             // polls before a wait gives up
constexpr uint32_t kMagic = 0x43004300u;              // bf16 pair (128.0, 128.0)
constexpr uint32_t kNibMask = 0x000F000Fu;
constexpr uint32_t kOnes = 0x3F803F80u;               // bf16 pair (1.0, 1.0)
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
  int xrow_bytes;    // bytes between token rows inside an activation buffer
  int xbuf_bytes;    // bytes of one activation buffer
  float* partial;
  unsigned* counters;  // [tiles * 8 + 1], zero between launches
  int argmax;
  int32_t* ids;
  void* pairs_out;  // M x {float,int}
  int row_offset;
  void* cta_pairs;  // [grid][16] x {float,int}
  int* status;
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
// Every role (weight producer, activation warp, consumers) runs the same iterator.
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
//   [weight ring D stages][x buffers kXBufs][x sums kXBufs x 32 groups x 16][32 B zeros][mbarriers][flag]
constexpr int kXsumFloats = kMaxChunkGroups * 16;
template <int D>
__host__ __device__ constexpr int skinny_fixed_smem() {
  return D * kStageBytes + kXBufs * kXsumFloats * 4 + 32 + (2 * D + 3 * kXBufs) * 8 + 16;
}

template <int NT, int D>
__global__ void __launch_bounds__(kWarps * 32, 2) k_skinny(const SkinnyParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int SLOT = CW * 16 * 8 * NT;  // floats per partial tile
  constexpr int NCT = CW * 32;            // consumer threads

  uint8_t* ring = smem;
  uint8_t* xbuf = ring + D * kStageBytes;
  float* xsum = reinterpret_cast<float*>(xbuf + kXBufs * p.xbuf_bytes);
  uint8_t* zeros = reinterpret_cast<uint8_t*>(xsum + kXBufs * kXsumFloats);
  uint64_t* bars = reinterpret_cast<uint64_t*>(zeros + 32);
  int* sflag = reinterpret_cast<int*>(bars + 2 * D + 3 * kXBufs);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, M = p.M;
  const int U = p.tiles * G;
  const int u0 = static_cast<int>(static_cast<long long>(U) * blockIdx.x / gridDim.x);
  const int u1 = static_cast<int>(static_cast<long long>(U) * (blockIdx.x + 1) / gridDim.x);

  const uint32_t ring_a = smem_u32(ring);
  const uint32_t xbuf_a = smem_u32(xbuf);
  const uint32_t wfull_a = smem_u32(bars);        // [D]  weights landed
  const uint32_t wempty_a = wfull_a + D * 8;      // [D]  stage free again (8 consumer warps)
  const uint32_t xfull_a = wempty_a + D * 8;      // [kXBufs] activation chunk landed
  const uint32_t xsfull_a = xfull_a + kXBufs * 8; // [kXBufs] its per-group sums are ready
  const uint32_t xempty_a = xsfull_a + kXBufs * 8;// [kXBufs] buffer free again (8 consumers + activation warp)

  if (tid < 8) reinterpret_cast<uint32_t*>(zeros)[tid] = 0u;
  if (tid == 0) {
    for (int i = 0; i < D; ++i) {
      mbar_init(wfull_a + i * 8, 1);
      mbar_init(wempty_a + i * 8, CW);
    }
    for (int i = 0; i < kXBufs; ++i) {
      mbar_init(xfull_a + i * 8, 1);
      mbar_init(xsfull_a + i * 8, 1);
      mbar_init(xempty_a + i * 8, CW + 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  // B-fragment addressing of a lane: token row 8 nt + lane/4, k offset 16 (lane%4) within a
  // 64-k step. Lanes whose token row does not exist read a block of zeros (all strides 0).
  const int grow = lane >> 2, t = lane & 3;
  uint32_t xlane[NT], xstep[NT], xbufoff[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int mm = nt * 8 + grow;
    const bool valid = mm < M;
    xlane[nt] = valid ? xbuf_a + mm * p.xrow_bytes + t * 32 : smem_u32(zeros);
    xstep[nt] = valid ? 128 : 0;
    xbufoff[nt] = valid ? p.xbuf_bytes : 0;
  }

  // ================================================================ weight producer
  // One thread streams this CTA's share of the weight stream, one stage (two k groups of all
  // eight 16-row blocks, 17 KB, contiguous in memory) per bulk copy. It does not wait for the
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
                   p.stream + (static_cast<size_t>(c.tile) * G + c.g + gi) * kTileGroupBytes,
                   ng * kTileGroupBytes, wfull_a + st * 8);
          if (++st == D) {
            st = 0;
            ph ^= 1;
          }
        }
      }
    }
    return;
  }

  // ================================================================ activation warp
  // Waits for the previous kernel (it produced x), then per chunk: bulk-copies the token rows,
  // and turns them into per-(group, token) sums with the tensor core (ones(16x16) * X).
  if (warp == CW + 1) {
    pdl_wait();
    WorkIter it;
    it.init(u0, u1, G, p.chunk_groups);
    Chunk c;
    int xb = 0;
    uint32_t fph = 0, eph = 1;
    while (it.next(c)) {
      if (!mbar_wait_bounded_relaxed(xempty_a + xb * 8, eph, kSpinLimit)) {
        atomicExch(p.status, W4A16_ETIMEOUT);
        break;
      }
      if (lane == 0) {
        mbar_expect_tx(xfull_a + xb * 8, M * c.n * 256);
        for (int m = 0; m < M; ++m)
          bulk_g2s(xbuf_a + xb * p.xbuf_bytes + m * p.xrow_bytes,
                   p.x + static_cast<size_t>(m) * p.K + c.g * kGroup, c.n * 256, xfull_a + xb * 8);
      }
      if (!mbar_wait_bounded(xfull_a + xb * 8, fph, kSpinLimit)) {
        atomicExch(p.status, W4A16_ETIMEOUT);
        break;
      }
      for (int gl = 0; gl < c.n; ++gl) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float ax[4][4];
          const uint8_t* xa = smem + (xlane[nt] - ring_a) + xb * xbufoff[nt] + gl * 2 * xstep[nt];
          const uint4 b0 = *reinterpret_cast<const uint4*>(xa);
          const uint4 b1 = *reinterpret_cast<const uint4*>(xa + 16);
          const uint4 b2 = *reinterpret_cast<const uint4*>(xa + xstep[nt]);
          const uint4 b3 = *reinterpret_cast<const uint4*>(xa + xstep[nt] + 16);
          mma_bf16_16816_zero(ax[0], kOnes, kOnes, kOnes, kOnes, b0.x, b0.y);
          mma_bf16_16816_zero(ax[1], kOnes, kOnes, kOnes, kOnes, b1.x, b1.y);
          mma_bf16_16816_zero(ax[2], kOnes, kOnes, kOnes, kOnes, b2.x, b2.y);
          mma_bf16_16816_zero(ax[3], kOnes, kOnes, kOnes, kOnes, b3.x, b3.y);
          mma_bf16_16816(ax[0], kOnes, kOnes, kOnes, kOnes, b0.z, b0.w);
          mma_bf16_16816(ax[1], kOnes, kOnes, kOnes, kOnes, b1.z, b1.w);
          mma_bf16_16816(ax[2], kOnes, kOnes, kOnes, kOnes, b2.z, b2.w);
          mma_bf16_16816(ax[3], kOnes, kOnes, kOnes, kOnes, b3.z, b3.w);
          if (grow == 0) {
            float* xs = xsum + xb * kXsumFloats + gl * 16 + nt * 8 + 2 * t;
            xs[0] = (ax[0][0] + ax[1][0]) + (ax[2][0] + ax[3][0]);
            xs[1] = (ax[0][1] + ax[1][1]) + (ax[2][1] + ax[3][1]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(xsfull_a + xb * 8);  // sums published
        mbar_arrive(xempty_a + xb * 8);  // this warp no longer reads the chunk
      }
      if (++xb == kXBufs) {
        xb = 0;
        fph ^= 1;
        eph ^= 1;
      }
    }
    return;
  }

  // ================================================================ consumer warps
  // Byte offsets of this lane's 8-byte weight pieces inside a (tile, group) block: chunk t/2 of
  // the step, the slot of its row (rotated by four slots in odd chunks, which keeps the 8-byte
  // loads of a half-warp on distinct banks), half t%2 of the slot.
  const int wrow = warp * 16 + grow;
  const int woff_lo = (t >> 1) * kChunkBytes + weight_slot(wrow, t >> 1) * 16 + (t & 1) * 8;
  const int woff_hi = (t >> 1) * kChunkBytes + weight_slot(wrow + 8, t >> 1) * 16 + (t & 1) * 8;

  float fin[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) fin[nt][0] = fin[nt][1] = fin[nt][2] = fin[nt][3] = 0.f;

  float best_v[NT][2];
  int best_i[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      best_v[nt][c] = -FLT_MAX;
      best_i[nt][c] = INT_MAX;
    }

  // Final values of one row tile are in registers: write them out / fold into the argmax.
  auto finalize = [&](int tile, const float (&v)[NT][4]) {
    const int rb = tile * CW + warp;
    if (rb * 16 >= p.N) return;  // zero-padded rows of the last tile
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = nt * 8 + 2 * t + (j & 1);
        const int r = rb * 16 + grow + 8 * (j >> 1);
        if (m >= M) continue;
        const uint16_t hb = float_to_bf16_bits(v[nt][j]);
        if (p.y) {
          const size_t o = static_cast<size_t>(m) * p.ldy + p.y_col0 + r;
          if (p.y_f32) static_cast<float*>(p.y)[o] = v[nt][j];
          else static_cast<uint16_t*>(p.y)[o] = hb;
          for (int q = 0; q < p.npeers; ++q) p.y_peers[q][o] = hb;
        }
        if (p.argmax) {
          const float lv = bf16_bits_to_float(hb);
          if (better(lv, r, best_v[nt][j & 1], best_i[nt][j & 1])) {
            best_v[nt][j & 1] = lv;
            best_i[nt][j & 1] = r;
          }
        }
      }
  };

  // The 8 MMAs per token tile of one 128-k group of this warp's 16 rows, on bf16 (128+q) pairs.
  // `gb` = the (tile, group) block in the ring. Step s covers k chunks 2s and 2s+1; this lane's 16 k
  // of the step are one 8-byte half of the 16-byte slot of (row, chunk) for its low and high row.
  auto group_mma = [&](const uint8_t* gb, const uint8_t* const (&xp)[NT], float (&acc)[NT][2][4]) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const uint2 qlo = *reinterpret_cast<const uint2*>(gb + s * (2 * kChunkBytes) + woff_lo);
      const uint2 qhi = *reinterpret_cast<const uint2*>(gb + s * (2 * kChunkBytes) + woff_hi);
      const uint4 wq = make_uint4(qlo.x, qlo.y, qhi.x, qhi.y);
      uint32_t a[4][4];  // [mma][register]: rows (lo, hi, lo, hi) x k pairs
      a[0][0] = (wq.x & kNibMask) | kMagic;
      a[0][1] = (wq.z & kNibMask) | kMagic;
      a[0][2] = ((wq.x >> 4) & kNibMask) | kMagic;
      a[0][3] = ((wq.z >> 4) & kNibMask) | kMagic;
      a[1][0] = ((wq.x >> 8) & kNibMask) | kMagic;
      a[1][1] = ((wq.z >> 8) & kNibMask) | kMagic;
      a[1][2] = ((wq.x >> 12) & kNibMask) | kMagic;
      a[1][3] = ((wq.z >> 12) & kNibMask) | kMagic;
      a[2][0] = (wq.y & kNibMask) | kMagic;
      a[2][1] = (wq.w & kNibMask) | kMagic;
      a[2][2] = ((wq.y >> 4) & kNibMask) | kMagic;
      a[2][3] = ((wq.w >> 4) & kNibMask) | kMagic;
      a[3][0] = ((wq.y >> 8) & kNibMask) | kMagic;
      a[3][1] = ((wq.w >> 8) & kNibMask) | kMagic;
      a[3][2] = ((wq.y >> 12) & kNibMask) | kMagic;
      a[3][3] = ((wq.w >> 12) & kNibMask) | kMagic;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 bl = *reinterpret_cast<const uint4*>(xp[nt] + s * xstep[nt]);
        const uint4 bh = *reinterpret_cast<const uint4*>(xp[nt] + s * xstep[nt] + 16);
        if (s == 0) {
          mma_bf16_16816_zero(acc[nt][0], a[0][0], a[0][1], a[0][2], a[0][3], bl.x, bl.y);
          mma_bf16_16816_zero(acc[nt][1], a[1][0], a[1][1], a[1][2], a[1][3], bl.z, bl.w);
        } else {
          mma_bf16_16816(acc[nt][0], a[0][0], a[0][1], a[0][2], a[0][3], bl.x, bl.y);
          mma_bf16_16816(acc[nt][1], a[1][0], a[1][1], a[1][2], a[1][3], bl.z, bl.w);
        }
        mma_bf16_16816(acc[nt][0], a[2][0], a[2][1], a[2][2], a[2][3], bh.x, bh.y);
        mma_bf16_16816(acc[nt][1], a[3][0], a[3][1], a[3][2], a[3][3], bh.z, bh.w);
      }
    }
  };
  // y += s * (acc - (128 + zp) * sum(x)) for the lane's two rows
  auto group_fix = [&](const uint8_t* gb, const float* xs, const float (&acc)[NT][2][4]) {
    const uint16_t* scp = reinterpret_cast<const uint16_t*>(gb + kTgScaleOff) + warp * 16 + grow;
    const uint8_t* zpp = gb + kTgZpOff + warp * 16 + grow;
    const float s_lo = bf16_bits_to_float(scp[0]), s_hi = bf16_bits_to_float(scp[8]);
    const float z_lo = __uint_as_float(__byte_perm(zpp[0], 0x43000000u, 0x7044));  // 128 + zp, low row
    const float z_hi = __uint_as_float(__byte_perm(zpp[8], 0x43000000u, 0x7044));  // high row
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float2 x2 = *reinterpret_cast<const float2*>(xs + nt * 8 + 2 * t);
      fin[nt][0] = fmaf(s_lo, fmaf(-z_lo, x2.x, acc[nt][0][0] + acc[nt][1][0]), fin[nt][0]);
      fin[nt][1] = fmaf(s_lo, fmaf(-z_lo, x2.y, acc[nt][0][1] + acc[nt][1][1]), fin[nt][1]);
      fin[nt][2] = fmaf(s_hi, fmaf(-z_hi, x2.x, acc[nt][0][2] + acc[nt][1][2]), fin[nt][2]);
      fin[nt][3] = fmaf(s_hi, fmaf(-z_hi, x2.y, acc[nt][0][3] + acc[nt][1][3]), fin[nt][3]);
    }
  };

  // (tile, first/last contributing CTA, arrival ticket) of up to two split tiles, in lane 0
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
  int wst = 0, xb = 0;
  uint32_t wph = 0, xph = 0;
  bool dead = false;

  while (it.next(c)) {
    // ---- one activation chunk: groups [c.g, c.g + c.n) of row tile c.tile ----
    if (!dead && !mbar_wait_bounded(xfull_a + xb * 8, xph, kSpinLimit)) {
      dead = true;
      atomicExch(p.status, W4A16_ETIMEOUT);
    }
    const uint8_t* xchunk[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xchunk[nt] = smem + (xlane[nt] - ring_a) + xb * xbufoff[nt];
    const float* xs = xsum + xb * kXsumFloats;
    bool sums_ready = false;

    for (int gi = 0; gi < c.n; gi += kItemGroups) {
      if (!dead && !mbar_wait_bounded(wfull_a + wst * 8, wph, kSpinLimit)) {
        dead = true;
        atomicExch(p.status, W4A16_ETIMEOUT);
      }
      const uint8_t* up = ring + wst * kStageBytes;
      {
        float acc0[NT][2][4], acc1[NT][2][4];
        const uint8_t* xp[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) xp[nt] = xchunk[nt] + gi * 2 * xstep[nt];
        const bool two = gi + 1 < c.n;
        group_mma(up, xp, acc0);
        if (two) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) xp[nt] += 2 * xstep[nt];
          group_mma(up + kTileGroupBytes, xp, acc1);
        }
        if (!sums_ready) {
          if (!dead && !mbar_wait_bounded(xsfull_a + xb * 8, xph, kSpinLimit)) {
            dead = true;
            atomicExch(p.status, W4A16_ETIMEOUT);
          }
          sums_ready = true;
        }
        group_fix(up, xs + gi * 16, acc0);
        if (two) group_fix(up + kTileGroupBytes, xs + (gi + 1) * 16, acc1);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(wempty_a + wst * 8);  // this warp is done with the stage
      if (++wst == D) {
        wst = 0;
        wph ^= 1;
      }
    }
    if (lane == 0) mbar_arrive(xempty_a + xb * 8);  // (the __syncwarp above ordered every lane's reads)
    if (++xb == kXBufs) {
      xb = 0;
      xph ^= 1;
    }

    if (c.seg_last) {
      // ---- end of this CTA's segment of row tile c.tile: groups [seg_g0, seg_g1) ----
      before_global_write();
      const int tile = c.tile;
      if (c.seg_g0 == 0 && c.seg_g1 == G) {
        finalize(tile, fin);
      } else {
        // split tile: this warp publishes its 16 rows and moves on; no CTA-wide barrier
        const long long X0 = static_cast<long long>(tile) * G;
        const int c_first = static_cast<int>(((X0 + 1) * gridDim.x - 1) / U);
        const int c_last = static_cast<int>(((X0 + G) * gridDim.x - 1) / U);
        const int which = (u0 / G == tile) ? 0 : 1;
        float* slot = p.partial + (static_cast<size_t>(blockIdx.x) * 2 + which) * SLOT;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            slot[(warp * 16 + grow + 8 * (j >> 1)) * 8 * NT + nt * 8 + 2 * t + (j & 1)] = fin[nt][j];
        __syncwarp();
        if (lane == 0) {
          __threadfence();  // release: this warp's partial rows (ordered by the __syncwarp) before the ticket
          const unsigned old = atomicAdd(p.counters + tile * CW + warp, 1u);
          if (sp_n == 0) {
            sp_tile0 = tile; sp_cf0 = c_first; sp_cl0 = c_last; sp_old0 = old;
          } else {
            sp_tile1 = tile; sp_cf1 = c_first; sp_cl1 = c_last; sp_old1 = old;
          }
          ++sp_n;
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) fin[nt][0] = fin[nt][1] = fin[nt][2] = fin[nt][3] = 0.f;
    }
  }

  // ---- split tiles: the warp that drew the last ticket for its rows adds the pieces up ----
  {
    const int n = __shfl_sync(0xffffffffu, sp_n, 0);
    for (int i = 0; i < n; ++i) {
      const int tile = __shfl_sync(0xffffffffu, i ? sp_tile1 : sp_tile0, 0);
      const int c_first = __shfl_sync(0xffffffffu, i ? sp_cf1 : sp_cf0, 0);
      const int c_last = __shfl_sync(0xffffffffu, i ? sp_cl1 : sp_cl0, 0);
      const unsigned old = __shfl_sync(0xffffffffu, i ? sp_old1 : sp_old0, 0);
      if (old != static_cast<unsigned>(c_last - c_first)) continue;  // another warp finishes these rows
      if (lane == 0) {
        p.counters[tile * CW + warp] = 0;  // every contributor has arrived: leave it clean
        __threadfence();                   // acquire side for the reads below
      }
      __syncwarp();
      float v[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) v[nt][0] = v[nt][1] = v[nt][2] = v[nt][3] = 0.f;
      for (int cc = c_first; cc <= c_last; ++cc) {  // fixed order: bitwise reproducible
        const int cu0 = static_cast<int>(static_cast<long long>(U) * cc / gridDim.x);
        const int wc = (cu0 / G == tile) ? 0 : 1;
        const float* sl = p.partial + (static_cast<size_t>(cc) * 2 + wc) * SLOT;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[nt][j] += __ldcg(sl + (warp * 16 + grow + 8 * (j >> 1)) * 8 * NT + nt * 8 + 2 * t + (j & 1));
      }
      finalize(tile, v);
    }
  }

  if (dead) {  // let whatever is still in flight land before the CTA exits
    for (int s = 0; s < D; ++s) mbar_wait_bounded(wfull_a + s * 8, 0, 1u << 16);
  }

  if (p.argmax) {
    before_global_write();
    // ---- fused argmax: thread -> warp -> CTA -> grid, larger value then lower index ----
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int cc = 0; cc < 2; ++cc)
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best_v[nt][cc], off);
          const int oi = __shfl_xor_sync(0xffffffffu, best_i[nt][cc], off);
          if (better(ov, oi, best_v[nt][cc], best_i[nt][cc])) {
            best_v[nt][cc] = ov;
            best_i[nt][cc] = oi;
          }
        }
    named_bar_sync(kConsumerBar, NCT);
    // per-warp candidates go through the (now idle) weight ring: every stage was consumed
    Pair* cand = reinterpret_cast<Pair*>(ring);  // [CW][16]
    if (grow == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) cand[warp * 16 + nt * 8 + 2 * t + cc] = Pair{best_v[nt][cc], best_i[nt][cc]};
    }
    named_bar_sync(kConsumerBar, NCT);
    Pair* cta_pairs = static_cast<Pair*>(p.cta_pairs);
    if (tid < M) {
      Pair b{-FLT_MAX, INT_MAX};
      for (int w = 0; w < CW; ++w) {
        const Pair q = cand[w * 16 + tid];
        if (better(q.v, q.i, b.v, b.i)) b = q;
      }
      cta_pairs[blockIdx.x * 16 + tid] = b;
    }
    named_bar_sync(kConsumerBar, NCT);
    if (tid == 0) {
      __threadfence();
      const unsigned old = atomicAdd(p.counters + p.tiles * CW, 1u);
      const int last = (old == gridDim.x - 1);
      if (last) {
        p.counters[p.tiles * CW] = 0;
        __threadfence();
      }
      *sflag = last;
    }
    named_bar_sync(kConsumerBar, NCT);
    if (*sflag && tid < M) {
      Pair b{-FLT_MAX, INT_MAX};
      for (unsigned cc = 0; cc < gridDim.x; ++cc) {
        Pair q;
        q.v = __ldcg(&cta_pairs[cc * 16 + tid].v);
        q.i = __ldcg(&cta_pairs[cc * 16 + tid].i);
        if (better(q.v, q.i, b.v, b.i)) b = q;
      }
      const int idx = (b.i == INT_MAX) ? 0 : b.i;  // nothing finite: index 0, as a plain scan gives
      if (p.ids) p.ids[tid] = idx + p.row_offset;
      if (p.pairs_out)
        static_cast<Pair*>(p.pairs_out)[tid] = Pair{b.v, (b.i == INT_MAX) ? INT_MAX : b.i + p.row_offset};
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
struct Config {
  int depth;  // weight ring stages (17 KB each)
  int ctas;   // CTAs per SM
  int xbuf;   // bytes of one activation chunk buffer
  int pdl;
};

const Config& config() {
  static Config c = [] {
    Config k{4, 2, 8192, 1};
    if (const char* e = getenv("W4A16_DEPTH")) k.depth = atoi(e);
    if (const char* e = getenv("W4A16_CTAS")) k.ctas = atoi(e) >= 2 ? 2 : 1;
    if (const char* e = getenv("W4A16_XBUF")) k.xbuf = atoi(e);
    if (const char* e = getenv("W4A16_PDL")) k.pdl = atoi(e) != 0;
    if (k.depth != 3 && k.depth != 4 && k.depth != 6) k.depth = 4;
    if (k.xbuf < 4096) k.xbuf = 4096;
    if (k.xbuf > 16384) k.xbuf = 16384;
    k.xbuf &= ~1023;
    return k;
  }();
  return c;
}

constexpr int kMaxCtasPerSm = 2;

template <int NT, int D>
int launch_cfg(SkinnyParams& p, int grid, cudaStream_t st) {
  const int smem = skinny_fixed_smem<D>() + kXBufs * p.xbuf_bytes;
  static int attr_set[64] = {};
  int dev = 0;
  W4_CUDA(cudaGetDevice(&dev));
  if (attr_set[dev & 63] < smem) {
    W4_CUDA(cudaFuncSetAttribute(k_skinny<NT, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
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
  W4_CUDA(cudaLaunchKernelEx(&cfg, k_skinny<NT, D>, p));
  return W4A16_OK;
}

template <int NT>
int launch_depth(SkinnyParams& p, int grid, cudaStream_t st) {
  switch (config().depth) {
    case 3: return launch_cfg<NT, 3>(p, grid, st);
    case 6: return launch_cfg<NT, 6>(p, grid, st);
    default: return launch_cfg<NT, 4>(p, grid, st);
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
  p.partial = s->partial;
  p.counters = reinterpret_cast<unsigned*>(s->xgsum);
  p.cta_pairs = s->xf;
  p.status = di->status;
  // groups per activation chunk: what one buffer holds (256 B per token per group), even.
  // Token rows sit 16 bytes past a multiple of 128 apart, which keeps the B-fragment loads of
  // neighbouring token rows on different banks.
  int cg = config().xbuf / (256 * M);
  if (cg > kMaxChunkGroups) cg = kMaxChunkGroups;
  cg &= ~1;
  if (cg < 2) cg = 2;
  p.chunk_groups = cg;
  p.xrow_bytes = cg * 256 + 16;
  p.xbuf_bytes = (M * p.xrow_bytes + 127) & ~127;
  const int grid = grid_for_shape(w->out_f, w->num_groups, di->sms);
  if (int rc = w4a16_scratch_check(s, w->out_f, M)) return rc;
  return M <= 8 ? launch_depth<1>(p, grid, st) : launch_depth<2>(p, grid, st);
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
  s->partial_elems = static_cast<size_t>(s->max_splits) * 2 * kTileRows * 16;
  const size_t counters = ((static_cast<size_t>(max_out) / kTileRows + 2) * CW + 8) * sizeof(unsigned);
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
  const size_t need = static_cast<size_t>(ctas) * 2 * kTileRows * 16;
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

// ---------------------------------------------------------------------------------------------
// GEMV without any scratch argument and without any allocation, for callers that cannot call
// cudaMalloc: code that runs after the serving process has handed every remaining byte of HBM
// to its KV cache, or on a path where the implicit device-wide synchronisation of an allocation
// is not acceptable. The split-tile partial sums and arrival counters live in this file-scope
// device array instead; every GPU that loads the library carries it (about 5.3 MB) until exit.
constexpr int kStaticMaxCtas = 320;     // 2 CTAs x 160 SMs
constexpr int kStaticMaxOut = 65536;    // widest layer the static scratch serves
constexpr size_t kStaticPartialBytes = static_cast<size_t>(kStaticMaxCtas) * 2 * kTileRows * 16 * sizeof(float);
constexpr size_t kStaticCounterBytes = ((kStaticMaxOut / kTileRows + 2) * 8 + 8) * sizeof(unsigned);
constexpr size_t kStaticPairBytes = static_cast<size_t>(kStaticMaxCtas) * 16 * 8;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticPartialBytes + kStaticCounterBytes + kStaticPairBytes];

int w4a16_gemv_static(void* y, int y_is_f32, const w4a16_weights_t* w, const uint16_t* x, void* stream) {
  W4_REQUIRE(y != nullptr, "gemv_static: y is null");
  W4_REQUIRE(w != nullptr, "gemv_static: null weights");
  W4_REQUIRE(w->out_f <= kStaticMaxOut, "gemv_static: out_f %d exceeds the static scratch limit of %d rows", w->out_f,
             kStaticMaxOut);
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  W4_REQUIRE(di->sms * kMaxCtasPerSm <= kStaticMaxCtas, "gemv_static: %d SMs exceed the static scratch limit of %d CTAs",
             di->sms, kStaticMaxCtas);
  // The array's name is only a host-side handle: the device address has to be asked for, once
  // per device and with that device current. The first call on a device does this (and clears the
  // counters), so it should come before any stream capture.
  static unsigned char* base[64] = {};
  unsigned char* b = base[di->device & 63];
  if (!b) {
    void* p0 = nullptr;
    W4_CUDA(cudaGetSymbolAddress(&p0, g_static_scratch));
    b = static_cast<unsigned char*>(p0);
    W4_CUDA(cudaMemsetAsync(b + kStaticPartialBytes, 0, kStaticCounterBytes, static_cast<cudaStream_t>(stream)));
    base[di->device & 63] = b;
  }
  w4a16_scratch_t s = {};
  s.partial = reinterpret_cast<float*>(b);
  s.xgsum = reinterpret_cast<float*>(b + kStaticPartialBytes);
  s.xf = reinterpret_cast<float*>(b + kStaticPartialBytes + kStaticCounterBytes);
  s.max_out = kStaticMaxOut;
  s.max_splits = kStaticMaxCtas;
  s.max_m = 1;
  s.partial_elems = kStaticPartialBytes / sizeof(float);
  SkinnyParams p = {};
  p.y = y;
  p.y_f32 = y_is_f32 ? 1 : 0;
  p.ldy = w->out_f;
  return launch_skinny(p, w, x, 1, &s, static_cast<cudaStream_t>(stream));
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
