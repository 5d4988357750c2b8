// The decode-side W4A16 kernel for sm_100a: one persistent kernel serves the
// M=1 GEMV, the skinny GEMM of a speculative-verify block (M <= 16) and the
// lm_head GEMV with the argmax fused into its epilogue.
//
// Replaces k_prep + k_gemv + k_reduce, k_prep_m + k_gemm_small + k_reduce_bf16_m
// and k_gemm_mma of the reference (src/kernels/gemv_w4a16.cu:74-279,673-865) and,
// for lm_head, the separate argmax kernels (src/kernels/elementwise.cu:96-194).
//
// Shape of the computation (HBM-bound: every packed weight byte is read once):
//   * grid = one CTA per SM; the (row tile, k group) units of the whole matrix are
//     dealt out as equal contiguous ranges, so every SM streams the same number of
//     bytes whatever N and K are. A row tile whose K range is shared by several
//     CTAs is finished by the last CTA to arrive, which adds the partial tiles in a
//     fixed order (bitwise reproducible, no float atomics).
//   * each warp owns 16 output rows and streams their packed int4 blocks, scales
//     and zero points through a private ring of shared-memory stages filled by 1-D
//     bulk async copies (cp.async.bulk + mbarrier); the ring is primed before the
//     kernel waits on its predecessor (programmatic dependent launch), so the
//     weight stream of one layer starts while the previous layer drains.
//   * activations are staged per 1024-k chunk with cp.async directly in MMA
//     fragment order; nibbles are turned into bf16 (128+q) pairs with one LOP3 per
//     two weights and fed from registers to mma.sync m16n8k16 (bf16 x bf16 -> fp32).
//     Per group:  y += s * (sum((128+q) x) - (128+zp) * sum(x)),  sum(x) coming from
//     one more MMA against a tile of ones.
#include <cfloat>
#include <climits>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace w4a16 {
namespace {

constexpr int kChunkGroups = 8;                       // k groups per activation chunk (1024 k)
constexpr int kChunkSteps = kChunkGroups * 2;         // 64-k steps per chunk
constexpr int kItemGroups = 2;                        // k groups per ring stage
constexpr int kItemQ = kItemGroups * 2 * kStepBytes;  // 2048 B of packed weights
constexpr int kItemS = kItemGroups * 32;              // 16 bf16 scales per group
constexpr int kItemZ = kItemGroups * 16;              // 16 u8 zero points per group
constexpr int kItemStride = 2176;                     // 2048 + 64 + 32, padded to 128
static_assert(kItemQ + kItemS + kItemZ <= kItemStride, "ring stage too small");
constexpr uint32_t kSpinLimit = 1u << 20;             // polls before a wait gives up
constexpr uint32_t kMagic = 0x43004300u;              // bf16 pair (128.0, 128.0)
constexpr uint32_t kNibMask = 0x000F000Fu;
constexpr uint32_t kOnes = 0x3F803F80u;               // bf16 pair (1.0, 1.0)

struct SkinnyParams {
  const uint4* qw;
  const uint16_t* sc;
  const uint8_t* zp;
  const uint16_t* x;  // [M][K] bf16
  void* y;            // bf16 or fp32 [M][ldy], may be null in argmax mode
  int y_f32;
  long long ldy;  // elements between rows of y
  int y_col0;     // first column of this launch's rows inside y
  int M, N, K, G, NRB, tiles;
  float* partial;
  unsigned* counters;  // [tiles + 1], zero between launches
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

template <int NT>
__host__ __device__ constexpr int xbuf_bytes() {
  return kChunkSteps * NT * 1024;
}

template <int NT, int WARPS, int D>
constexpr int skinny_smem_bytes() {
  return WARPS * D * kItemStride + 2 * xbuf_bytes<NT>() + 2 * kChunkGroups * 8 * NT * 4 + WARPS * D * 8 + 16;
}

template <int NT, int WARPS, int D>
__global__ void __launch_bounds__(WARPS * 32, 1) k_skinny(const SkinnyParams p) {
  static_assert(WARPS >= kChunkGroups, "one warp per group computes the activation sums");
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int XBUF = xbuf_bytes<NT>();
  constexpr int TILE_ROWS = WARPS * 16;
  constexpr int SLOT = TILE_ROWS * 8 * NT;  // floats per partial tile

  uint8_t* ring = smem;
  uint8_t* xbuf = ring + WARPS * D * kItemStride;
  float* xsum = reinterpret_cast<float*>(xbuf + 2 * XBUF);  // [2][8][8*NT]
  uint64_t* bars = reinterpret_cast<uint64_t*>(xsum + 2 * kChunkGroups * 8 * NT);
  int* sflag = reinterpret_cast<int*>(bars + WARPS * D);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grow = lane >> 2, t = lane & 3;
  const int G = p.G, KB = p.K / kStepK;
  const long long U = static_cast<long long>(p.tiles) * G;
  const long long u0 = U * blockIdx.x / gridDim.x;
  const long long u1 = U * (blockIdx.x + 1) / gridDim.x;

  const uint32_t ring_w = smem_u32(ring) + warp * D * kItemStride;
  const uint32_t bars_w = smem_u32(bars) + warp * D * 8;
  const uint32_t xbuf_a = smem_u32(xbuf);

  // ---- prologue: nothing here depends on the previous kernel's output ----
  for (int i = tid; i < 2 * XBUF / 16; i += WARPS * 32) reinterpret_cast<uint4*>(xbuf)[i] = make_uint4(0, 0, 0, 0);
  if (lane == 0) {
    for (int s = 0; s < D; ++s) mbar_init(bars_w + s * 8, 1);
    fence_mbar_init();
  }
  __syncthreads();

  // Producer cursor (meaningful in lane 0 only): next unit to fetch, next stage to fill.
  long long pu = u0;
  int pstage = 0;
  auto issue_next = [&]() {
    while (pu < u1) {
      const int tile = static_cast<int>(pu / G);
      const int g = static_cast<int>(pu - static_cast<long long>(tile) * G);
      int ng = kItemGroups;
      if (G - g < ng) ng = G - g;
      if (u1 - pu < ng) ng = static_cast<int>(u1 - pu);
      pu += ng;
      const int rb = tile * WARPS + warp;
      if (rb >= p.NRB) continue;  // rows past the end of the matrix: this warp has no item
      const uint32_t bar = bars_w + pstage * 8;
      const uint32_t dst = ring_w + pstage * kItemStride;
      mbar_expect_tx(bar, ng * (2 * kStepBytes + 32 + 16));
      bulk_g2s(dst, p.qw + (static_cast<size_t>(rb) * KB + g * 2) * 32, ng * 2 * kStepBytes, bar);
      bulk_g2s(dst + kItemQ, p.sc + (static_cast<size_t>(rb) * G + g) * 16, ng * 32, bar);
      bulk_g2s(dst + kItemQ + kItemS, p.zp + (static_cast<size_t>(rb) * G + g) * 16, ng * 16, bar);
      pstage = (pstage + 1 == D) ? 0 : pstage + 1;
      return;
    }
  };
  if (lane == 0)
    for (int s = 0; s < D; ++s) issue_next();

  pdl_launch_dependents();
  pdl_wait();  // activations (and the scratch this kernel shares) are now safe to touch

  // Stage the activation chunk that starts at unit `u` into buffer `buf`, in
  // fragment order: slot (step, nt, h, lane) holds x[8nt + lane/4][k0 + 64 step + 16 (lane%4) + 8h .. +8).
  auto stage_x = [&](long long u, int buf) {
    const int tile = static_cast<int>(u / G);
    const int g0 = static_cast<int>(u - static_cast<long long>(tile) * G);
    int ngc = kChunkGroups;
    if (G - g0 < ngc) ngc = G - g0;
    if (u1 - u < ngc) ngc = static_cast<int>(u1 - u);
    const int nslots = ngc * 2 * NT * 64;
    for (int i = tid; i < nslots; i += WARPS * 32) {
      const int l = i & 31, h = (i >> 5) & 1, nt = (i >> 6) % NT, step = i / (64 * NT);
      const int n = nt * 8 + (l >> 2);
      if (n < p.M)
        cp_async16(xbuf_a + buf * XBUF + ((step * NT + nt) * 2 + h) * 512 + l * 16,
                   p.x + static_cast<size_t>(n) * p.K + g0 * kGroup + step * kStepK + 16 * (l & 3) + 8 * h);
    }
    cp_async_commit();
  };

  float fin[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j) fin[nt][j] = 0.f;

  // running argmax candidates of this thread: [nt][column parity]
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
    const int rb = tile * WARPS + warp;
    if (rb >= p.NRB) return;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = nt * 8 + 2 * t + (j & 1);
        const int r = rb * 16 + grow + 8 * (j >> 1);
        if (m >= p.M) continue;
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

  int cb = 0, cstage = 0;
  uint32_t cphase = 0;
  bool dead = false;
  long long u = u0;
  int seg_begin = static_cast<int>(u0 % G);
  if (u < u1) stage_x(u, 0);

  while (u < u1) {
    const int tile = static_cast<int>(u / G);
    const int g0 = static_cast<int>(u - static_cast<long long>(tile) * G);
    int ngc = kChunkGroups;
    if (G - g0 < ngc) ngc = G - g0;
    if (u1 - u < ngc) ngc = static_cast<int>(u1 - u);

    cp_async_wait_all();
    __syncthreads();  // chunk `cb` is complete; everyone is done with the other buffer
    const long long un = u + ngc;
    if (un < u1) stage_x(un, cb ^ 1);

    // Activation sums per (group, token) through the tensor core: ones(16x16) * X.
    if (warp < ngc) {
      float ax[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) ax[nt][0] = ax[nt][1] = ax[nt][2] = ax[nt][3] = 0.f;
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t xa = xbuf_a + cb * XBUF + (((warp * 2 + s) * NT + nt) * 2) * 512 + lane * 16;
          const uint4 bl = lds128(xa), bh = lds128(xa + 512);
          mma_bf16_16816(ax[nt], kOnes, kOnes, kOnes, kOnes, bl.x, bl.y);
          mma_bf16_16816(ax[nt], kOnes, kOnes, kOnes, kOnes, bl.z, bl.w);
          mma_bf16_16816(ax[nt], kOnes, kOnes, kOnes, kOnes, bh.x, bh.y);
          mma_bf16_16816(ax[nt], kOnes, kOnes, kOnes, kOnes, bh.z, bh.w);
        }
      if (grow == 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float* xs = xsum + (cb * kChunkGroups + warp) * 8 * NT + nt * 8 + 2 * t;
          xs[0] = ax[nt][0];
          xs[1] = ax[nt][1];
        }
      }
    }
    __syncthreads();

    const int rb = tile * WARPS + warp;
    if (rb < p.NRB) {
      for (int gi = 0; gi < ngc; gi += kItemGroups) {
        const int ng = (ngc - gi < kItemGroups) ? ngc - gi : kItemGroups;
        if (!dead && !mbar_wait_bounded(bars_w + cstage * 8, cphase, kSpinLimit)) {
          dead = true;
          atomicExch(p.status, W4A16_ETIMEOUT);
        }
        const uint32_t base = ring_w + cstage * kItemStride;
        for (int gg = 0; gg < ng; ++gg) {
          const int gl = gi + gg;
          float acc[NT][2][4];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < 2; ++c) acc[nt][c][0] = acc[nt][c][1] = acc[nt][c][2] = acc[nt][c][3] = 0.f;
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint4 wq = lds128(base + (gg * 2 + s) * kStepBytes + lane * 16);
            uint32_t a[4][4];  // [mma j][register]
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
              const uint32_t xa = xbuf_a + cb * XBUF + (((gl * 2 + s) * NT + nt) * 2) * 512 + lane * 16;
              const uint4 bl = lds128(xa), bh = lds128(xa + 512);
              mma_bf16_16816(acc[nt][0], a[0][0], a[0][1], a[0][2], a[0][3], bl.x, bl.y);
              mma_bf16_16816(acc[nt][1], a[1][0], a[1][1], a[1][2], a[1][3], bl.z, bl.w);
              mma_bf16_16816(acc[nt][0], a[2][0], a[2][1], a[2][2], a[2][3], bh.x, bh.y);
              mma_bf16_16816(acc[nt][1], a[3][0], a[3][1], a[3][2], a[3][3], bh.z, bh.w);
            }
          }
          // group fix-up: y += s * (acc - (128 + zp) * sum(x))
          const uint8_t* itm = ring + (warp * D + cstage) * kItemStride;
          const uint16_t* isc = reinterpret_cast<const uint16_t*>(itm + kItemQ) + gg * 16;
          const uint8_t* izp = itm + kItemQ + kItemS + gg * 16;
          const float s_lo = bf16_bits_to_float(isc[grow]), s_hi = bf16_bits_to_float(isc[grow + 8]);
          const float z_lo = 128.f + static_cast<float>(izp[grow]);
          const float z_hi = 128.f + static_cast<float>(izp[grow + 8]);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const float2 xs =
                *reinterpret_cast<const float2*>(xsum + (cb * kChunkGroups + gl) * 8 * NT + nt * 8 + 2 * t);
            fin[nt][0] = fmaf(s_lo, fmaf(-z_lo, xs.x, acc[nt][0][0] + acc[nt][1][0]), fin[nt][0]);
            fin[nt][1] = fmaf(s_lo, fmaf(-z_lo, xs.y, acc[nt][0][1] + acc[nt][1][1]), fin[nt][1]);
            fin[nt][2] = fmaf(s_hi, fmaf(-z_hi, xs.x, acc[nt][0][2] + acc[nt][1][2]), fin[nt][2]);
            fin[nt][3] = fmaf(s_hi, fmaf(-z_hi, xs.y, acc[nt][0][3] + acc[nt][1][3]), fin[nt][3]);
          }
        }
        __syncwarp();
        if (lane == 0) {
          fence_proxy_async();  // our reads of this stage precede the async refill
          issue_next();
        }
        if (++cstage == D) {
          cstage = 0;
          cphase ^= 1;
        }
      }
    }

    u = un;
    cb ^= 1;
    const long long tile_end = static_cast<long long>(tile + 1) * G;
    if (u == u1 || u == tile_end) {
      // ---- end of this CTA's segment of row tile `tile`: groups [seg_begin, g_end) ----
      const int g_end = static_cast<int>(u - static_cast<long long>(tile) * G);
      if (seg_begin == 0 && g_end == G) {
        finalize(tile, fin);
      } else {
        const long long X0 = static_cast<long long>(tile) * G;
        const int c_first = static_cast<int>(((X0 + 1) * gridDim.x - 1) / U);
        const int c_last = static_cast<int>((tile_end * gridDim.x - 1) / U);
        const int which = (static_cast<int>(u0 / G) == tile) ? 0 : 1;
        float* slot = p.partial + (static_cast<size_t>(blockIdx.x) * 2 + which) * SLOT;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            slot[(warp * 16 + grow + 8 * (j >> 1)) * 8 * NT + nt * 8 + 2 * t + (j & 1)] = fin[nt][j];
        __threadfence();
        __syncthreads();
        if (tid == 0) {
          const unsigned old = atomicAdd(p.counters + tile, 1u);
          const int last = (old == static_cast<unsigned>(c_last - c_first));
          if (last) p.counters[tile] = 0;  // every contributor has arrived: leave it clean
          *sflag = last;
        }
        __syncthreads();
        if (*sflag) {
          __threadfence();
          float v[NT][4];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) v[nt][0] = v[nt][1] = v[nt][2] = v[nt][3] = 0.f;
          for (int c = c_first; c <= c_last; ++c) {  // fixed order: bitwise reproducible
            const int wc = (static_cast<int>((U * c / gridDim.x) / G) == tile) ? 0 : 1;
            const float* sl = p.partial + (static_cast<size_t>(c) * 2 + wc) * SLOT;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int j = 0; j < 4; ++j)
                v[nt][j] += __ldcg(sl + (warp * 16 + grow + 8 * (j >> 1)) * 8 * NT + nt * 8 + 2 * t + (j & 1));
          }
          finalize(tile, v);
        }
        __syncthreads();  // sflag may be rewritten by the next segment
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) fin[nt][0] = fin[nt][1] = fin[nt][2] = fin[nt][3] = 0.f;
      seg_begin = 0;
    }
  }

  if (dead) {  // drain whatever this warp still has in flight before the CTA exits
    for (int s = 0; s < D; ++s) mbar_wait_bounded(bars_w + s * 8, 0, 1u << 16);
  }

  if (p.argmax) {
    // ---- fused argmax: thread -> warp -> CTA -> grid, larger value then lower index ----
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best_v[nt][c], off);
          const int oi = __shfl_xor_sync(0xffffffffu, best_i[nt][c], off);
          if (better(ov, oi, best_v[nt][c], best_i[nt][c])) {
            best_v[nt][c] = ov;
            best_i[nt][c] = oi;
          }
        }
    __syncthreads();  // xbuf is free now: reuse it for the per-warp candidates
    Pair* cand = reinterpret_cast<Pair*>(xbuf);  // [WARPS][16]
    if (grow == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 2; ++c) cand[warp * 16 + nt * 8 + 2 * t + c] = Pair{best_v[nt][c], best_i[nt][c]};
    }
    __syncthreads();
    Pair* cta_pairs = static_cast<Pair*>(p.cta_pairs);
    if (tid < p.M) {
      Pair b{-FLT_MAX, INT_MAX};
      if (tid < 8 * NT)
        for (int w = 0; w < WARPS; ++w) {
          const Pair c = cand[w * 16 + tid];
          if (better(c.v, c.i, b.v, b.i)) b = c;
        }
      cta_pairs[blockIdx.x * 16 + tid] = b;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned old = atomicAdd(p.counters + p.tiles, 1u);
      const int last = (old == gridDim.x - 1);
      if (last) p.counters[p.tiles] = 0;
      *sflag = last;
    }
    __syncthreads();
    if (*sflag && tid < p.M) {
      __threadfence();
      Pair b{-FLT_MAX, INT_MAX};
      for (unsigned c = 0; c < gridDim.x; ++c) {
        Pair q;
        q.v = __ldcg(&cta_pairs[c * 16 + tid].v);
        q.i = __ldcg(&cta_pairs[c * 16 + tid].i);
        if (better(q.v, q.i, b.v, b.i)) b = q;
      }
      const int idx = (b.i == INT_MAX) ? 0 : b.i;  // nothing finite: index 0, as a plain scan gives
      if (p.ids) p.ids[tid] = idx + p.row_offset;
      if (p.pairs_out) static_cast<Pair*>(p.pairs_out)[tid] = Pair{b.v, (b.i == INT_MAX) ? INT_MAX : b.i + p.row_offset};
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
  int warps;
  int pdl;
  int ctas_per_sm_cap;  // grid = min(sms, units)
};

const Config& config() {
  static Config c = [] {
    Config k{8, 1, 1};
    if (const char* e = getenv("W4A16_WARPS")) k.warps = atoi(e) == 16 ? 16 : 8;
    if (const char* e = getenv("W4A16_PDL")) k.pdl = atoi(e) != 0;
    return k;
  }();
  return c;
}

constexpr int kMaxTileRows = 256;  // scratch is sized for the widest tile any configuration uses

template <int NT, int WARPS, int D>
int launch_cfg(const SkinnyParams& p, int grid, cudaStream_t st) {
  constexpr int smem = skinny_smem_bytes<NT, WARPS, D>();
  static bool attr_set[64] = {};
  int dev = 0;
  W4_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    W4_CUDA(cudaFuncSetAttribute(k_skinny<NT, WARPS, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = config().pdl ? 1 : 0;
  W4_CUDA(cudaLaunchKernelEx(&cfg, k_skinny<NT, WARPS, D>, p));
  return W4A16_OK;
}

int tile_rows() { return config().warps * 16; }

int grid_for_shape(int out_f, int G, int sms) {
  const int tiles = (out_f + tile_rows() - 1) / tile_rows();
  const long long U = static_cast<long long>(tiles) * G;
  return static_cast<int>(U < sms ? U : sms);
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
  p.qw = reinterpret_cast<const uint4*>(w->qweight);
  p.sc = w->scale;
  p.zp = w->zp;
  p.x = x;
  p.M = M;
  p.N = w->out_f;
  p.K = w->in_f;
  p.G = w->num_groups;
  p.NRB = w->out_f / kRowBlock;
  p.tiles = (w->out_f + TR - 1) / TR;
  p.partial = s->partial;
  p.counters = reinterpret_cast<unsigned*>(s->xgsum);
  p.cta_pairs = s->xf;
  p.status = di->status;
  const int grid = grid_for_shape(w->out_f, w->num_groups, di->sms);
  if (int rc = w4a16_scratch_check(s, w->out_f, M)) return rc;
  const int nt = M <= 8 ? 1 : 2;
  if (config().warps == 16) return nt == 1 ? launch_cfg<1, 16, 4>(p, grid, st) : launch_cfg<2, 16, 4>(p, grid, st);
  return nt == 1 ? launch_cfg<1, 8, 6>(p, grid, st) : launch_cfg<2, 8, 6>(p, grid, st);
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
  s->max_splits = di->sms;  // CTAs of the persistent grid
  // two partial tiles per CTA (head and tail of its unit range), widest tile, 16 tokens
  s->partial_elems = static_cast<size_t>(di->sms) * 2 * kMaxTileRows * 16;
  const size_t counters = (static_cast<size_t>(max_out) / 128 + 2) * sizeof(unsigned);
  const size_t pairs = static_cast<size_t>(di->sms) * 16 * sizeof(Pair);
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
  const size_t need = static_cast<size_t>(di->sms) * 2 * kMaxTileRows * 16;
  if (need > s->partial_elems)
    return fail(W4A16_ESCRATCH, "scratch: partial buffer holds %zu floats, %zu needed", s->partial_elems, need);
  if (out_f > s->max_out)
    return fail(W4A16_ESCRATCH, "scratch: sized for out_f <= %d, got %d", s->max_out, out_f);
  if (di->sms > s->max_splits)
    return fail(W4A16_ESCRATCH, "scratch: sized for %d CTAs, device has %d SMs", s->max_splits, di->sms);
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
  if (out_f <= 0 || out_f % (kRowBlock * nranks) != 0)
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
  if (row_begin < 0 || row_begin % kRowBlock != 0 || row_begin + w_shard->out_f > out_f_total)
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
