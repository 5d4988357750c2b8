// The decode-side W4A16 kernel for sm_100a: one persistent kernel serves the
// M=1 GEMV, the skinny GEMM of a speculative-verify block (M <= 16) and the
// lm_head GEMV with the argmax fused into its epilogue.
//
// Replaces k_prep + k_gemv + k_reduce, k_prep_m + k_gemm_small + k_reduce_bf16_m
// and k_gemm_mma of the reference (src/kernels/gemv_w4a16.cu:74-279,673-865) and,
// for lm_head, the separate argmax kernels (src/kernels/elementwise.cu:96-194).
//
// Shape of the computation (HBM-bound: every weight byte is read exactly once):
//   * persistent grid, one CTA per SM (24 warps, all 512 tensor-memory columns, about 160 KB of shared
//     memory). The (128-row tile, k group) units of the matrix are dealt out as equal contiguous
//     ranges, so every CTA streams the same number of bytes whatever N and K are. A row tile whose K
//     range is shared by several CTAs is finished by the CTA that owns its first units: the others
//     publish their partial rows as (sum, tag) words, the owner adds them in CTA order (bitwise
//     reproducible, no float atomics, no fences). Shared tiles are processed FIRST, so that this
//     overlaps everybody's main loop.
//   * the arithmetic is exact integer work on the 5th-generation tensor cores
//     (tcgen05.mma kind::i8, 128 x N x 32, int32 accumulators in tensor memory):
//       - weights: a nibble becomes an int8 with ONE logic instruction per four weights
//         (w & 0x0F0F0F0F, (w >> 4) & 0x0F0F0F0F) and goes straight from registers into tensor
//         memory as the A operand (tcgen05.st), one TMEM lane per output row;
//       - activations: per (token, k group) the 128 bf16 values are turned into block
//         fixed point, X = rint(x * 2^p) with |X| < 2^22 (exact for every element within 2^-14 of
//         the group's largest; smaller ones are rounded at 2^-22 of the largest), and X is split
//         into three signed 8-bit digits that form three rows of the B operand;
//       - per group:  y += s * 2^-p * ((D0 + 2^8 D1 + 2^16 D2) - zp * sum(X)),  Dj = sum(q * digit_j),
//         with the integer dot products exact and only this last step in fp32.
//     This keeps the per-byte instruction count low enough for the ALU pipe (LOP3/SHF issue at
//     half rate on this part) to keep up with HBM, which the bf16 formulations could not.
//   * every hand-off moves a STEP of two k groups; the roles are decoupled by mbarrier rings so that
//     none waits for a round trip:
//       producer    1 thread   one 17 KB bulk async copy per step into a shared-memory ring and the
//                              step's table entry; it never waits for the previous kernel
//       unpack      8 warps    nibbles -> int8 -> tensor memory (two warps per TMEM lane quarter,
//                              alternating steps), and the row's (scale, zero point) into a side ring
//       issuers     2 warps    even / odd steps: eight tcgen05.mma and one tcgen05.commit per step
//       fix-up      4 warps    tcgen05.ld of the int32 sums, the fp32 step above, the split-tile
//                  (+4)        reduction, output / fused argmax; for M >= 3 a second warp per lane
//                              quarter takes half of the tokens
//       converters  9 warps    M = 1 only; after griddepcontrol.wait: bf16 x -> digit rows of the B operand,
//                  (+fix-up)   once per CTA, for exactly the k groups it multiplies; issuers start on a
//                              group as soon as its rows are in
//   * M >= 2 (verify blocks): the digit rows are made ONCE per call by a small pre-pass kernel
//     (k_digits) into the scratch and every CTA streams the rows of the groups it multiplies through
//     a second ring of bulk copies (they come from L2), instead of 148 identical conversions of M
//     tokens and a cache of M x K digit bytes per CTA. 3 M <= 48 rows of B: one launch for every
//     M <= 16. The converter warps become more fix-up warps (up to three token sets).
#include <cfloat>
#include <climits>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace w4a16 {
namespace {

constexpr int CW = 4;                      // fix-up warps per CTA: 32 rows of the 128-row tile each
constexpr int kWarps = 24;
constexpr int kThreads = kWarps * 32;
constexpr int kWUnpack0 = 4;               // warps 4..11 unpack
constexpr int kWProducer = 12;
constexpr int kWMma = 13;                  // MMA issuer of the even steps; owns the tensor-memory allocation
constexpr int kWMma2 = 15;                 // MMA issuer of the odd steps
constexpr int kWConv0 = 16;                // warps 16..23 (and the otherwise idle warp 14) only convert activations
constexpr int kTeam = 4 + 1 + 8;           // converting warps: the fix-up warps, warp 14, warps 16..23
constexpr int kStepGroups = 2;             // k groups per step: every hand-off between roles moves two groups
// Weight formats: WB = 4 (AWQ int4 + zero points) or 8 (symmetric int8). A ring stage holds one step.
template <int WB>
struct Fmt {
  static constexpr int kBlock = WB == 4 ? kTileGroupBytes : kW8BlockBytes;  // bytes per (row tile, group)
  static constexpr int kStage = kStepGroups * kBlock;                        // 17152 / 33280
};
constexpr int kSideSteps = 12;             // (scale, zp) side ring, in steps: a slot is rewritten by the unpack warps
                                           // A-ring + D-ring depths (at most 4 + 8 steps) after the fix-up read it
constexpr int kSide = kSideSteps * 2;      // in groups
constexpr int kTable = 64;                 // step table entries (ring)
constexpr uint32_t kSpinLimit = 1u << 20;  // polls before a wait gives up
constexpr uint32_t kPieceTag = 0x7A6B5C4Du;  // upper half of a published (sum, tag) word of a split tile's piece
constexpr int kFixBar = 1;                 // named barrier of the fix-up warps
constexpr int kTmemCols = 512;             // all of tensor memory; the next launch's CTA, resident beside this one,
                                           // gets it when this CTA exits (it cannot multiply before that anyway)
constexpr int kAColsG = 32;                // 128 int8 along k = 32 columns of 32 bits per group


// Per token-count geometry. N = rows of the B operand the tensor core reads (3 digit rows per token are
// real). Ring depths are in steps: AD2 for A, DD2 for D and for the ring of "step done" barriers.
template <int MT, bool ST>
struct Geo {
  static constexpr bool kStream = ST;  // digit rows streamed from the pre-pass output instead of converted here
  static_assert(ST || MT == 1, "only the M = 1 kernel converts activations itself");
  // Token sets: the fix-up warps of one lane quarter split the tokens into FW sets of TM tokens; set F owns the
  // accumulator columns [CB F, CB F + 3 TM), so every set runs the SAME code on its own aligned column block
  // (one copy of the fix-up code per kernel: the instruction footprint of all roles has to stay cache resident).
  //   MT:        1    2    4    6    8    9   12   15   16
  //   FW x TM: 1x1  2x1  2x2  2x3  2x4  3x3  3x4  3x5  2x8
  static constexpr int FW = MT <= 1 ? 1 : ((MT == 9 || MT == 12 || MT == 15) ? 3 : 2);
  static constexpr int TM = (MT + FW - 1) / FW;                // tokens per fix-up warp
  static constexpr int CB = !ST ? 16 : (3 * TM <= 8 ? 8 : (3 * TM <= 16 ? 16 : 24));  // accumulator columns per set
  static constexpr int N = !ST ? 16 : ((FW * CB + 15) / 16) * 16;  // rows of the B operand the tensor core reads
  static constexpr int AD2 = N == 48 ? 2 : 4;
  static constexpr int DD2 = N == 16 ? 8 : 4;
  static constexpr int kAColsS = kStepGroups * kAColsG;  // A columns per step
  static constexpr int kDColsS = kStepGroups * N;        // D columns per step
  static constexpr int kDCol0 = AD2 * kAColsS;           // first D column
  static constexpr int GB = 4;                           // M = 1: groups whose tensor-memory loads are in flight together
  // Who waits for "the D slot this step fills has been read out". With a deep D ring (8 steps) the unpack warps
  // do, long before it matters, and the issuers - the busiest threads at M = 1 - are spared the wait; with a
  // shallow one (4 steps) the wait is on the critical loop and belongs to the issuer, so that the operand is
  // already unpacked when the slot comes free.
  static constexpr bool kIssuerWaitsD = DD2 < 8;
  static_assert(3 * TM <= CB && FW * CB <= N, "token sets must fit their column blocks");
  static_assert(kDCol0 + DD2 * kDColsS <= kTmemCols, "tensor memory budget");
  static_assert(AD2 <= DD2 && 2 <= DD2 / 2, "ring depths");
  static_assert(AD2 + DD2 <= kSideSteps, "a (scale, zp) slot must have been read before the unpack warps reuse it");
};

struct SkinnyParams {
  const uint8_t* stream;  // weight stream, Fmt<WB>::kBlock bytes per (row tile, group)
  const uint16_t* x;      // [M][K] bf16
  void* y;                // bf16 or fp32 [M][ldy], may be null in argmax mode
  int y_f32;
  long long ldy;  // elements between rows of y
  int y_col0;     // first column of this launch's rows inside y
  int M, N, K, G, tiles;
  int b_bytes;       // bytes of the B region (M = 1: digit rows of the groups this CTA multiplies; else the digit ring)
  int xs_bytes;      // bytes of the (sum, 2^-p) region (M = 1)
  const uint8_t* dig;  // pre-pass output: G blocks of db_bytes = [8 chunks of 16 k][3 M digit rows] 16 B, then G x M (sum, 2^-p) pairs
  int db_bytes;
  int bdepth;        // M >= 2: steps in the digit ring (a power of two)
  int bshift;        //         and its log2
  unsigned long long mg_grid, mg_G;  // ceil(2^40 / d) for d = gridDim.x and G: exact division by multiply
  uint32_t hint;     // suspend-time hint of the mbarrier waits, ns
  int depth;         // weight ring stages
  float* partial;
  unsigned* counters;  // [tiles * CW + 1], zero between launches
  int argmax;
  int32_t* ids;
  void* pairs_out;  // M x {float,int}
  int row_offset;
  void* cta_pairs;  // [grid][16] x {float,int}
  int* status;
  int npeers;  // extra destinations for y (fused all-gather / partial sums for a cross-rank reduction), 0 = none
  void* y_peers[8];  // bf16, or fp32 when y_f32
  const uint16_t* ln_w;  // RMSNorm fused into the pre-pass: x is normalised with these bf16 weights first (null: off)
  float ln_eps;
  uint16_t* xn_out;      // optional [M][K] copy of the normalised activations
  int epilogue;      // kEpiNone, kEpiSwiglu (rows interleaved gate, up, gate, up ...: y[m][row / 2] = silu(gate) * up)
                     // or kEpiResidual (y[m][row] = bf16(float(y[m][row]) + float(bf16(sum))))
  // cross-rank completion flags of the sharded calls (all null / 0 when unused). A rank's block:
  // words [0, 8) counters written by the ranks (word r by rank r), word 16 this rank's count of signalling launches.
  unsigned* comm_local;
  unsigned* comm_peers[8];   // every rank's block, index = rank (the local one included)
  int comm_n, comm_rank;
  int ordered;               // launch without the programmatic-serialisation attribute (a weight write is in front)
  int comm_wait;             // before x is read: wait until every rank has signalled its previous launch
  int comm_signal;           // after the last store of the grid: raise this rank's flag on every rank
  void* pairs_peers[8];      // vocab-sharded lm_head: every rank's [ranks][16] table of (max, index) pairs
};

constexpr int kEpiNone = 0, kEpiSwiglu = 1, kEpiResidual = 2;

struct Pair {
  float v;
  int i;
};

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

// ---- the order in which a CTA walks its unit range [u0,u1) -------------------------------
// A segment is a run of consecutive k groups of one row tile. The piece at the START of the range (the end of
// a row tile that the previous CTA began) always comes first: it is only published, and the CTA that adds that
// tile up finds it early. The piece at the END of the range (the beginning of a row tile, which this CTA adds
// up once the other CTAs' pieces are there) comes second where an idle warp can do the waiting while the whole
// tiles stream (tail_last = false: M = 1 without the fused argmax), and last otherwise, when every piece it
// waits for - first or only segments of their CTAs - has long been published. A segment of L groups is
// ceil(L/2) steps.
struct Seg {
  int tile, g0, L;
  bool whole;  // the segment is the tile's full K range
};

struct SegIter {
  int G, t_first, t_last, head_g0, tail_g1;
  bool single, head_partial, tail_partial, tail_last;
  int phase, t;

  __device__ void init(int u0, int u1, int G_, unsigned long long mg_G, bool tail_last_) {
    G = G_;
    tail_last = tail_last_;
    t_first = static_cast<int>(static_cast<uint32_t>((static_cast<unsigned long long>(u0) * mg_G) >> 40));
    t_last = static_cast<int>(static_cast<uint32_t>((static_cast<unsigned long long>(u1 - 1) * mg_G) >> 40));
    head_g0 = u0 - t_first * G;
    tail_g1 = u1 - t_last * G;
    single = (t_first == t_last);
    head_partial = single ? !(head_g0 == 0 && tail_g1 == G) : (head_g0 != 0);
    tail_partial = single ? false : (tail_g1 != G);
    phase = 0;
    t = t_first;
  }
  __device__ bool next(Seg& s) {
    if (phase == 0) {
      phase = 1;
      if (head_partial) {
        s.tile = t_first; s.g0 = head_g0; s.L = (single ? tail_g1 : G) - head_g0; s.whole = false;
        return true;
      }
    }
    if (phase == 1) {
      phase = 2;
      if (tail_partial && !tail_last) {
        s.tile = t_last; s.g0 = 0; s.L = tail_g1; s.whole = false;
        return true;
      }
    }
    while (t <= t_last) {
      const int tt = t++;
      if (tt == t_first && head_partial) continue;
      if (tt == t_last && tail_partial) continue;
      s.tile = tt; s.g0 = 0; s.L = G; s.whole = true;
      return true;
    }
    if (phase == 2) {
      phase = 3;
      if (tail_partial && tail_last) {
        s.tile = t_last; s.g0 = 0; s.L = tail_g1; s.whole = false;
        return true;
      }
    }
    return false;
  }
  // number of steps of the whole walk
  __device__ int steps() const {
    int n = 0;
    if (tail_partial) n += (tail_g1 + 1) >> 1;
    if (head_partial) n += ((single ? tail_g1 : G) - head_g0 + 1) >> 1;
    int whole = t_last - t_first + 1 - (head_partial ? 1 : 0) - (tail_partial ? 1 : 0);
    n += whole * ((G + 1) >> 1);
    return n;
  }
};

// Step table entry, written by the producer, read by the MMA issuers and the fix-up warps:
//   x = slot0 | slot1 << 8 | (groups - 1) << 16 | last step of its segment << 17 | whole tile << 18 | first k group << 19
//   y = row tile
__device__ __forceinline__ uint32_t step_word(int slot0, int slot1, int ng, bool seg_last, bool whole, int g0) {
  return static_cast<uint32_t>(slot0) | (static_cast<uint32_t>(slot1) << 8) | (static_cast<uint32_t>(ng - 1) << 16) |
         (seg_last ? 1u << 17 : 0u) | (whole ? 1u << 18 : 0u) | (static_cast<uint32_t>(g0) << 19);
}

// ---- PTX used only here ------------------------------------------------------------------
// One lane of the (converged) warp; unlike a test of the lane index this keeps the code around it
// warp-uniform for the compiler, so tensor-core operands stay in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
// Bounded wait with a per-launch suspend hint: how long one try_wait may park the thread.
__device__ __forceinline__ bool wait_h(uint32_t bar, uint32_t parity, uint32_t hint_ns, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity, hint_ns)) return true;
  return false;
}
// Instruction descriptor for kind::i8: signed 8-bit A and B (both K-major), int32 accumulate.
__host__ __device__ constexpr uint32_t umma_idesc_s8(int M, int N) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem desc], int8 x int8 -> int32; issued by ONE thread.
__device__ __forceinline__ void umma_s8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t* d) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* d) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* d) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]),
        "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
      : "r"(taddr)
      : "memory");
}
// Columns [C0, C0 + CNT) of this thread's lane, relative to `base` (a multiple of CNT's block size; C0 and CNT
// multiples of 8), as loads of 16 or 8 columns whose start is a multiple of their width; the caller awaits
// them all at once.
template <int C0, int CNT>
__device__ __forceinline__ void tmem_ld_span(uint32_t base, uint32_t* d) {
  if constexpr (CNT > 0) {
    // (a 24-column block starts at a multiple of 8 only: three loads of 8)
    constexpr int W = (C0 % 16 == 0 && CNT == 16) ? 16 : 8;
    if constexpr (W == 16) tmem_ld16(base + C0, d);
    else tmem_ld8(base + C0, d);
    tmem_ld_span<C0 + W, CNT - W>(base, d + W);
  }
}
__device__ __forceinline__ unsigned long long tagged(float v) {
  return (static_cast<unsigned long long>(kPieceTag) << 32) | __float_as_uint(v);
}
// u / d for u * d < 2^40, with m = ceil(2^40 / d) from the host: a multiply and a shift instead of the
// division loop (three of them sat in the start-up path of every launch).
__device__ __forceinline__ uint32_t fdiv(uint32_t u, unsigned long long m) {
  return static_cast<uint32_t>((static_cast<unsigned long long>(u) * m) >> 40);
}
// exact int -> float for |v| < 2^22 without the conversion pipe
__device__ __forceinline__ float small_int_to_float(uint32_t v) {
  return __uint_as_float(0x4B400000u + v) - 12582912.0f;
}

// dynamic shared memory:
//   [weight ring: depth x 17152][B region: b_bytes][(scale,zp) ring: kSide x 128 x 4][(sum, 2^-p): xs_bytes]
//   [step table: kTable x 8][ready counters: 256 x 4][mbarriers][tmem base, flag]
// The B operand of one k group is eight 16-k chunks, 48 M bytes apart, each holding the 3 M digit rows in
// use as consecutive 16-byte rows (an 8-row core matrix every 128 bytes). The rows the tensor core reads
// beyond them are the next chunk's bytes: they only produce accumulator columns nobody reads, and the
// whole K range of a token fits: 384 bytes per group for M = 1.
// M = 1 with the conversion inside the kernel: warps 16..19 have nothing to do once the activations are
// converted. When a fix-up warp reaches the end of a split tile's piece that this CTA has to add up, and more of
// the CTA's walk follows, the waiting for the other CTAs' pieces (a global-memory round trip of 1 to 2 us under
// load, which a fix-up warp in the middle of the stream cannot make up for) goes to the helper warp of its lane
// quarter: a mailbox entry of 32 sums and the tile number (two entries per quarter; one is used).
template <int MT, bool ST>
__host__ __device__ constexpr bool tile_end_helper() { return MT == 1 && !ST; }
constexpr int kMailStride = 40;                    // words per mailbox entry (32 sums, the tile, padding)
constexpr int kMailWords = 2 * CW * kMailStride;
template <int MT, bool ST>
__host__ __device__ constexpr int bar_count(int depth, int bdepth) {
  return 2 * depth + Geo<MT, ST>::AD2 + 2 * Geo<MT, ST>::DD2 + 2 + (ST ? 2 * bdepth : 0) + 1 + (tile_end_helper<MT, ST>() ? 2 * CW : 0);
}
template <int MT, bool ST>
__host__ __device__ inline int total_smem(int depth, int stage_bytes, int b_bytes, int xs_bytes, int bdepth) {
  return depth * stage_bytes + b_bytes + kSide * kTileRows * 4 + xs_bytes + kTable * 8 + 256 * 4 +
         (tile_end_helper<MT, ST>() ? kMailWords * 4 : 0) + bar_count<MT, ST>(depth, bdepth) * 8 + 16;
}

// One token's 128 values of one k group (this lane: k = 4 lane .. 4 lane + 3, `rv`) -> three int8 digit
// rows of the B operand at `bslot` (rows row0, row0 + 1, row0 + 2 of every 16-k chunk, chunks `lbo` bytes apart)
// and (sum of X, 2^-p) at `xs`.
//   X = rint(x * 2^p), p chosen per group so that the largest |X| lies in [2^21, 2^22).
//   The fp32 magic constant 1.5 * 2^23 makes the FMA deliver X in the low mantissa bits; adding 0x808080
//   turns the balanced base-256 digits (d0, d1 in [-128,127], |d2| <= 64) into plain bytes, the XOR
//   with 0x808080 turns those bytes back into signed digits: X = d0 + 2^8 d1 + 2^16 d2.
// K index j of the operand holds k = 8 (j/8) + perm(j%8) with perm = {0,4,1,5,2,6,3,7}: the order in which
// the two nibble masks deliver a packed word's weights.
__device__ __forceinline__ void convert_group(uint2 rv, uint8_t* bslot, int lbo, int row0, float2* xs, int lane) {
  const uint32_t mx = __vmaxu2(rv.x & 0x7FFF7FFFu, rv.y & 0x7FFF7FFFu);
  const uint32_t am = max(mx & 0xFFFFu, mx >> 16);               // bf16 bits of the lane's largest magnitude
  const uint32_t e = __reduce_max_sync(0xffffffffu, am) >> 7;    // its biased exponent, group-wide
  // 2^p with p = 148 - e puts the largest magnitude into [2^21, 2^22); tiny groups are capped at 2^123
  const uint32_t me = min(275u - e, 250u);
  const float mult = (e == 255u) ? 0.f : __uint_as_float(me << 23);
  const float inv = (e == 255u) ? __uint_as_float(0x7FC00000u) : __uint_as_float((254u - me) << 23);  // NaN for inf/NaN input
  const float f0 = __uint_as_float(rv.x << 16), f1 = __uint_as_float(rv.x & 0xFFFF0000u);
  const float f2 = __uint_as_float(rv.y << 16), f3 = __uint_as_float(rv.y & 0xFFFF0000u);
  constexpr float kMagic = 12582912.0f;  // 0x4B400000
  const uint32_t u0 = __float_as_uint(fmaf(f0, mult, kMagic)), u1 = __float_as_uint(fmaf(f1, mult, kMagic));
  const uint32_t u2 = __float_as_uint(fmaf(f2, mult, kMagic)), u3 = __float_as_uint(fmaf(f3, mult, kMagic));
  const int tot = __reduce_add_sync(0xffffffffu, static_cast<int>((u0 + u1) + (u2 + u3) - 4u * 0x4B400000u));
  constexpr uint32_t kOff = 0x00808080u - 0x4B400000u;
  const uint32_t D0 = (u0 + kOff) ^ 0x00808080u, D1 = (u1 + kOff) ^ 0x00808080u;
  const uint32_t D2 = (u2 + kOff) ^ 0x00808080u, D3 = (u3 + kOff) ^ 0x00808080u;
  // 4 x 3 byte transpose: digit planes of the lane's four k
  const uint32_t t01 = __byte_perm(D0, D1, 0x5140), t23 = __byte_perm(D2, D3, 0x5140);
  const uint32_t P0 = __byte_perm(t01, t23, 0x5410), P1 = __byte_perm(t01, t23, 0x7632);
  const uint32_t P2 = __byte_perm(__byte_perm(D0, D1, 0x0062), __byte_perm(D2, D3, 0x0062), 0x5410);
  const uint32_t Q0 = __shfl_xor_sync(0xffffffffu, P0, 1), Q1 = __shfl_xor_sync(0xffffffffu, P1, 1);
  const uint32_t Q2 = __shfl_xor_sync(0xffffffffu, P2, 1);
  // even lane: k offsets 0..3 of its 8-block -> operand bytes {E0,O0,E1,O1}; odd lane: {E2,O2,E3,O3}
  const uint32_t sel = (lane & 1) ? 0x3726u : 0x5140u;
  uint8_t* dst = bslot + (lane >> 2) * lbo + 4 * (lane & 3) + 16 * row0;
  *reinterpret_cast<uint32_t*>(dst) = __byte_perm(P0, Q0, sel);
  *reinterpret_cast<uint32_t*>(dst + 16) = __byte_perm(P1, Q1, sel);
  *reinterpret_cast<uint32_t*>(dst + 32) = __byte_perm(P2, Q2, sel);
  if (lane == 0) *xs = make_float2(static_cast<float>(tot), inv);
}

// COMM: the cross-rank flag code (wait before x is read, signal after the last store, the pair exchange of the
// vocab-sharded head) is compiled into separate instances, so that single-GPU launches run exactly the code
// they ran without it.
template <int MT, int WB, bool ST, bool COMM>
__global__ void __launch_bounds__(kThreads, 1) k_skinny(const SkinnyParams p) {
  using GE = Geo<MT, ST>;
  constexpr int kBlock = Fmt<WB>::kBlock, kStageBytes = Fmt<WB>::kStage;
  constexpr int N = GE::N, AD2 = GE::AD2, DD2 = GE::DD2;
  constexpr bool kStream = GE::kStream;
  constexpr int SLOT = kTileRows * MT;  // floats per partial tile
  extern __shared__ __align__(128) uint8_t smem[];

  const int DS = p.depth;
  uint8_t* ring = smem;
  uint8_t* bq = ring + DS * kStageBytes;
  uint8_t* side = bq + p.b_bytes;
  uint8_t* xsinv = side + kSide * kTileRows * 4;
  uint2* table = reinterpret_cast<uint2*>(xsinv + p.xs_bytes);
  uint32_t* ready = reinterpret_cast<uint32_t*>(table + kTable);  // [slot]: tokens whose digit rows are written
  float* mail = reinterpret_cast<float*>(ready + 256);  // [2 entries][lane quarter][kMailStride] (helper instances only)
  constexpr bool kHelper = tile_end_helper<MT, ST>();
  uint64_t* bars = reinterpret_cast<uint64_t*>(ready + 256 + (kHelper ? kMailWords : 0));
  const int BD = p.bdepth, BS = p.bshift;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + bar_count<MT, ST>(DS, BD));
  int* sflag = reinterpret_cast<int*>(tmem_slot + 1);

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // the same value, but provably warp-uniform
  const int G = p.G, M = p.M;
  const int U = p.tiles * G;
  // (U * gridDim.x fits 32 bits: checked on the host; a 64-bit division here costs a visible part of the start-up)
  const int u0 = static_cast<int>(fdiv(static_cast<uint32_t>(U) * blockIdx.x, p.mg_grid));
  const int u1 = static_cast<int>(fdiv(static_cast<uint32_t>(U) * (blockIdx.x + 1), p.mg_grid));
  // the digit rows of the groups this CTA multiplies, (g_first + j) % G for j < min(G, u1 - u0), live in slot j
  const int g_first = u0 - static_cast<int>(fdiv(static_cast<uint32_t>(u0), p.mg_G)) * G;
  auto cache_slot = [&](int g) { return g - g_first + (g < g_first ? G : 0); };
  // bytes between the digit rows of consecutive groups (cache slots for M = 1, ring slots otherwise), and
  // between the 16-k chunks of one group
  const int b_slot = kStream ? p.db_bytes : 384 * M, b_lbo = kStream ? 16 * N : 48 * M;
  const bool tail_last = !(tile_end_helper<MT, ST>() && !p.argmax);  // see SegIter
  int T;       // steps of this CTA
  int nsplit;  // 1 if the helper warps get a segment of this CTA: the piece at the end of its range (the first
               // piece of that tile, so this CTA adds the tile up) with whole tiles still to come after it
  {
    SegIter si;
    si.init(u0, u1, G, p.mg_G, tail_last);
    T = si.steps();
    const int whole = si.t_last - si.t_first + 1 - (si.head_partial ? 1 : 0) - (si.tail_partial ? 1 : 0);
    nsplit = (si.tail_partial && whole > 0 && !tail_last) ? 1 : 0;
  }

  const uint32_t ring_a = smem_u32(ring);
  const uint32_t bq_a = smem_u32(bq);
  const uint32_t side_a = smem_u32(side);
  const uint32_t xsinv_a = smem_u32(xsinv);
  const uint32_t wfull_a = smem_u32(bars);          // [DS]  weights of a step landed (tx bytes)
  const uint32_t wempty_a = wfull_a + DS * 8;       // [DS]  stage free again (4 unpack warps)
  const uint32_t afull_a = wempty_a + DS * 8;       // [AD2] A slot written (4 unpack warps)
  const uint32_t done_a = afull_a + AD2 * 8;        // [DD2] step t's MMAs have completed (tcgen05.commit): its sums are
                                                    //       in D slot t % DD2, its A slot t % AD2 is free again
  const uint32_t dempty_a = done_a + DD2 * 8;       // [DD2] D slot read out (4 fix-up warps)
  const uint32_t bready_a = dempty_a + DD2 * 8;     // every needed group's digit rows are written
  const uint32_t tmemrdy_a = bready_a + 8;          // tensor memory allocated, base address published
  const uint32_t bfull_a = tmemrdy_a + 8;           // [BD]  M >= 2: digit rows of a step landed (tx bytes)
  const uint32_t bempty_a = bfull_a + BD * 8;       // [BD]  M >= 2: the step's MMAs have completed (seen by the first fix-up warp)
  const uint32_t commrdy_a = bfull_a + (kStream ? 2 * BD : 0) * 8;  // every rank's flag of the previous launch has been seen
  const uint32_t mailfull_a = commrdy_a + 8;        // [2][CW] helper instances: a split segment's sums are in the mailbox

  if (tid < 256) ready[tid] = 0u;
  {
    // barrier i of the block [wfull | wempty | afull | done | dempty | bready | tmemrdy]: arrival counts
    // (+ [bfull | bempty] for M >= 2)
    const int nb = bar_count<MT, ST>(DS, BD), nb0 = 2 * DS + AD2 + 2 * DD2 + 2;
    const uint32_t nfix = CW * ((M + GE::TM - 1) / GE::TM);                // active fix-up warps
    if (tid < nb) {
      uint32_t cnt = 1;                                                    // wfull, done, tmemrdy, bfull
      if (tid >= DS && tid < 2 * DS + AD2) cnt = 4;                        // wempty, afull: 4 unpack warps
      else if (tid >= 2 * DS + AD2 + DD2 && tid < 2 * DS + AD2 + 2 * DD2) cnt = nfix;  // dempty
      else if (tid == nb0 - 2) cnt = kStream ? 1 : kTeam;                  // bready
      mbar_init(wfull_a + tid * 8, cnt);
    }
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  // The previous launch's CTA on this SM may still hold tensor memory: only this warp waits for it.
  if (warp == kWMma) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(tmemrdy_a);
  }

  bool team_ok = true;
  const bool converts = !kStream && (warp < CW || warp == 14 || warp >= kWConv0);
  if (converts) {
    // ================================================================ activations -> digit rows, once per CTA
    // The fix-up warps (idle until the first sums exist) and nine warps that do nothing else. The unpack
    // warps and the issuers do not take part: they fill the A ring from the weights meanwhile. x comes straight from global memory (L2); a round's loads are all in
    // flight before its first conversion.
    pdl_wait();  // the previous kernel produced x
    if (COMM && p.comm_wait) {
      // x is a gathered output: every rank's slice of it must have landed here. ONE thread of the CTA polls
      // the flags (thousands of pollers on one line would stand in the way of the very store they wait
      // for); the other converting warps park on a barrier of the CTA.
      if (warp == kWConv0) {
        const bool seen = wait_flags(p.comm_local, p.comm_n, comm_seq(p.comm_local), kFlagSpinLimit);
        if (lane == 0) {
          if (!seen) atomicExch(p.status, W4A16_ETIMEOUT);
          mbar_arrive(commrdy_a);
        }
        __syncwarp();
      } else if (!wait_h(commrdy_a, 0, p.hint, 4 * kSpinLimit)) {
        atomicExch(p.status, W4A16_ETIMEOUT);
      }
    }
    const int ti = warp < CW ? warp : (warp == 14 ? CW : warp - kWConv0 + CW + 1);
    const int cnt = (u1 - u0 < G) ? u1 - u0 : G;
    const int total = cnt * M;  // (group, token) items; item i belongs to warp i % kTeam
    constexpr int kBatch = 4;
    for (int i0 = ti; i0 < total; i0 += kBatch * kTeam) {
      uint2 rv[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int i = i0 + j * kTeam;
        if (i < total) {
          const int gj = i, m = 0;
          int g = g_first + gj;
          if (g >= G) g -= G;
          rv[j] = __ldcg(reinterpret_cast<const uint2*>(p.x + static_cast<size_t>(m) * p.K + g * kGroup) + lane);
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int i = i0 + j * kTeam;
        if (i < total) {
          const int gj = i, m = 0;
          convert_group(rv[j], bq + gj * b_slot, b_lbo, m, reinterpret_cast<float2*>(xsinv) + gj * MT + m, lane);
          // publish the item: B was written through the generic proxy, the tensor core reads it through the
          // async one; the slot counts as ready once all M tokens are in. Slots are numbered in the order the
          // CTA walks its groups, and items are taken in slot order, so the first steps can start after the
          // first round.
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            __threadfence_block();
            atomicAdd(ready + gj, 1u);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bready_a);
  }

  // This CTA owns all 512 columns, so its tensor-memory addresses start at 0: a compile-time constant
  // keeps every tcgen05 address warp-uniform. (Checked once; anything else is reported, not used.)
  constexpr uint32_t tmem = 0;
  const bool uses_tmem = warp < kWProducer || warp == kWMma || warp == kWMma2 || warp >= kWConv0;
  if (uses_tmem) {
    if (!wait_h(tmemrdy_a, 0, p.hint, kSpinLimit) || *reinterpret_cast<volatile uint32_t*>(tmem_slot) != 0u) {
      atomicExch(p.status, W4A16_ETIMEOUT);
      team_ok = false;
    }
    tc_fence_after();
  }

  if (warp == kWProducer) {
    // ================================================================ weight producer
    // One thread streams this CTA's share of the weight stream, one step (two consecutive (tile, group)
    // blocks, 17 KB) per bulk copy, and writes the step's table entry. It does not wait for the previous
    // kernel: weights never depend on it.
    if (lane == 0) {
      SegIter it;
      it.init(u0, u1, G, p.mg_G, tail_last);
      Seg sg;
      int st = 0, t = 0;
      uint32_t ph = 1;  // a fresh "empty" barrier reads as already released
      bool ok = true;
      while (ok && it.next(sg)) {
        const uint8_t* src = p.stream + (static_cast<size_t>(sg.tile) * G + sg.g0) * kBlock;
        for (int gl = 0; gl < sg.L; gl += kStepGroups, ++t) {
          const int ng = (sg.L - gl < kStepGroups) ? sg.L - gl : kStepGroups;
          if (!mbar_wait_bounded_relaxed(wempty_a + st * 8, ph, kSpinLimit)) {
            atomicExch(p.status, W4A16_ETIMEOUT);
            ok = false;
            break;
          }
          // where the step's digit rows are: cache slots (M = 1) or the two halves of digit-ring slot t % BD
          const int s0 = kStream ? 2 * (t & (BD - 1)) : cache_slot(sg.g0 + gl);
          const int s1 = ng == 2 ? (kStream ? s0 + 1 : cache_slot(sg.g0 + gl + 1)) : s0;
          table[t & (kTable - 1)] =
              make_uint2(step_word(s0, s1, ng, gl + kStepGroups >= sg.L, sg.whole, sg.g0 + gl), static_cast<uint32_t>(sg.tile));
          mbar_expect_tx(wfull_a + st * 8, ng * kBlock);
          bulk_g2s(ring_a + st * kStageBytes, src + static_cast<size_t>(gl) * kBlock, ng * kBlock, wfull_a + st * 8);
          if (++st == DS) {
            st = 0;
            ph ^= 1;
          }
        }
      }
      // every copy this thread started has to land before the CTA may exit
      for (int i = 0; i < DS && i < t; ++i) {
        const int k = t - 1 - i;  // the last copy into stage k % DS
        mbar_wait_bounded_relaxed(wfull_a + (k % DS) * 8, static_cast<uint32_t>(k / DS) & 1u, 1u << 14);
      }
    }
  } else if (warp == kWMma || warp == kWMma2) {
    // ================================================================ MMA issuers
    // Two warps, even and odd steps; one elected lane issues. Issuing a step's eight small MMAs and its
    // commit costs one thread more than the step's share of the HBM time; two issuers run side by side.
    // A step with a single group still issues both groups' MMAs: the second reads stale operands and
    // fills accumulator columns nobody reads.
    if (team_ok) {
      constexpr uint32_t idesc = umma_idesc_s8(128, N);
      const int mine = (warp == kWMma) ? 0 : 1;
      bool ok = true;
      bool all_ready = false;  // true once every slot is known to be written: no more polling
      // descriptor of the B region's first block, first 32-k step; other blocks and steps only move the address field
      const uint64_t desc0 = umma_desc_kmajor(bq_a, b_lbo, 128);
      const uint32_t step16 = (2 * b_lbo) >> 4, slot16 = static_cast<uint32_t>(b_slot) >> 4;
      for (int t = mine; ok && t < T; t += 2) {
        const int a = t & (AD2 - 1), d = t & (DD2 - 1);
        // A written (its writers also saw the step's weights and table entry landed), and the D slot this
        // step fills has been read out by every fix-up warp
        if (!wait_h(afull_a + a * 8, static_cast<uint32_t>(t / AD2) & 1u, p.hint, kSpinLimit) ||
            (GE::kIssuerWaitsD && t >= DD2 &&
             !wait_h(dempty_a + d * 8, static_cast<uint32_t>(t / DD2 - 1) & 1u, p.hint, kSpinLimit))) {
          atomicExch(p.status, W4A16_ETIMEOUT);
          break;
        }
        const uint32_t e = table[t & (kTable - 1)].x;
        if constexpr (kStream) {
          // the step's digit rows have landed in their ring slot (bulk copy: async proxy, as the MMA reads them)
          if (!wait_h(bfull_a + (t & (BD - 1)) * 8, static_cast<uint32_t>(t >> BS) & 1u, p.hint, kSpinLimit)) {
            atomicExch(p.status, W4A16_ETIMEOUT);
            break;
          }
        } else if (!all_ready) {
          // the digit rows of this step's two slots (all M tokens each) must be in shared memory
          const volatile uint32_t* rdy = ready;
          const uint32_t s0 = e & 0xFFu, s1 = (e >> 8) & 0xFFu, need = static_cast<uint32_t>(M);
          uint32_t spins = 0;
          while (rdy[s0] < need || rdy[s1] < need) {
            if (++spins > kSpinLimit) break;
            __nanosleep(40);
          }
          if (spins > kSpinLimit) {
            atomicExch(p.status, W4A16_ETIMEOUT);
            break;
          }
          __threadfence_block();
          all_ready = mbar_try_wait(bready_a, 0, 0);
        }
        tc_fence_after();
        const uint32_t d_t = tmem + GE::kDCol0 + d * GE::kDColsS;
        const uint32_t a_t = tmem + a * GE::kAColsS;
        const uint64_t db0 = desc0 + (e & 0xFFu) * slot16;
        const uint64_t db1 = desc0 + ((e >> 8) & 0xFFu) * slot16;
        if (elect_one()) {
          umma_s8_ts(d_t, a_t, db0, idesc, 0);
          umma_s8_ts(d_t, a_t + 8, db0 + step16, idesc, 1);
          umma_s8_ts(d_t, a_t + 16, db0 + 2 * step16, idesc, 1);
          umma_s8_ts(d_t, a_t + 24, db0 + 3 * step16, idesc, 1);
          umma_s8_ts(d_t + N, a_t + kAColsG, db1, idesc, 0);
          umma_s8_ts(d_t + N, a_t + kAColsG + 8, db1 + step16, idesc, 1);
          umma_s8_ts(d_t + N, a_t + kAColsG + 16, db1 + 2 * step16, idesc, 1);
          umma_s8_ts(d_t + N, a_t + kAColsG + 24, db1 + 3 * step16, idesc, 1);
          umma_commit(done_a + d * 8);
        }
        __syncwarp();
      }
    }
  } else if (warp >= kWUnpack0 && warp < kWUnpack0 + 8) {
    // ================================================================ unpack warps
    // Thread = one row of the tile = one TMEM lane. Per group: the row's 64 bytes of nibbles (four 16-byte
    // slots; int8 weights: 128 bytes, eight slots) -> 32 registers of int8 -> 32 TMEM columns of the A slot. Two warps per lane quarter, alternating
    // steps. Both groups of a step are always unpacked (a missing second group is stale bytes that feed
    // only unread accumulator columns), so this role needs nothing but the step number.
    const int q = warp & 3, pair = (warp - kWUnpack0) >> 2, r = q * 32 + lane;
    const uint32_t lane_t = tmem + (static_cast<uint32_t>(q * 32) << 16);
    // the row's slot in even and odd 32-k chunks (rotated by four slots in odd chunks)
    const uint32_t off_e = static_cast<uint32_t>(r) * 16, off_o = static_cast<uint32_t>((r + 4) & 127) * 16 + kChunkBytes;
    int st = pair % DS;
    uint32_t wph = static_cast<uint32_t>(pair / DS) & 1u;
    bool ok = team_ok;
    for (int t = pair; ok && t < T; t += 2) {
      const int a = t & (AD2 - 1);
      if (!wait_h(wfull_a + st * 8, wph, p.hint, kSpinLimit)) {
        atomicExch(p.status, W4A16_ETIMEOUT);
        break;
      }
      const uint8_t* base = ring + st * kStageBytes;
      // the first group's words are requested before the waits below
      constexpr int NW = WB == 4 ? 4 : 8;  // 16-byte pieces of a row per group
      uint4 wv[NW];
      auto load_row = [&](const uint8_t* gb) {
        if constexpr (WB == 4) {
          wv[0] = *reinterpret_cast<const uint4*>(gb + off_e);
          wv[1] = *reinterpret_cast<const uint4*>(gb + off_o);
          wv[2] = *reinterpret_cast<const uint4*>(gb + off_e + 2 * kChunkBytes);
          wv[3] = *reinterpret_cast<const uint4*>(gb + off_o + 2 * kChunkBytes);
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) wv[c] = *reinterpret_cast<const uint4*>(gb + c * kW8ChunkBytes + off_e);
        }
      };
      load_row(base);
      // the A slot's previous step has been multiplied (whether the D slot is free is the issuer's concern: the
      // operand can be unpacked while the fix-up warps are still reading the sums of DD2 steps ago)
      if ((t >= AD2 && !wait_h(done_a + ((t - AD2) & (DD2 - 1)) * 8, static_cast<uint32_t>((t - AD2) / DD2) & 1u, p.hint,
                               kSpinLimit)) ||
          (!GE::kIssuerWaitsD && t >= DD2 &&
           !wait_h(dempty_a + (t & (DD2 - 1)) * 8, static_cast<uint32_t>(t / DD2 - 1) & 1u, p.hint, kSpinLimit))) {
        atomicExch(p.status, W4A16_ETIMEOUT);
        break;
      }
      tc_fence_after();
      uint32_t* side_w = reinterpret_cast<uint32_t*>(side) + ((t % kSideSteps) * kStepGroups) * kTileRows + r;
#pragma unroll
      for (int j = 0; j < kStepGroups; ++j) {
        const uint8_t* gb = base + j * kBlock;
        if (j > 0) load_row(gb);
        uint32_t v[32];
        uint32_t sz;  // (bf16 scale << 16) | zero-point nibble
        if constexpr (WB == 4) {
          const uint32_t sc = *reinterpret_cast<const uint16_t*>(gb + kTgScaleOff + 2 * r);
          sz = (sc << 16) | *(gb + kTgZpOff + r);
          const uint32_t ww[16] = {wv[0].x, wv[0].y, wv[0].z, wv[0].w, wv[1].x, wv[1].y, wv[1].z, wv[1].w,
                                   wv[2].x, wv[2].y, wv[2].z, wv[2].w, wv[3].x, wv[3].y, wv[3].z, wv[3].w};
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            v[2 * i] = ww[i] & 0x0F0F0F0Fu;
            v[2 * i + 1] = (ww[i] >> 4) & 0x0F0F0F0Fu;
          }
        } else {
          // int8 codes are the operand as they are; symmetric, so the zero-point field stays 0
          sz = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(gb + kW8ScaleOff + 2 * r)) << 16;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            v[4 * c] = wv[c].x;
            v[4 * c + 1] = wv[c].y;
            v[4 * c + 2] = wv[c].z;
            v[4 * c + 3] = wv[c].w;
          }
        }
        const uint32_t a_t = lane_t + a * GE::kAColsS + j * kAColsG;
        tmem_st16(a_t, reinterpret_cast<const uint32_t(&)[16]>(v[0]));
        tmem_st16(a_t + 16, reinterpret_cast<const uint32_t(&)[16]>(v[16]));
        side_w[j * kTileRows] = sz;
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(afull_a + a * 8);
        mbar_arrive(wempty_a + st * 8);
      }
      st += 2;
      if (st >= DS) {
        st -= DS;
        wph ^= 1;
      }
    }
  } else if (warp == 14) {
    // ================================================================ digit-row producer (M >= 2)
    // One thread walks the same unit range as the weight producer and brings each step's digit rows (and the
    // tokens' (sum, 2^-p) pairs behind them) from the pre-pass output into the digit ring: one bulk copy per
    // step, two consecutive groups. The pre-pass is the previous kernel in the stream, so this thread - and
    // only this one - waits for it; the weights are already streaming meanwhile.
    if constexpr (kStream) {
      if (lane == 0 && team_ok) {
        pdl_wait();
        SegIter it;
        it.init(u0, u1, G, p.mg_G, tail_last);
        Seg sg;
        int t = 0;
        bool ok = true;
        const uint32_t db = static_cast<uint32_t>(p.db_bytes);
        // all (sum, 2^-p) pairs of the call, once: G x M x 8 bytes, read by the fix-up warps to the end
        mbar_expect_tx(bready_a, static_cast<uint32_t>(p.xs_bytes));
        bulk_g2s(xsinv_a, p.dig + static_cast<size_t>(G) * db, static_cast<uint32_t>(p.xs_bytes), bready_a);
        while (ok && it.next(sg)) {
          const uint8_t* src = p.dig + static_cast<size_t>(sg.g0) * db;
          for (int gl = 0; gl < sg.L; gl += kStepGroups, ++t) {
            const int ng = (sg.L - gl < kStepGroups) ? sg.L - gl : kStepGroups;
            const int sl = t & (BD - 1);
            // slot free: the MMAs of the step that used it last have completed
            if (t >= BD && !mbar_wait_bounded_relaxed(bempty_a + sl * 8, static_cast<uint32_t>((t >> BS) - 1) & 1u, kSpinLimit)) {
              atomicExch(p.status, W4A16_ETIMEOUT);
              ok = false;
              break;
            }
            mbar_expect_tx(bfull_a + sl * 8, ng * db);
            bulk_g2s(bq_a + sl * 2 * db, src + static_cast<size_t>(gl) * db, ng * db, bfull_a + sl * 8);
          }
        }
        // every copy this thread started has to land before the CTA may exit
        mbar_wait_bounded_relaxed(bready_a, 0, 1u << 14);
        for (int i = 0; i < BD && i < t; ++i) {
          const int k = t - 1 - i;
          mbar_wait_bounded_relaxed(bfull_a + (k & (BD - 1)) * 8, static_cast<uint32_t>(k >> BS) & 1u, 1u << 14);
        }
      }
    }
  } else if (warp < CW || warp >= kWConv0) {
    // ================================================================ fix-up warps
    // One warp per TMEM lane quarter and token set: warps 0..3 take the first TM tokens, warps 16..19 and
    // 20..23 (idle after converting) the next ones when M is larger. Each keeps its own running sums, so
    // the sets never have to be combined; a D slot is released when every active warp has loaded from it.
    auto fixup = [&](const int F, const bool helper) {  // F: this warp's token set; helper: only the split segments' ends
    constexpr int TM = GE::TM, CB = GE::CB;
    const int m0 = F * TM;                    // its tokens: m0 .. m0 + TM - 1 (those below M)
    const int q = warp & 3, r = q * 32 + lane;
    const int fslot = F * CW + q;             // this warp's index among the fix-up warps
    const uint32_t lane_t = tmem + (static_cast<uint32_t>(q * 32) << 16) + GE::kDCol0 + (kStream ? F * CB : 0);

    float fin[TM];
    float best_v[TM];
    int best_i[TM];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      fin[i] = 0.f;
      best_v[i] = -FLT_MAX;
      best_i[i] = INT_MAX;
    }

    // Final values of one row tile are in registers: write them out (plain, with the SwiGLU or the residual add
    // fused in, to the peers of a sharded call) and / or fold them into the running argmax.
    auto finalize = [&](int tile, const float(&v)[TM]) {
      const int row = tile * kTileRows + r;
      if (p.epilogue == kEpiSwiglu) {
        // SwiGLU fused in (replaces the separate kernel over the [M][2 I] buffer): rows come in (gate, up) pairs
        // on neighbouring lanes; both are rounded to bf16 first, as the unfused path stores them, then
        // y[m][row / 2] = bf16(gate / (1 + exp(-gate)) * up). All lanes take part in the exchange.
#pragma unroll
        for (int i = 0; i < TM; ++i) {
          const int m = m0 + i;
          if (m >= M) continue;  // (the same for the whole warp)
          const float mine = bf16_bits_to_float(float_to_bf16_bits(v[i]));
          const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
          if (!(lane & 1) && row < p.N) {
            const uint16_t hb = float_to_bf16_bits((mine / (1.f + expf(-mine))) * other);
            const size_t o = static_cast<size_t>(m) * p.ldy + p.y_col0 + (row >> 1);
            static_cast<uint16_t*>(p.y)[o] = hb;
            for (int pq = 0; pq < p.npeers; ++pq) static_cast<uint16_t*>(p.y_peers[pq])[o] = hb;
          }
        }
        return;
      }
      if (row >= p.N) return;  // zero-padded rows of the last tile
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        const int m = m0 + i;
        if (m >= M) continue;
        const uint16_t hb = float_to_bf16_bits(v[i]);
        if (p.y) {
          const size_t o = static_cast<size_t>(m) * p.ldy + p.y_col0 + row;
          if (p.y_f32) {
            static_cast<float*>(p.y)[o] = v[i];
            for (int pq = 0; pq < p.npeers; ++pq) static_cast<float*>(p.y_peers[pq])[o] = v[i];
          } else if (p.epilogue == kEpiResidual) {
            // residual add fused in: the running hidden state is read, the bf16-rounded sum added, written back
            uint16_t* h = static_cast<uint16_t*>(p.y) + o;
            *h = float_to_bf16_bits(bf16_bits_to_float(*h) + bf16_bits_to_float(hb));
          } else {
            static_cast<uint16_t*>(p.y)[o] = hb;
            for (int pq = 0; pq < p.npeers; ++pq) static_cast<uint16_t*>(p.y_peers[pq])[o] = hb;
          }
        }
        if (p.argmax) {
          const float lv = bf16_bits_to_float(hb);
          if (better(lv, row, best_v[i], best_i[i])) {
            best_v[i] = lv;
            best_i[i] = row;
          }
        }
      }
    };

    bool ok = team_ok;
    constexpr int GB = GE::GB;
    // accumulator columns this warp reads per group: its CB-column block, token m0 + i's three sums in columns
    // 3 i .. 3 i + 2 of it
    constexpr int NLD = kStream ? CB : 4;
    const uint32_t* side_r = reinterpret_cast<const uint32_t*>(side) + r;
    const float2* xs_tab = reinterpret_cast<const float2*>(xsinv);  // (sum, 2^-p): per cache slot (M = 1), else [k group][token]
    if constexpr (kStream) {
      // the pair table of the call arrives once, by bulk copy
      if (!wait_h(bready_a, 0, p.hint, kSpinLimit)) {
        atomicExch(p.status, W4A16_ETIMEOUT);
        ok = false;
      }
    }
    const bool hands_over = kHelper && !helper && !p.argmax;  // split segments end in the helper warp
    int nmail = 0;                                            // mailbox entries sent (fix-up) or taken (helper)
    for (int t = 0; ok && (helper ? nmail < nsplit : t < T);) {
      bool seg_end = true, seg_whole = false;
      int seg_tile = 0;
      if (helper) {
        const float* mslot = mail + (nmail * CW + q) * kMailStride;
        if (!wait_h(mailfull_a + (nmail * CW + q) * 8, 0, p.hint, 4 * kSpinLimit)) {
          atomicExch(p.status, W4A16_ETIMEOUT);
          break;
        }
        fin[0] = mslot[lane];
        seg_tile = reinterpret_cast<const int*>(mslot)[32];
        ++nmail;
      } else {
      // A round is one or two steps (two unless the first ends its segment): one wait per issuer (a commit
      // covers everything its thread issued before), GB groups' tensor-memory loads in flight together.
      if (!wait_h(done_a + (t & (DD2 - 1)) * 8, static_cast<uint32_t>(t / DD2) & 1u, p.hint, kSpinLimit)) {
        atomicExch(p.status, W4A16_ETIMEOUT);
        ok = false;
        break;
      }
      const uint2 e0 = table[t & (kTable - 1)];  // written before the step's weights were requested
      const bool two = !((e0.x >> 17) & 1u) && t + 1 < T;
      if (two && !wait_h(done_a + ((t + 1) & (DD2 - 1)) * 8, static_cast<uint32_t>((t + 1) / DD2) & 1u, p.hint, kSpinLimit)) {
        atomicExch(p.status, W4A16_ETIMEOUT);
        ok = false;
        break;
      }
      tc_fence_after();
      if constexpr (kStream) {
        // the round's MMAs are done with their digit rows: the ring slots go back to the digit producer
        if (F == 0 && q == 0 && lane == 0) {
          mbar_arrive(bempty_a + (t & (BD - 1)) * 8);
          if (two) mbar_arrive(bempty_a + ((t + 1) & (BD - 1)) * 8);
        }
      }
      const uint2 e1 = two ? table[(t + 1) & (kTable - 1)] : e0;
      const int ng0 = static_cast<int>((e0.x >> 16) & 1u) + 1;
      const int rg = two ? ng0 + static_cast<int>((e1.x >> 16) & 1u) + 1 : ng0;  // groups of the round (ng0 == 2 if two)
      // group k of the round: step t + (k >> 1), position k & 1
      if constexpr (!kStream || MT == 1) {
#pragma unroll
      for (int k0 = 0; k0 < 4; k0 += GB) {
        if (k0 < rg) {
          uint32_t dv[GB][NLD];
          uint32_t sz[GB];
#pragma unroll
          for (int j = 0; j < GB; ++j) {
            const int k = k0 + j;
            if (k < rg) {
              const int ts = t + (k >> 1);
              const uint32_t d_t = lane_t + (ts & (DD2 - 1)) * GE::kDColsS + (k & 1) * N;
              tmem_ld4(d_t, dv[j]);
              sz[j] = side_r[((ts % kSideSteps) * kStepGroups + (k & 1)) * kTileRows];
            }
          }
          tmem_wait_ld();
          if (k0 + GB >= rg) {  // the round's last loads are in registers: release its D slots
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(dempty_a + (t & (DD2 - 1)) * 8);
              if (two) mbar_arrive(dempty_a + ((t + 1) & (DD2 - 1)) * 8);
            }
          }
#pragma unroll
          for (int j = 0; j < GB; ++j) {
            const int k = k0 + j;
            if (k < rg) {
              const uint32_t ew = (k >> 1) ? e1.x : e0.x;
              const uint32_t slot = (k & 1) ? (ew >> 8) & 0xFFu : ew & 0xFFu;
              const float s = __uint_as_float(sz[j] & 0xFFFF0000u);
              const float z = __uint_as_float(0x4B000000u | (sz[j] & 0xFFu)) - 8388608.0f;
              {
                // (sum of X, 2^-p): by cache slot, or (pre-pass) by k group
                const float2 xv = xs_tab[kStream ? ((ew >> 19) & 0xFFu) + (k & 1) : slot];
                const float d0 = small_int_to_float(dv[j][0]);
                const float d1 = small_int_to_float(dv[j][1]);
                const float d2 = small_int_to_float(dv[j][2]);
                const float dot = fmaf(d2, 65536.f, fmaf(d1, 256.f, d0));
                fin[0] = fmaf(s * xv.y, fmaf(-z, xv.x, dot), fin[0]);
              }
            }
          }
        }
      }
      } else {
        // Per step: both groups' tensor-memory loads in flight together, one wait, and the step's D slot goes
        // back at once (the issuer of step t + DD2 is waiting for it); then the two groups are added up. (With
        // 24-column blocks the registers only allow one group at a time.)
        constexpr int kInFlight = NLD <= 16 ? 2 : 1;
        uint32_t dv[kInFlight][NLD];
        auto add_group = [&](const uint32_t* d, uint32_t szv, int g) {
          const float2* xs_g = xs_tab + g * M + m0;
          const float s = __uint_as_float(szv & 0xFFFF0000u);
          const float z = __uint_as_float(0x4B000000u | (szv & 0xFFu)) - 8388608.0f;
#pragma unroll
          for (int i = 0; i < TM; ++i) {
            // No test for "token exists" here: the TM chains stay independent straight-line code. A set's
            // tokens past M add up whatever their columns and the pair table's next entries hold, and are
            // never stored.
            const float2 xv = xs_g[i];  // (sum of X, 2^-p)
            const float d0 = small_int_to_float(d[3 * i]);
            const float d1 = small_int_to_float(d[3 * i + 1]);
            const float d2 = small_int_to_float(d[3 * i + 2]);
            const float dot = fmaf(d2, 65536.f, fmaf(d1, 256.f, d0));
            fin[i] = fmaf(s * xv.y, fmaf(-z, xv.x, dot), fin[i]);
          }
        };
#pragma unroll
        for (int sI = 0; sI < 2; ++sI) {
          if (sI == 0 || two) {
            const int ts = t + sI;
            const uint32_t ew = sI ? e1.x : e0.x;
            const int ng = static_cast<int>((ew >> 16) & 1u) + 1;
            const uint32_t d_t = lane_t + (ts & (DD2 - 1)) * GE::kDColsS;
            const int g0 = static_cast<int>((ew >> 19) & 0xFFu);  // the step's first k group: row of the pair table
            const uint32_t* side_s = side_r + ((ts % kSideSteps) * kStepGroups) * kTileRows;
            auto release = [&]() {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(dempty_a + (ts & (DD2 - 1)) * 8);
            };
            if constexpr (kInFlight == 2) {
              uint32_t sz[2];
              tmem_ld_span<0, NLD>(d_t, dv[0]);
              sz[0] = side_s[0];
              if (ng == 2) {
                tmem_ld_span<0, NLD>(d_t + N, dv[1]);
                sz[1] = side_s[kTileRows];
              }
              tmem_wait_ld();
              release();
              add_group(dv[0], sz[0], g0);
              if (ng == 2) add_group(dv[kInFlight - 1], sz[1], g0 + 1);
            } else {
              tmem_ld_span<0, NLD>(d_t, dv[0]);
              const uint32_t sz0 = side_s[0], sz1 = side_s[kTileRows];
              tmem_wait_ld();
              if (ng == 1) release();
              add_group(dv[0], sz0, g0);
              if (ng == 2) {
                tmem_ld_span<0, NLD>(d_t + N, dv[0]);
                tmem_wait_ld();
                release();
                add_group(dv[0], sz1, g0 + 1);
              }
            }
          }
        }
      }
      const uint2 el = two ? e1 : e0;  // the round's last step
      t += two ? 2 : 1;
      seg_end = ((el.x >> 17) & 1u) != 0;
      seg_whole = ((el.x >> 18) & 1u) != 0;
      seg_tile = static_cast<int>(el.y);
      }
      if (seg_end) {
        // ---- end of this CTA's segment of row tile seg_tile ----
        const int tile = seg_tile;
        bool last = seg_whole;  // a whole tile is final at once
        float v[TM];
#pragma unroll
        for (int i = 0; i < TM; ++i) v[i] = fin[i];
        if (!last) {
          // Split tile. Every piece but the tile's first is PUBLISHED: its 32 rows go to this CTA's slot as
          // 8-byte (sum, tag) words and the warp moves on - no fence, no ticket, nothing to wait for. The CTA
          // that owns the tile's first units is the one that adds up: it polls the other pieces' words until
          // their tags are there, adds them in CTA order to its own sums (a fixed order: bitwise reproducible),
          // zeroes the words for the next launch and writes the rows out. That piece is always the last one
          // of its owner's walk apart from whole tiles (the piece at the END of a range comes second, after
          // the piece at its start), and the pieces it waits for are the first or only segments of theirs.
          // first and last CTA whose unit range touches this tile (32-bit: U * gridDim.x < 2^32, host-checked)
          const uint32_t X0 = static_cast<uint32_t>(tile) * G, Uu = static_cast<uint32_t>(U);
          const int c_first = static_cast<int>(((X0 + 1) * gridDim.x - 1) / Uu);
          const int c_last = static_cast<int>(((X0 + G) * gridDim.x - 1) / Uu);
          unsigned long long* slots = reinterpret_cast<unsigned long long*>(p.partial);
          if (static_cast<int>(blockIdx.x) != c_first) {
            const int which = (static_cast<int>(fdiv(static_cast<uint32_t>(u0), p.mg_G)) == tile) ? 0 : 1;
            unsigned long long* slotp = slots + (static_cast<size_t>(blockIdx.x) * 2 + which) * SLOT;
#pragma unroll
            for (int i = 0; i < TM; ++i)
              if (m0 + i < M) st_relaxed_gpu_u64(slotp + (m0 + i) * kTileRows + r, tagged(fin[i]));
          } else {
            if constexpr (kHelper) {
              if (hands_over && t < T) {  // more of the walk follows: the helper warp does the waiting
                float* mslot = mail + (nmail * CW + q) * kMailStride;
                mslot[lane] = fin[0];
                if (lane == 0) reinterpret_cast<int*>(mslot)[32] = tile;
                __syncwarp();
                if (lane == 0) mbar_arrive(mailfull_a + (nmail * CW + q) * 8);
                ++nmail;
                fin[0] = 0.f;
                continue;
              }
            }
            last = true;
            constexpr int PB = TM <= 2 ? 4 : (TM <= 4 ? 2 : 1);  // pieces whose loads are in flight together
            for (int cb = c_first + 1; cb <= c_last && ok; cb += PB) {
              unsigned long long piece[PB][TM];
              const unsigned long long* sl[PB];
#pragma unroll
              for (int k = 0; k < PB; ++k) {
                const int cc = cb + k <= c_last ? cb + k : c_last;
                const uint32_t cu0 = fdiv(Uu * static_cast<uint32_t>(cc), p.mg_grid);
                const int wc = (static_cast<int>(fdiv(cu0, p.mg_G)) == tile) ? 0 : 1;
                sl[k] = slots + (static_cast<size_t>(cc) * 2 + wc) * SLOT + r;
              }
              uint32_t spins = 0;
              for (;;) {
                bool all = true;
#pragma unroll
                for (int k = 0; k < PB; ++k)
                  if (cb + k <= c_last) {
#pragma unroll
                    for (int i = 0; i < TM; ++i)
                      if (m0 + i < M) {
                        piece[k][i] = ld_relaxed_gpu_u64(sl[k] + (m0 + i) * kTileRows);
                        all = all && static_cast<uint32_t>(piece[k][i] >> 32) == kPieceTag;
                      }
                  }
                if (__all_sync(0xffffffffu, all)) break;
                if (++spins > kSpinLimit) {
                  atomicExch(p.status, W4A16_ETIMEOUT);
                  ok = false;
                  break;
                }
              }
#pragma unroll
              for (int k = 0; k < PB; ++k)
                if (cb + k <= c_last) {
#pragma unroll
                  for (int i = 0; i < TM; ++i)
                    if (m0 + i < M) {
                      v[i] += __uint_as_float(static_cast<uint32_t>(piece[k][i]));
                      st_relaxed_gpu_u64(const_cast<unsigned long long*>(sl[k]) + (m0 + i) * kTileRows, 0ull);
                    }
                }
            }
          }
        }
        if (last) finalize(tile, v);
#pragma unroll
        for (int i = 0; i < TM; ++i) fin[i] = 0.f;
      }
    }
    if (p.argmax) {
      // ---- fused argmax: thread -> warp -> CTA -> grid, larger value then lower index ----
      const int nfix = 32 * CW * ((M + TM - 1) / TM);  // threads of all active fix-up warps
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best_v[i], off);
          const int oi = __shfl_xor_sync(0xffffffffu, best_i[i], off);
          if (better(ov, oi, best_v[i], best_i[i])) {
            best_v[i] = ov;
            best_i[i] = oi;
          }
        }
      named_bar_sync(kFixBar, nfix);
      // per-warp candidates go through the (now idle) side ring: every unit has been read
      Pair* cand = reinterpret_cast<Pair*>(side);  // [fix-up warp][16 tokens]
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < TM; ++i) cand[fslot * 16 + m0 + i] = Pair{best_v[i], best_i[i]};
      }
      named_bar_sync(kFixBar, nfix);
      Pair* cta_pairs = static_cast<Pair*>(p.cta_pairs);
      if (tid < M) {
        Pair b{-FLT_MAX, INT_MAX};
        for (int w = 0; w < CW; ++w) {
          const Pair qv = cand[((tid / TM) * CW + w) * 16 + tid];  // the set that owns token `tid`, its four quarters
          if (better(qv.v, qv.i, b.v, b.i)) b = qv;
        }
        cta_pairs[blockIdx.x * 16 + tid] = b;
      }
      named_bar_sync(kFixBar, nfix);
      if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(p.counters + 3 * p.tiles * CW, 1u);
        const int last = (old == gridDim.x - 1);
        if (last) {
          p.counters[3 * p.tiles * CW] = 0;
          __threadfence();
        }
        *sflag = last;
      }
      named_bar_sync(kFixBar, nfix);
      if (*sflag) {
        // The last CTA to arrive: every CTA's pairs are in memory. One warp per token (in turn): its lanes load
        // the CTAs' pairs side by side - one L2 round trip instead of a thread walking all the CTAs - and a
        // shuffle tree picks the winner (larger value, else lower index: the order of comparisons does not matter).
        const int nw = nfix >> 5;
        for (int m = fslot; m < M; m += nw) {
          Pair b{-FLT_MAX, INT_MAX};
          for (unsigned cc = lane; cc < gridDim.x; cc += 32) {
            Pair qv;
            qv.v = __ldcg(&cta_pairs[cc * 16 + m].v);
            qv.i = __ldcg(&cta_pairs[cc * 16 + m].i);
            if (better(qv.v, qv.i, b.v, b.i)) b = qv;
          }
#pragma unroll
          for (int off = 16; off; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, b.v, off);
            const int oi = __shfl_xor_sync(0xffffffffu, b.i, off);
            if (better(ov, oi, b.v, b.i)) b = Pair{ov, oi};
          }
          if (lane == 0) cand[m] = b;
        }
        named_bar_sync(kFixBar, nfix);
      }
      if (*sflag && tid < M) {
        const Pair b = cand[tid];
        const int idx = (b.i == INT_MAX) ? 0 : b.i;  // nothing finite: index 0, as a plain scan gives
        const Pair mine{b.v, (b.i == INT_MAX) ? INT_MAX : b.i + p.row_offset};
        if (p.pairs_out) static_cast<Pair*>(p.pairs_out)[tid] = mine;
        if (COMM && p.comm_signal) {
          // vocab-sharded head: this rank's pair of every token goes to every rank's table (8 M bytes per
          // peer, no logits cross the link), then the flag; then the same threads wait for the other ranks'
          // pairs and pick the winner: larger value, else lower index.
          for (int r = 0; r < p.comm_n; ++r) static_cast<Pair*>(p.pairs_peers[r])[p.comm_rank * 16 + tid] = mine;
          __threadfence_system();
          const unsigned mask = (M >= 32) ? 0xffffffffu : ((1u << M) - 1u);
          __syncwarp(mask);
          unsigned seq = 0;
          if (tid == 0) seq = signal_whole_launch(p.comm_local, p.comm_peers, p.comm_n, p.comm_rank);
          seq = __shfl_sync(mask, seq, 0);
          if (!wait_flags(p.comm_local, p.comm_n, seq, kFlagSpinLimit, mask)) atomicExch(p.status, W4A16_ETIMEOUT);
          const Pair* tab = static_cast<const Pair*>(p.pairs_peers[p.comm_rank]);
          Pair w{-FLT_MAX, INT_MAX};
          for (int r = 0; r < p.comm_n; ++r) {
            Pair qv;
            qv.v = __ldcg(&tab[r * 16 + tid].v);
            qv.i = __ldcg(&tab[r * 16 + tid].i);
            if (better(qv.v, qv.i, w.v, w.i)) w = qv;
          }
          if (p.ids) p.ids[tid] = (w.i == INT_MAX) ? 0 : w.i;
        } else if (p.ids) {
          p.ids[tid] = idx + p.row_offset;
        }
      }
    }
    };
    const int fset = warp < CW ? 0 : (warp - kWConv0) / CW + 1;
    const bool helper = kHelper && warp >= kWConv0 && warp < kWConv0 + CW && !p.argmax;
    if (helper || (fset < GE::FW && fset * GE::TM < M)) fixup(helper ? 0 : fset, helper);
  }

  // every role ends here: tensor memory goes back only after all its readers and writers are done
  tc_fence_before();
  __syncthreads();
  if (warp == kWMma) {
    tc_fence_after();
    tmem_dealloc(*reinterpret_cast<volatile uint32_t*>(tmem_slot), kTmemCols);
  }
  // fused all-gather: every store of this CTA was issued before the barrier above
  if (COMM && p.comm_signal && !p.argmax && tid == 0) signal_cta_done(p.comm_local, p.comm_peers, p.comm_n, p.comm_rank);
}

// Pre-pass of the M >= 2 calls: one warp per (k group, token) turns the token's 128 bf16 values of the
// group into three digit rows of the B operand and its (sum, 2^-p) pair, laid out per group exactly as
// the main kernel's digit ring wants them ([8 chunks of 16 k][3 M rows] 16 B), the pairs as one [G][M] table
// behind all groups' rows. Small CTAs
// (four warps, at most 32 registers) so that they fit beside a resident main-kernel CTA of the previous
// layer and are ready to run the moment that layer completes.
__global__ void __launch_bounds__(128, 16) k_digits(const uint16_t* __restrict__ x, uint8_t* __restrict__ dig, int M,
                                                    int K, int G, int db_bytes, int tm, int cb,
                                                    const unsigned* comm_local, int comm_n, int* status,
                                                    const uint16_t* __restrict__ ln_w, float ln_eps,
                                                    uint16_t* __restrict__ xn_out) {
  pdl_launch_dependents();
  pdl_wait();  // the previous kernel produced x (and the main kernel before it may still be reading `dig`)
  if (comm_local) {
    // x is a gathered output: every rank's slice of it must have landed here
    if (threadIdx.x < 32 && !wait_flags(comm_local, comm_n, comm_seq(comm_local), kFlagSpinLimit))
      atomicExch(status, W4A16_ETIMEOUT);
    __syncthreads();
  }
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= G * M) return;
  const int g = item / M, m = item - g * M;
  uint2 rv = __ldcg(reinterpret_cast<const uint2*>(x + static_cast<size_t>(m) * K + g * kGroup) + lane);
  if (ln_w) {
    // RMSNorm fused in (replaces the separate kernel in front of the linear layer): the token's
    // inv = rsqrt(mean(x^2) + eps) over the whole row - every warp of the token recomputes it from L2 - then
    // xn = bf16(x * inv * (1 + w)), rounded to bf16 as the unfused path stores it, and the digits are taken of xn.
    const uint2* row = reinterpret_cast<const uint2*>(x + static_cast<size_t>(m) * K);
    float ss = 0.f;
    for (int j = lane; j < K / 4; j += 32) {
      const uint2 q = __ldcg(row + j);
      const float a0 = __uint_as_float(q.x << 16), a1 = __uint_as_float(q.x & 0xFFFF0000u);
      const float a2 = __uint_as_float(q.y << 16), a3 = __uint_as_float(q.y & 0xFFFF0000u);
      ss += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float inv = rsqrtf(ss / static_cast<float>(K) + ln_eps);
    const uint2 wq = __ldg(reinterpret_cast<const uint2*>(ln_w + g * kGroup) + lane);
    auto nrm = [&](uint32_t xb, uint32_t wb) {  // both bf16 bit patterns in the high half
      return static_cast<uint32_t>(float_to_bf16_bits(__uint_as_float(xb) * inv * (1.0f + __uint_as_float(wb))));
    };
    rv.x = nrm(rv.x << 16, wq.x << 16) | (nrm(rv.x & 0xFFFF0000u, wq.x & 0xFFFF0000u) << 16);
    rv.y = nrm(rv.y << 16, wq.y << 16) | (nrm(rv.y & 0xFFFF0000u, wq.y & 0xFFFF0000u) << 16);
    if (xn_out) reinterpret_cast<uint2*>(xn_out + static_cast<size_t>(m) * K + g * kGroup)[lane] = rv;
  }
  float2* pairs = reinterpret_cast<float2*>(dig + static_cast<size_t>(G) * db_bytes);
  // token m belongs to set m / tm; its digit rows are rows cb (m / tm) + 3 (m % tm) .. + 2 of every 16-k chunk,
  // a chunk being db_bytes / 8 bytes (N rows of 16 bytes)
  const int f = m / tm;
  convert_group(rv, dig + static_cast<size_t>(g) * db_bytes, db_bytes >> 3, cb * f + 3 * (m - f * tm), pairs + g * M + m, lane);
}

// Cross-rank reduction of a K-sharded layer: every rank's fp32 partial [M][N] sits in slot r of this rank's buffer
// (stored there by the producers' epilogues over NVLink); once every rank's flag is up, the slots are added in
// rank order - the same order on every rank, so all ranks get the same bits - and rounded to bf16 once; with
// `residual` the result is added to the running hidden state in place, as residual_add does.
__global__ void k_reduce_partials(uint16_t* __restrict__ y, const float* __restrict__ partials, int nranks, long long n,
                                  int residual, const unsigned* comm_local, int* status) {
  pdl_wait();
  if (threadIdx.x < 32 && !wait_flags(comm_local, nranks, comm_seq(comm_local), kFlagSpinLimit))
    atomicExch(status, W4A16_ETIMEOUT);
  __syncthreads();
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  float acc = 0.f;
  for (int r = 0; r < nranks; ++r) acc += __ldcg(partials + r * n + i);
  const uint16_t hb = float_to_bf16_bits(acc);
  y[i] = residual ? float_to_bf16_bits(bf16_bits_to_float(y[i]) + bf16_bits_to_float(hb)) : hb;
}

// Stand-alone wait for consumers that are not kernels of this library: returns once every rank has
// signalled the last gather (or sets W4A16_ETIMEOUT when the bounded wait runs out).
__global__ void k_wait_gather(const unsigned* comm_local, int n, int* status) {
  pdl_wait();
  if (threadIdx.x < 32 && !wait_flags(comm_local, n, comm_seq(comm_local), kFlagSpinLimit))
    atomicExch(status, W4A16_ETIMEOUT);
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
  int depth;     // weight ring stages (two blocks, 17152 B, each); even
  int pdl;
  int hint;      // suspend-time hint of the in-kernel mbarrier waits, ns
  int gemv_prepass;  // M = 1 through the pre-pass + digit ring as well (experiment; default off)
};

const Config& config() {
  static Config c = [] {
    Config k{6, 1, 2000, 0};
    if (const char* e = getenv("W4A16_GEMV_PREPASS")) k.gemv_prepass = atoi(e) != 0;
    if (const char* e = getenv("W4A16_DEPTH")) k.depth = atoi(e);
    if (const char* e = getenv("W4A16_PDL")) k.pdl = atoi(e) != 0;
    if (const char* e = getenv("W4A16_HINT")) k.hint = atoi(e);
    if (k.hint < 0) k.hint = 0;
    if (k.depth < 2) k.depth = 2;
    if (k.depth > 12) k.depth = 12;
    k.depth &= ~1;  // even: see the ring-depth note in launch_cfg
    return k;
  }();
  return c;
}

// counters of the scratch (sized for one per (token set, tile, lane quarter); in use: the fused argmax's arrival
// ticket behind them), for layers of up to max_out rows
size_t counter_bytes(int max_out) {
  return (3 * (static_cast<size_t>(max_out) / kTileRows + 2) * CW + 8) * sizeof(unsigned);
}

// bytes of the per-CTA argmax pair area at the front of the scratch's `xf` buffer
size_t pair_bytes(int max_splits) { return (static_cast<size_t>(max_splits) * 16 * sizeof(Pair) + 255) & ~static_cast<size_t>(255); }

constexpr int kMaxCtasPerSm = 2;  // what the scratch is sized for (the grid itself is one CTA per SM)

int tile_rows() { return kTileRows; }

int grid_for_shape(int out_f, int G, int sms) {
  const int tiles = (out_f + tile_rows() - 1) / tile_rows();
  const long long U = static_cast<long long>(tiles) * G;
  return static_cast<int>(U < sms ? U : sms);
}

// groups whose digit rows one CTA keeps: the most (tile, group) units any CTA gets, at most all of K
int cache_groups_for(int tiles, int G, int grid) {
  const long long U = static_cast<long long>(tiles) * G;
  const int per_cta = static_cast<int>((U + grid - 1) / grid);
  return per_cta < G ? per_cta : G;
}

template <int MT, int WB, bool ST, bool COMM>
int launch_kernel(const SkinnyParams& p, int grid, cudaStream_t st, int smem);

template <int MT, int WB, bool ST, bool COMM>
int launch_cfg(SkinnyParams& p, int grid, cudaStream_t st, int smem_optin) {
  constexpr int kStageBytes = Fmt<WB>::kStage;
  constexpr bool kStream = ST;
  const int groups = cache_groups_for(p.tiles, p.G, grid);
  const int limit = smem_optin;
  if constexpr (kStream) {
    // weight ring first (up to the configured depth), then the deepest digit ring that still fits
    static const int kTry[][2] = {{8, 8}, {8, 4}, {6, 4}, {4, 4}, {4, 2}, {2, 2}};
    int smem = 0;
    bool found = false;
    for (const auto& c : kTry) {
      if (c[0] > config().depth) continue;
      p.depth = c[0];
      p.bdepth = c[1];
      p.bshift = c[1] == 8 ? 3 : (c[1] == 4 ? 2 : 1);
      p.b_bytes = p.bdepth * kStepGroups * p.db_bytes;
      p.xs_bytes = (p.G * p.M * 8 + 15) & ~15;
      smem = total_smem<MT, ST>(p.depth, kStageBytes, p.b_bytes, p.xs_bytes, p.bdepth);
      if (smem <= limit) {
        found = true;
        break;
      }
    }
    if (!found)
      return fail(W4A16_EINVAL, "decode kernel needs %d bytes of shared memory for M = %d; the device offers %d", smem,
                  p.M, smem_optin);
    return launch_kernel<MT, WB, ST, COMM>(p, grid, st, smem);
  }
  p.b_bytes = groups * 384 * p.M + 256;
  p.xs_bytes = groups * MT * 8;
  p.bdepth = 0;
  p.bshift = 0;
  // The depth stays EVEN. The two unpack warps of a lane quarter take alternate steps, and a parity wait on
  // an mbarrier only tells the current phase from the previous one: with an odd depth a stage's consecutive
  // uses would belong to different warps, and a warp that runs ahead could take "the other warp's copy has
  // not landed yet" for "my copy has landed".
  p.depth = config().depth;
  int smem = total_smem<MT, ST>(p.depth, kStageBytes, p.b_bytes, p.xs_bytes, 0);
  while (smem > limit && p.depth > 2) {
    p.depth -= 2;
    smem = total_smem<MT, ST>(p.depth, kStageBytes, p.b_bytes, p.xs_bytes, 0);
  }
  if (smem > smem_optin)
    return fail(W4A16_EINVAL, "decode kernel needs %d bytes of shared memory for in_f = %d, M = %d; the device offers %d",
                smem, p.K, p.M, smem_optin);
  return launch_kernel<MT, WB, ST, COMM>(p, grid, st, smem);
}

template <int MT, int WB, bool ST, bool COMM>
int launch_kernel(const SkinnyParams& p, int grid, cudaStream_t st, int smem) {
  static int attr_set[64] = {};
  int dev = 0;
  W4_CUDA(cudaGetDevice(&dev));
  if (attr_set[dev & 63] < smem) {
    W4_CUDA(cudaFuncSetAttribute(k_skinny<MT, WB, ST, COMM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[dev & 63] = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (config().pdl && !p.ordered) ? 1 : 0;
  W4_CUDA(cudaLaunchKernelEx(&cfg, k_skinny<MT, WB, ST, COMM>, p));
  return W4A16_OK;
}

// M = 1: the digit rows of `groups` k groups (384 B + one pair per group) must fit beside a two-stage
// weight ring.
bool gemv_cache_fits(int groups, int stage_bytes, int smem_optin) {
  const int fixed = 2 * stage_bytes + kSide * kTileRows * 4 + kTable * 8 + 256 * 4 + kMailWords * 4 + 64 * 8 + 16 + 256;
  return groups * (384 + 8) <= smem_optin - fixed;
}

// The template instance that serves M tokens (sets as balanced as the instances allow), and through it the
// geometry the pre-pass has to write for: tokens per set, accumulator columns per set, rows of the B operand.
int instance_for(int M) {
  return M <= 2 ? M : (M <= 4 ? 4 : (M <= 6 ? 6 : (M <= 8 ? 8 : (M == 9 ? 9 : (M <= 12 ? 12 : (M <= 15 ? 15 : 16))))));
}
template <int MT>
void geometry_of(int& tm, int& cb, int& nrows) {
  tm = Geo<MT, true>::TM;
  cb = Geo<MT, true>::CB;
  nrows = Geo<MT, true>::N;
}
void set_geometry(int M, int& tm, int& cb, int& nrows) {
  switch (instance_for(M)) {
    case 1: geometry_of<1>(tm, cb, nrows); break;
    case 2: geometry_of<2>(tm, cb, nrows); break;
    case 4: geometry_of<4>(tm, cb, nrows); break;
    case 6: geometry_of<6>(tm, cb, nrows); break;
    case 8: geometry_of<8>(tm, cb, nrows); break;
    case 9: geometry_of<9>(tm, cb, nrows); break;
    case 12: geometry_of<12>(tm, cb, nrows); break;
    case 15: geometry_of<15>(tm, cb, nrows); break;
    default: geometry_of<16>(tm, cb, nrows); break;
  }
}
// pre-pass output: per k group the B operand's digit rows, [8 chunks of 16 k][at most 48 rows] 16 B; behind all
// groups' rows the table of (sum, 2^-p) pairs, G x M x 8 bytes (+ 16 so that a bulk copy of the rounded-up size
// stays inside)
size_t prepass_bytes(int G, int M) { return static_cast<size_t>(G) * (128 * 48 + 8 * M) + 16; }

// A validated layer in either weight format, as the launcher sees it.
struct LayerRef {
  const uint8_t* stream = nullptr;
  int out_f = 0, in_f = 0, num_groups = 0, wbits = 4;
};
int layer_of(LayerRef& L, const w4a16_weights_t* w) {
  if (int rc = check_weights(w)) return rc;
  L = LayerRef{reinterpret_cast<const uint8_t*>(w->qweight), w->out_f, w->in_f, w->num_groups, 4};
  return W4A16_OK;
}
int layer_of(LayerRef& L, const w4a16_w8_weights_t* w) {
  if (int rc = check_w8(w)) return rc;
  L = LayerRef{reinterpret_cast<const uint8_t*>(w->qweight), w->out_f, w->in_f, w->num_groups, 8};
  return W4A16_OK;
}

template <int WB, bool COMM>
int launch_batch_c(SkinnyParams& q, int grid, cudaStream_t st, int smem_optin) {
  switch (instance_for(q.M)) {
    case 1: return q.dig ? launch_cfg<1, WB, true, COMM>(q, grid, st, smem_optin)
                         : launch_cfg<1, WB, false, COMM>(q, grid, st, smem_optin);
    case 2: return launch_cfg<2, WB, true, COMM>(q, grid, st, smem_optin);    // token sets (1, 1)
    case 4: return launch_cfg<4, WB, true, COMM>(q, grid, st, smem_optin);    // (2, M - 2)
    case 6: return launch_cfg<6, WB, true, COMM>(q, grid, st, smem_optin);    // (3, M - 3)
    case 8: return launch_cfg<8, WB, true, COMM>(q, grid, st, smem_optin);    // (4, M - 4)
    case 9: return launch_cfg<9, WB, true, COMM>(q, grid, st, smem_optin);    // (3, 3, 3)
    case 12: return launch_cfg<12, WB, true, COMM>(q, grid, st, smem_optin);  // (4, 4, M - 8)
    case 15: return launch_cfg<15, WB, true, COMM>(q, grid, st, smem_optin);  // (5, 5, M - 10)
    default: return launch_cfg<16, WB, true, COMM>(q, grid, st, smem_optin);  // (8, 8)
  }
}
template <int WB>
int launch_batch(SkinnyParams& q, int grid, cudaStream_t st, int smem_optin) {
  return (q.comm_wait || q.comm_signal) ? launch_batch_c<WB, true>(q, grid, st, smem_optin)
                                         : launch_batch_c<WB, false>(q, grid, st, smem_optin);
}

int launch_skinny(SkinnyParams& p, const LayerRef* w, const uint16_t* x, int M, w4a16_scratch_t* s,
                  cudaStream_t st) {
  W4_REQUIRE(x != nullptr && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "x null or not 16-byte aligned");
  W4_REQUIRE(M >= 1 && M <= 16, "M = %d outside [1,16]", M);
  W4_REQUIRE(s != nullptr && s->xf && s->xgsum && s->partial, "scratch not allocated");
  W4_REQUIRE(w->num_groups <= 256, "in_f = %d is wider than the decode kernel supports (32768)", w->in_f);
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  p.ordered = take_weight_write(st) ? 1 : 0;
  const int TR = tile_rows();
  p.stream = w->stream;
  p.N = w->out_f;
  p.K = w->in_f;
  p.G = w->num_groups;
  p.tiles = (w->out_f + TR - 1) / TR;
  p.partial = s->partial;
  p.counters = reinterpret_cast<unsigned*>(s->xgsum);
  p.cta_pairs = s->xf;
  p.status = di->status;
  p.hint = static_cast<uint32_t>(config().hint);
  const int grid = grid_for_shape(w->out_f, w->num_groups, di->sms);
  W4_REQUIRE(static_cast<long long>(p.tiles) * p.G * (grid + 1) < (1LL << 32), "out_f x in_f too large for the decode kernel");
  auto magic = [](long long d) { return static_cast<unsigned long long>(((1LL << 40) + d - 1) / d); };
  p.mg_grid = magic(grid);
  p.mg_G = magic(p.G);
  if (int rc = w4a16_scratch_check(s, w->out_f, M)) return rc;
  p.M = M;
  p.x = x;
  const bool prepass = M >= 2 || p.ln_w != nullptr || (config().gemv_prepass && s->max_m >= 2 && p.G <= s->max_groups);
  if (!prepass) {
    if (!gemv_cache_fits(cache_groups_for(p.tiles, p.G, grid), w->wbits == 4 ? Fmt<4>::kStage : Fmt<8>::kStage,
                         di->smem_optin))
      return fail(W4A16_EINVAL, "in_f = %d is too wide for the decode kernel's activation cache", w->in_f);
  } else {
    // the pre-pass: digit rows of all M tokens, once per call, into the scratch (behind the argmax pairs)
    if (M > (s->max_m >= 2 ? s->max_m : 0) || p.G > s->max_groups)
      return fail(W4A16_ESCRATCH, "scratch: sized for max_m = %d and in_f <= %d, got M = %d, in_f = %d", s->max_m,
                  s->max_groups * kGroup, M, w->in_f);
    uint8_t* dig = reinterpret_cast<uint8_t*>(s->xf) + pair_bytes(s->max_splits);
    p.dig = dig;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.G * M + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    // the first launch of the call carries the ordering behind a weight write; the main kernel may then overlap
    // with this one as usual
    cfg.numAttrs = (config().pdl && !p.ordered) ? 1 : 0;
    p.ordered = 0;
    int tm = 1, cb = 8, nrows = 16;
    set_geometry(M, tm, cb, nrows);
    p.db_bytes = 128 * nrows;
    const unsigned* wait_block = p.comm_wait ? p.comm_local : nullptr;
    W4_CUDA(cudaLaunchKernelEx(&cfg, k_digits, x, dig, M, p.K, p.G, p.db_bytes, tm, cb, wait_block, p.comm_n, p.status,
                               p.ln_w, p.ln_eps, p.xn_out));
  }
  if (int rc = w->wbits == 4 ? launch_batch<4>(p, grid, st, di->smem_optin) : launch_batch<8>(p, grid, st, di->smem_optin))
    return rc;
  return W4A16_OK;
}

}  // namespace
}  // namespace w4a16

using namespace w4a16;

namespace {
template <class W>
int run_gemm(void* y, int y_is_f32, const W* w, const uint16_t* x, int M, w4a16_scratch_t* s, void* stream) {
  LayerRef L;
  if (int rc = layer_of(L, w)) return rc;
  SkinnyParams p = {};
  p.y = y;
  p.y_f32 = y_is_f32 ? 1 : 0;
  p.ldy = L.out_f;
  return launch_skinny(p, &L, x, M, s, static_cast<cudaStream_t>(stream));
}
// Validates a communicator and copies it into the launch parameters.
int set_comm(SkinnyParams& p, const w4a16_comm_t* comm, int wait_prev, int signal) {
  W4_REQUIRE(comm != nullptr, "null communicator");
  if (comm->nranks < 1 || comm->nranks > 8 || comm->rank < 0 || comm->rank >= comm->nranks)
    return fail(W4A16_ECOMM, "communicator: rank %d of %d (1..8 ranks)", comm->rank, comm->nranks);
  for (int r = 0; r < comm->nranks; ++r) {
    if (comm->blocks[r] == nullptr || (reinterpret_cast<uintptr_t>(comm->blocks[r]) & 15) != 0)
      return fail(W4A16_ECOMM, "communicator: flag block of rank %d is null or misaligned", r);
    p.comm_peers[r] = comm->blocks[r];
  }
  p.comm_local = comm->blocks[comm->rank];
  p.comm_n = comm->nranks;
  p.comm_rank = comm->rank;
  p.comm_wait = wait_prev ? 1 : 0;
  p.comm_signal = signal ? 1 : 0;
  return W4A16_OK;
}

template <class W>
int run_gather(uint16_t* const* y_peers, const w4a16_comm_t* comm, int wait_prev, int out_f_total, int row_begin,
               const W* w_shard, const uint16_t* x, int M, w4a16_scratch_t* s, void* stream) {
  W4_REQUIRE(y_peers != nullptr, "gemm_skinny_gather: null peer table");
  SkinnyParams p = {};
  if (int rc = set_comm(p, comm, wait_prev, 1)) return rc;
  LayerRef L;
  if (int rc = layer_of(L, w_shard)) return rc;
  if (row_begin < 0 || row_begin % kRowGranule != 0 || row_begin + L.out_f > out_f_total)
    return fail(W4A16_ECOMM, "gemm_skinny_gather: rows [%d,%d) outside [0,%d)", row_begin, row_begin + L.out_f,
                out_f_total);
  for (int r = 0; r < comm->nranks; ++r) W4_REQUIRE(y_peers[r] != nullptr, "gemm_skinny_gather: null peer %d", r);
  p.y = y_peers[comm->rank];
  p.ldy = out_f_total;
  p.y_col0 = row_begin;
  int q = 0;
  for (int r = 0; r < comm->nranks; ++r)
    if (r != comm->rank) p.y_peers[q++] = y_peers[r];
  p.npeers = q;
  return launch_skinny(p, &L, x, M, s, static_cast<cudaStream_t>(stream));
}

template <class W>
int run_argmax_sharded(int32_t* ids, void* const* pairs_peers, const w4a16_comm_t* comm, int wait_prev, int row_offset,
                       const W* w_shard, const uint16_t* x, int M, w4a16_scratch_t* s, void* stream) {
  W4_REQUIRE(ids != nullptr && pairs_peers != nullptr, "lm_head_argmax_sharded: null ids or pair tables");
  SkinnyParams p = {};
  if (int rc = set_comm(p, comm, wait_prev, 1)) return rc;
  LayerRef L;
  if (int rc = layer_of(L, w_shard)) return rc;
  for (int r = 0; r < comm->nranks; ++r) {
    W4_REQUIRE(pairs_peers[r] != nullptr && (reinterpret_cast<uintptr_t>(pairs_peers[r]) & 7) == 0,
               "lm_head_argmax_sharded: pair table of rank %d is null or misaligned", r);
    p.pairs_peers[r] = pairs_peers[r];
  }
  p.ldy = L.out_f;
  p.argmax = 1;
  p.ids = ids;
  p.row_offset = row_offset;
  return launch_skinny(p, &L, x, M, s, static_cast<cudaStream_t>(stream));
}

// The fused forms of a linear layer's neighbours (all optional, combinable): RMSNorm in front, SwiGLU or the
// residual add behind.
struct Fusion {
  const uint16_t* ln_w = nullptr;
  float ln_eps = 0.f;
  uint16_t* xn_out = nullptr;
  int epilogue = kEpiNone;
};
template <class W>
int run_fused(uint16_t* y, const W* w, const uint16_t* x, int M, const Fusion& f, w4a16_scratch_t* s, void* stream) {
  W4_REQUIRE(y != nullptr, "fused linear: y is null");
  LayerRef L;
  if (int rc = layer_of(L, w)) return rc;
  SkinnyParams p = {};
  p.y = y;
  p.ln_w = f.ln_w;
  p.ln_eps = f.ln_eps;
  p.xn_out = f.xn_out;
  p.epilogue = f.epilogue;
  if (f.ln_w) W4_REQUIRE((reinterpret_cast<uintptr_t>(f.ln_w) & 7) == 0, "fused linear: norm weights not 8-byte aligned");
  if (f.epilogue == kEpiSwiglu) {
    W4_REQUIRE(L.out_f % 32 == 0, "swiglu epilogue: out_f %d must be a multiple of 32 (gate, up interleaved)", L.out_f);
    p.ldy = L.out_f / 2;
  } else {
    p.ldy = L.out_f;
  }
  return launch_skinny(p, &L, x, M, s, static_cast<cudaStream_t>(stream));
}

template <class W>
int run_argmax(int32_t* ids, uint16_t* logits, void* pairs, int row_offset, const W* w, const uint16_t* x, int M,
               w4a16_scratch_t* s, void* stream) {
  W4_REQUIRE(ids != nullptr || pairs != nullptr, "lm_head_argmax: both ids and pairs are null");
  LayerRef L;
  if (int rc = layer_of(L, w)) return rc;
  SkinnyParams p = {};
  p.y = logits;
  p.ldy = L.out_f;
  p.argmax = 1;
  p.ids = ids;
  p.pairs_out = pairs;
  p.row_offset = row_offset;
  return launch_skinny(p, &L, x, M, s, static_cast<cudaStream_t>(stream));
}
}  // namespace

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

namespace {
// The array's name is only a host-side handle: the device address has to be asked for, once per device
// and with that device current. The first use on a device does this and clears the counters on `stream`.
// Guarded: two host threads may make their first call at the same time.
int static_scratch_base(unsigned char** out, int device, cudaStream_t stream) {
  static unsigned char* base[64] = {};
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  unsigned char* b = base[device & 63];
  if (!b) {
    void* p0 = nullptr;
    W4_CUDA(cudaGetSymbolAddress(&p0, g_static_scratch));
    b = static_cast<unsigned char*>(p0);
    W4_CUDA(cudaMemsetAsync(b + kStaticPartialBytes, 0, kStaticCounterBytes, stream));
    base[device & 63] = b;
  }
  *out = b;
  return W4A16_OK;
}
}  // namespace

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
  // two partial tiles per CTA (head and tail of its unit range), widest tile, 16 tokens, 8-byte (sum, tag) words
  s->partial_elems = static_cast<size_t>(s->max_splits) * 2 * kTileRows * 16 * 2;
  const size_t counters = counter_bytes(max_out);
  // per-CTA argmax pairs, then (max_m >= 2) the pre-pass output: digit rows of max_m tokens for every k group
  const size_t pairs = pair_bytes(s->max_splits) +
                       (max_m >= 2 ? prepass_bytes(s->max_groups, max_m > 16 ? 16 : max_m) : 0);
  void *xf = nullptr, *cn = nullptr, *pa = nullptr;
  cudaError_t e = cudaMalloc(&xf, pairs);
  if (e == cudaSuccess) e = cudaMalloc(&cn, counters);
  if (e == cudaSuccess) e = cudaMalloc(&pa, s->partial_elems * sizeof(float));
  if (e == cudaSuccess) e = cudaMemset(cn, 0, counters);
  if (e == cudaSuccess) e = cudaMemset(pa, 0, s->partial_elems * sizeof(float));  // no piece published yet
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
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  const int ctas = di->sms * kMaxCtasPerSm;
  const size_t need = static_cast<size_t>(ctas) * 2 * kTileRows * (M > 0 && M <= 16 ? M : 16) * 2;
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

int w4a16_scratch_reset(w4a16_scratch_t* s, void* stream) {
  W4_REQUIRE(s != nullptr && s->xgsum != nullptr, "scratch_reset: scratch not allocated");
  W4_CUDA(cudaMemsetAsync(s->xgsum, 0, counter_bytes(s->max_out), static_cast<cudaStream_t>(stream)));
  if (s->partial) W4_CUDA(cudaMemsetAsync(s->partial, 0, s->partial_elems * sizeof(float), static_cast<cudaStream_t>(stream)));
  return W4A16_OK;
}

int w4a16_gemv(void* y, int y_is_f32, const w4a16_weights_t* w, const uint16_t* x, w4a16_scratch_t* s,
               void* stream) {
  W4_REQUIRE(y != nullptr, "gemv: y is null");
  return run_gemm(y, y_is_f32, w, x, 1, s, stream);
}

int w4a16_gemm_skinny(uint16_t* y, const w4a16_weights_t* w, const uint16_t* x, int M, w4a16_scratch_t* s,
                      void* stream) {
  W4_REQUIRE(y != nullptr, "gemm_skinny: y is null");
  return run_gemm(y, 0, w, x, M, s, stream);
}

int w4a16_lm_head_argmax(int32_t* ids, uint16_t* logits, void* pairs, int row_offset, const w4a16_weights_t* w,
                         const uint16_t* x, int M, w4a16_scratch_t* s, void* stream) {
  return run_argmax(ids, logits, pairs, row_offset, w, x, M, s, stream);
}

int w4a16_w8_gemv(uint16_t* y, const w4a16_w8_weights_t* w, const uint16_t* x, w4a16_scratch_t* s, void* stream) {
  W4_REQUIRE(y != nullptr, "w8_gemv: y is null");
  return run_gemm(y, 0, w, x, 1, s, stream);
}

int w4a16_w8_gemm_skinny(uint16_t* y, const w4a16_w8_weights_t* w, const uint16_t* x, int M, w4a16_scratch_t* s,
                         void* stream) {
  W4_REQUIRE(y != nullptr, "w8_gemm_skinny: y is null");
  return run_gemm(y, 0, w, x, M, s, stream);
}

int w4a16_w8_lm_head_argmax(int32_t* ids, uint16_t* logits, void* pairs, int row_offset, const w4a16_w8_weights_t* w,
                            const uint16_t* x, int M, w4a16_scratch_t* s, void* stream) {
  return run_argmax(ids, logits, pairs, row_offset, w, x, M, s, stream);
}

int w4a16_argmax_pairs_reduce(int32_t* ids, const void* pairs, int nranks, int M, void* stream) {
  W4_REQUIRE(ids && pairs, "argmax_pairs_reduce: null pointer");
  W4_REQUIRE(nranks >= 1 && M >= 1 && M <= 16, "argmax_pairs_reduce: nranks %d, M %d", nranks, M);
  k_pairs_reduce<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ids, static_cast<const Pair*>(pairs), nranks, M);
  W4_CUDA(cudaGetLastError());
  return W4A16_OK;
}

int w4a16_gemv_static(void* y, int y_is_f32, const w4a16_weights_t* w, const uint16_t* x, void* stream) {
  W4_REQUIRE(y != nullptr, "gemv_static: y is null");
  W4_REQUIRE(w != nullptr, "gemv_static: null weights");
  W4_REQUIRE(w->out_f <= kStaticMaxOut, "gemv_static: out_f %d exceeds the static scratch limit of %d rows", w->out_f,
             kStaticMaxOut);
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  W4_REQUIRE(di->sms * kMaxCtasPerSm <= kStaticMaxCtas, "gemv_static: %d SMs exceed the static scratch limit of %d CTAs",
             di->sms, kStaticMaxCtas);
  // The first call on a device looks the array up (and clears its counters), so it should come before any
  // stream capture.
  unsigned char* b = nullptr;
  if (int rc = static_scratch_base(&b, di->device, static_cast<cudaStream_t>(stream))) return rc;
  w4a16_scratch_t s = {};
  s.partial = reinterpret_cast<float*>(b);
  s.xgsum = reinterpret_cast<float*>(b + kStaticPartialBytes);
  s.xf = reinterpret_cast<float*>(b + kStaticPartialBytes + kStaticCounterBytes);
  s.max_out = kStaticMaxOut;
  s.max_splits = kStaticMaxCtas;
  s.max_m = 1;
  s.partial_elems = kStaticPartialBytes / sizeof(float);
  return run_gemm(y, y_is_f32, w, x, 1, &s, stream);
}

int w4a16_gemv_static_reset(void* stream) {
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  unsigned char* b = nullptr;
  if (int rc = static_scratch_base(&b, di->device, static_cast<cudaStream_t>(stream))) return rc;
  W4_CUDA(cudaMemsetAsync(b, 0, kStaticPartialBytes + kStaticCounterBytes, static_cast<cudaStream_t>(stream)));
  return W4A16_OK;
}

int w4a16_gemm_skinny_gather(uint16_t* const* y_peers, const w4a16_comm_t* comm, int wait_prev, int out_f_total,
                             int row_begin, const w4a16_weights_t* w_shard, const uint16_t* x, int M, w4a16_scratch_t* s,
                             void* stream) {
  return run_gather(y_peers, comm, wait_prev, out_f_total, row_begin, w_shard, x, M, s, stream);
}

int w4a16_lm_head_argmax_sharded(int32_t* ids, void* const* pairs_peers, const w4a16_comm_t* comm, int wait_prev,
                                 int row_offset, const w4a16_weights_t* w_shard, const uint16_t* x, int M,
                                 w4a16_scratch_t* s, void* stream) {
  return run_argmax_sharded(ids, pairs_peers, comm, wait_prev, row_offset, w_shard, x, M, s, stream);
}

int w4a16_w8_lm_head_argmax_sharded(int32_t* ids, void* const* pairs_peers, const w4a16_comm_t* comm, int wait_prev,
                                    int row_offset, const w4a16_w8_weights_t* w_shard, const uint16_t* x, int M,
                                    w4a16_scratch_t* s, void* stream) {
  return run_argmax_sharded(ids, pairs_peers, comm, wait_prev, row_offset, w_shard, x, M, s, stream);
}

int w4a16_gemm_skinny_partial(float* const* partial_peers, const w4a16_comm_t* comm, const w4a16_weights_t* w_kshard,
                              const uint16_t* x_slice, int M, w4a16_scratch_t* s, void* stream) {
  W4_REQUIRE(partial_peers != nullptr, "gemm_skinny_partial: null buffer table");
  SkinnyParams p = {};
  if (int rc = set_comm(p, comm, 0, 1)) return rc;
  LayerRef L;
  if (int rc = layer_of(L, w_kshard)) return rc;
  W4_REQUIRE(M >= 1 && M <= 16, "gemm_skinny_partial: M = %d outside [1,16]", M);
  const size_t slot = static_cast<size_t>(comm->rank) * M * L.out_f;  // this rank's slot in every rank's buffer
  int q = 0;
  for (int r = 0; r < comm->nranks; ++r) {
    W4_REQUIRE(partial_peers[r] != nullptr, "gemm_skinny_partial: null buffer of rank %d", r);
    if (r == comm->rank) p.y = partial_peers[r] + slot;
    else p.y_peers[q++] = partial_peers[r] + slot;
  }
  p.npeers = q;
  p.y_f32 = 1;
  p.ldy = L.out_f;
  return launch_skinny(p, &L, x_slice, M, s, static_cast<cudaStream_t>(stream));
}

int w4a16_reduce_partials(uint16_t* y, const float* partials_local, const w4a16_comm_t* comm, int M, int out_f,
                          int residual, void* stream) {
  W4_REQUIRE(y != nullptr && partials_local != nullptr, "reduce_partials: null pointer");
  W4_REQUIRE(M >= 1 && out_f >= 1, "reduce_partials: M = %d, out_f = %d", M, out_f);
  SkinnyParams p = {};
  if (int rc = set_comm(p, comm, 1, 0)) return rc;
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  const long long n = static_cast<long long>(M) * out_f;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((n + 255) / 256));
  cfg.blockDim = dim3(256);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = config().pdl ? 1 : 0;
  W4_CUDA(cudaLaunchKernelEx(&cfg, k_reduce_partials, y, partials_local, comm->nranks, n, residual ? 1 : 0,
                             static_cast<const unsigned*>(p.comm_local), di->status));
  return W4A16_OK;
}

int w4a16_wait_gather(const w4a16_comm_t* comm, void* stream) {
  SkinnyParams p = {};
  if (int rc = set_comm(p, comm, 1, 0)) return rc;
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = config().pdl ? 1 : 0;
  W4_CUDA(cudaLaunchKernelEx(&cfg, k_wait_gather, static_cast<const unsigned*>(p.comm_local), p.comm_n, di->status));
  return W4A16_OK;
}

int w4a16_linear_fused(uint16_t* y, const w4a16_weights_t* w, const uint16_t* x, int M, const uint16_t* ln_weight,
                       float ln_eps, uint16_t* xn_out, int epilogue, w4a16_scratch_t* s, void* stream) {
  W4_REQUIRE(epilogue == W4A16_EPILOGUE_NONE || epilogue == W4A16_EPILOGUE_SWIGLU || epilogue == W4A16_EPILOGUE_RESIDUAL,
             "linear_fused: unknown epilogue %d", epilogue);
  Fusion f;
  f.ln_w = ln_weight;
  f.ln_eps = ln_eps;
  f.xn_out = xn_out;
  f.epilogue = epilogue;
  return run_fused(y, w, x, M, f, s, stream);
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
  LayerRef L;
  if (int rc = layer_of(L, w_shard)) return rc;
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
  return launch_skinny(p, &L, x, M, s, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
