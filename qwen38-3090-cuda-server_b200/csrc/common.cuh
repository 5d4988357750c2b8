// Shared host/device helpers for the sm_100a W4A16 kernels: error reporting for
// the C ABI, PTX wrappers (mbarrier, bulk async copy, tcgen05 / tensor memory,
// programmatic dependent launch) and the private weight layout's index arithmetic.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/w4a16_b200.h"

namespace w4a16 {

// ------------------------------------------------------------------ host errors
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define W4_CUDA(expr)                                                                  \
  do {                                                                                 \
    cudaError_t e_ = (expr);                                                           \
    if (e_ != cudaSuccess)                                                             \
      return ::w4a16::fail(W4A16_ECUDA, "%s:%d %s: %s", __FILE__, __LINE__, #expr,     \
                           cudaGetErrorString(e_));                                    \
  } while (0)

#define W4_REQUIRE(cond, ...)                                     \
  do {                                                            \
    if (!(cond)) return ::w4a16::fail(W4A16_EINVAL, __VA_ARGS__); \
  } while (0)

struct DeviceInfo {
  int device = -1;
  int sms = 0;
  int smem_optin = 0;
  int* status = nullptr;  // device address of the sticky status word (0 ok / W4A16_ETIMEOUT)
};
// Cached per device; returns nullptr (and sets the error) on failure.
const DeviceInfo* device_info();

// The matmul kernels start fetching weights before griddepcontrol.wait, and only that wait guarantees that the
// stores of the kernel in front of them are visible. So every entry that writes weight buffers notes its
// stream, and the next matmul call on that stream is enqueued without the programmatic-serialisation
// attribute: fully ordered behind the write. take_weight_write is true once per noted stream; with no write
// pending it costs one relaxed atomic load.
void note_weight_write(cudaStream_t st);
bool take_weight_write(cudaStream_t st);

// Validates a weight container (non-null 16-byte aligned buffers, supported shape).
int check_weights(const w4a16_weights_t* w);

// ------------------------------------------------------------------ layout
// Private weight layout ("stream"), group size 128. The matrix is cut into row tiles of 128
// output rows; for every (row tile, k group) the stream holds one 8576-byte block:
//     [4 k-chunks of 32][128 slots] uint4  8192 B   packed int4; row r of chunk c sits in slot weight_slot(r, c)
//     [128 rows] bf16 scale                  256 B
//     [128 rows] u8 zero point (raw nibble)  128 B
// Blocks are ordered [row tile][group], so consecutive groups of a tile follow each other and
// a CTA's whole share of the matrix is one sequential region of memory.
// Inside a uint4, word i holds k = 32 c + 8 i .. +7 of its row; k-offset o sits at nibble
// (o>>1) + 4*(o&1), so the masks 0x000F000F << {0,4,8,12} pull out pairs of adjacent k.
constexpr int kGroup = 128;                               // quantisation group along k
constexpr int kRowGranule = 16;                           // out_f and row offsets are multiples of this
constexpr int kTileRows = 128;                            // output rows per row tile
constexpr int kChunkBytes = kTileRows * 16;               // 2048: one 32-k chunk of a tile
constexpr int kTgScaleOff = 4 * kChunkBytes;              // 8192
constexpr int kTgZpOff = kTgScaleOff + kTileRows * 2;     // 8448
constexpr int kTileGroupBytes = kTgZpOff + kTileRows;     // 8576

__host__ __device__ inline size_t stream_bytes(int out_f, int G) {
  return static_cast<size_t>((out_f + kTileRows - 1) / kTileRows) * G * kTileGroupBytes;
}
// byte offset of the block of (row tile of `o`, group g)
__host__ __device__ inline size_t tile_group_offset(int o, int g, int G) {
  return (static_cast<size_t>(o / kTileRows) * G + g) * kTileGroupBytes;
}
// 16-byte slot of row r (0..127) inside 32-k chunk c of a block: rows of odd chunks are rotated by
// four slots, so that a thread which reads 8 bytes of two neighbouring chunks (the mma.sync
// fragment pattern) and a thread which reads its own row's 16 bytes (the tcgen05 pattern) are
// both free of shared-memory bank conflicts.
__host__ __device__ inline int weight_slot(int r, int c) { return (r + 4 * (c & 1)) & (kTileRows - 1); }
// nibble position inside a packed word for k-offset c (0..7)
__host__ __device__ inline int nib_pos(int c) { return (c >> 1) + 4 * (c & 1); }

// INT8 stream (W8A16: symmetric int8, group 128, the lm_head variant). Same tiling; a block is 16640 bytes:
//     [8 chunks of 16 k-bytes][128 rows] 16 B   16384 B   byte j (0..127) of a row holds k = 8 (j/8) + w8_k_of(j%8)
//     [128 rows] bf16 scale                       256 B
// The k order inside every 8 is the order in which the int4 unpack (two nibble masks) delivers a packed
// word's weights, so both formats multiply the same activation operand.
constexpr int kW8ChunkBytes = kTileRows * 16;               // 2048
constexpr int kW8ScaleOff = 8 * kW8ChunkBytes;              // 16384
constexpr int kW8BlockBytes = kW8ScaleOff + kTileRows * 2;  // 16640
__host__ __device__ inline size_t w8_stream_bytes(int out_f, int G) {
  return static_cast<size_t>((out_f + kTileRows - 1) / kTileRows) * G * kW8BlockBytes;
}
// position (0..7) inside its 8-block of k-offset o, and back
__host__ __device__ inline int w8_pos_of_k(int o) { return (o & 3) * 2 + (o >> 2); }
__host__ __device__ inline int w8_k_of_pos(int j) { return (j >> 1) + 4 * (j & 1); }

// Validates an INT8 weight container.
int check_w8(const w4a16_w8_weights_t* w);

#ifdef __CUDACC__
// ------------------------------------------------------------------ device PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// One potentially-blocking test of the barrier's phase: the hardware may park the thread for up
// to `hint_ns` (it is woken when the phase completes), so a waiting warp does not burn issue slots.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns = 2000) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` tests (each may block for the hint time) and returns
// false; never spins forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// Same, for roles that are not latency critical: back off between polls so the spinning thread
// leaves the issue slots of its scheduler to the warps doing the math.
__device__ __forceinline__ bool mbar_wait_bounded_relaxed(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity, 10000)) return true;
    __nanosleep(200);
  }
  return false;
}
// 1-D bulk async copy global -> this CTA's shared memory, completion on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// ------------------------------------------------------------------ tcgen05 / tensor memory
// Allocation is warp-collective; the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 16 consecutive 32-bit columns of this thread's TMEM lane (lane = 32*(warp%4) + laneid)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&d)[N]);
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, float (&d)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]), "=f"(d[4]), "=f"(d[5]), "=f"(d[6]), "=f"(d[7]), "=f"(d[8]),
        "=f"(d[9]), "=f"(d[10]), "=f"(d[11]), "=f"(d[12]), "=f"(d[13]), "=f"(d[14]), "=f"(d[15])
      : "r"(taddr)
      : "memory");
}
// Shared-memory operand descriptor, K-major, no swizzle: 8-row x 16-byte core matrices;
// lbo = byte distance between core matrices along K, sbo = along the row (M/N) direction.
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((saddr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(lbo >> 4) << 16) |
         (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor for kind::f16 with bf16 A/B (both K-major), fp32 accumulate.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem desc]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Programmatic dependent launch: wait until the grids this one depends on have
// completed and flushed (no-op when launched without the attribute) / allow the
// next grid in the stream to start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// packed bf16 subtract: exact for the small integers used here
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// 64-bit words that carry a value and its "valid" tag together: one store makes both visible at once, so the
// reader needs no fence and the writer no flag.
__device__ __forceinline__ void st_relaxed_gpu_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// ---- cross-rank flags: one system-scope fence per CTA, relaxed adds into the peers' flag words, bounded polling ----
// A rank's block: words [0, 8) are counters written by the ranks (word r by rank r), word 16 is this rank's own
// count of signalling launches. Every signalling launch adds exactly kCommUnit to this rank's counter on every
// rank - each CTA its share, right after its own last store - so "every rank's slice of launch number s has
// landed" reads: counter[r] >= s * kCommUnit for every r. No CTA waits for another one.
// Release side: the CTA's stores, the CTA barrier, then ONE thread issues one fence.acq_rel.sys (cumulative over
// the stores it observed through the barrier) and the adds without waiting for any of them; a release per add
// would put one NVLink round trip per peer in series. Acquire side: the lanes of one warp poll one counter each
// with acquire loads (a fence after relaxed polls measured slower); the warp's vote and the barrier the caller
// releases the CTA with carry the order on to the other threads.
constexpr int kCommSeq = 16;                   // word of a rank's block
constexpr unsigned kCommUnit = 1u << 16;       // what one launch adds in total (more than any grid has CTAs)
constexpr uint32_t kFlagSpinLimit = 1u << 20;  // polls (each a system-scope load and a short sleep): about a second
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_relaxed_sys(unsigned* p, unsigned v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
// Waits until every rank's counter in this rank's block has reached launch number `seq`; false if the limit ran
// out. Called by the lanes of `mask` (converged, all of one warp) with the same arguments: lane number i of the
// mask polls counters i, i + |mask|, ...; the answer is the same on every lane.
__device__ __forceinline__ bool wait_flags(const unsigned* local, int n, unsigned seq, uint32_t limit,
                                           unsigned mask = 0xffffffffu) {
  const unsigned target = seq * kCommUnit;
  const int lanes = __popc(mask), me = __popc(mask & ((1u << (threadIdx.x & 31)) - 1u));
  bool ok = true;
  for (int r = me; r < n && ok; r += lanes) {
    uint32_t spins = 0;
    while (static_cast<int>(ld_acquire_sys(local + r) - target) < 0) {
      if (++spins > limit) {
        ok = false;
        break;
      }
      __nanosleep(32);
    }
  }
  return __all_sync(mask, ok);
}
// This rank's own count of signalling launches so far (the launch number the counters are compared with).
__device__ __forceinline__ unsigned comm_seq(const unsigned* local) {
  return *reinterpret_cast<const volatile unsigned*>(local + kCommSeq);
}
// Called by ONE thread of every CTA after the CTA-wide barrier that follows its last store: this CTA's share of
// the launch's signal goes to every rank (the local block included); CTA 0 also counts the launch.
__device__ __forceinline__ void signal_cta_done(unsigned* local, unsigned* const* peers, int n, int rank) {
  const unsigned share = blockIdx.x == 0 ? kCommUnit - (gridDim.x - 1) : 1u;
  fence_sys();
  for (int r = 0; r < n; ++r) red_add_relaxed_sys(peers[r] + rank, share);
  if (blockIdx.x == 0) atomicAdd(local + kCommSeq, 1u);
}
// The same for a launch whose exchange is done by a single thread of the grid (the vocab-sharded lm_head); the
// caller has fenced after the stores the signal covers.
__device__ __forceinline__ unsigned signal_whole_launch(unsigned* local, unsigned* const* peers, int n, int rank) {
  const unsigned seq = atomicAdd(local + kCommSeq, 1u) + 1u;
  fence_sys();
  for (int r = 0; r < n; ++r) red_add_relaxed_sys(peers[r] + rank, kCommUnit);
  return seq;
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t h) {
  return __uint_as_float(static_cast<uint32_t>(h) << 16);
}
__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
#endif  // __CUDACC__

}  // namespace w4a16
