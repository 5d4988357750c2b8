// Shared host/device helpers for the sm_100a W4A16 kernels: error reporting for
// the C ABI, PTX wrappers (mbarrier, bulk async copy, cp.async, mma, programmatic
// dependent launch) and the private weight layout's index arithmetic.
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

// Validates a weight container (non-null 16-byte aligned buffers, supported shape).
int check_weights(const w4a16_weights_t* w);

// ------------------------------------------------------------------ layout
constexpr int kRowBlock = 16;   // rows per weight block
constexpr int kStepK = 64;      // k per weight block ("step")
constexpr int kGroup = 128;     // quantisation group along k
constexpr int kStepBytes = 512; // one 16x64 int4 block
// One "unit" of the weight stream = 16 rows x one 128-k group, everything a warp
// needs for it in one contiguous piece: two 512-byte int4 blocks, then the 16 bf16
// scales, then the 16 one-byte zero points. Scales and zero points are ordered
// r0,r8,r1,r9,...,r7,r15 so the lane that owns rows r and r+8 reads both with one load.
constexpr int kUnitScaleOff = 2 * kStepBytes;        // 1024
constexpr int kUnitZpOff = kUnitScaleOff + 32;       // 1056
constexpr int kUnitBytes = kUnitZpOff + 16;          // 1072
// The stream is ordered [row tile of 128 rows][group][16-row block within the tile], so the
// eight warps of a CTA working on one (tile, group) read 8576 contiguous bytes, consecutive
// groups follow each other, and a CTA's whole range of units is one sequential region.
constexpr int kTileBlocks = 8;                             // 16-row blocks per row tile
constexpr int kTileRows = kTileBlocks * kRowBlock;         // 128
constexpr int kTileGroupBytes = kTileBlocks * kUnitBytes;  // 8576

__host__ __device__ inline size_t stream_bytes(int out_f, int G) {
  return static_cast<size_t>((out_f + kTileRows - 1) / kTileRows) * G * kTileGroupBytes;
}
// byte offset of the unit holding output row `o`, group `g`
__host__ __device__ inline size_t unit_offset(int o, int g, int G) {
  return (static_cast<size_t>(o / kTileRows) * G + g) * kTileGroupBytes +
         static_cast<size_t>((o % kTileRows) / kRowBlock) * kUnitBytes;
}

// slot of row r (0..15) inside a unit's scale / zero-point arrays
__host__ __device__ inline int sz_pos(int r) { return (r & 7) * 2 + (r >> 3); }
// nibble position inside a packed word for k-offset c (0..7)
__host__ __device__ inline int nib_pos(int c) { return (c >> 1) + 4 * (c & 1); }

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
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls and returns false; never spins forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
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
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Programmatic dependent launch: wait until the grids this one depends on have
// completed and flushed (no-op when launched without the attribute) / allow the
// next grid in the stream to start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// D = A * B with a zero accumulator (starts an accumulation chain without clearing registers)
__device__ __forceinline__ void mma_bf16_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                    uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// packed bf16 subtract: exact for the small integers used here
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t h) {
  return __uint_as_float(static_cast<uint32_t>(h) << 16);
}
__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
#endif  // __CUDACC__

}  // namespace w4a16
