// Weight container management for the W4A16 path: allocation, the load-time
// repack from the checkpoint's on-disk layout into the private block layout, and
// the row dequantiser that anchors bit-exactness on the GPU.
//
// Replaces awq_alloc_fused / awq_repack_into / awq_free
// (src/kernels/gemv_w4a16.cu:308-334 of the reference project) and
// w4a16_dequant_rows (src/kernels/gemm_w4a16.cu:15-38,56-61).
#include <cstring>
#include <atomic>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace w4a16 {

// ------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
  return code;
}

// ------------------------------------------------------------------ device info
constexpr int kMaxDevices = 64;
static DeviceInfo g_dev[kMaxDevices];
static std::mutex g_dev_mu;
static std::mutex g_ww_mu;
static std::vector<cudaStream_t> g_ww_streams;  // streams with a weight write no matmul call has followed yet
static std::atomic<int> g_ww_count{0};

__device__ int g_status_word = 0;

const DeviceInfo* device_info() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("no current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DeviceInfo& d = g_dev[dev];
  if (d.device != dev) {
    int sms = 0, smem = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
      set_error("cudaDeviceGetAttribute failed");
      return nullptr;
    }
    int* st = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&st), g_status_word) != cudaSuccess) {
      set_error("cudaGetSymbolAddress(status word) failed");
      return nullptr;
    }
    d.sms = sms;
    d.smem_optin = smem;
    d.status = st;
    d.device = dev;
  }
  return &d;
}

// ------------------------------------------------------------------ kernels
namespace {

// Physical row of logical row o: the identity, or - for a gate|up layer repacked for the fused SwiGLU epilogue
// (inter > 0) - gate row o at 2 o and up row o - inter at 2 (o - inter) + 1.
__device__ __forceinline__ int physical_row(int o, int inter) {
  return inter <= 0 ? o : (o < inter ? 2 * o : 2 * (o - inter) + 1);
}

// One thread per destination uint4: (row, 32-k chunk).
__global__ void k_repack_q(uint8_t* __restrict__ dst, const uint32_t* __restrict__ sq, int out_f,
                           int words_per_row, int G, int row_offset, int inter) {
  const int C = G * 4;  // 32-k chunks per row
  const long long n = static_cast<long long>(out_f) * C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int so = static_cast<int>(i % out_f);  // consecutive threads -> consecutive rows (coalesced stores)
    const int c = static_cast<int>(i / out_f);
    const uint4 src = *reinterpret_cast<const uint4*>(sq + static_cast<size_t>(so) * words_per_row + c * 4);
    const uint32_t in[4] = {src.x, src.y, src.z, src.w};
    uint32_t out[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      uint32_t o = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) o |= ((in[w] >> (4 * k)) & 0xFu) << (4 * nib_pos(k));
      out[w] = o;
    }
    const int o = physical_row(so + row_offset, inter);
    *reinterpret_cast<uint4*>(dst + tile_group_offset(o, c >> 2, G) + (c & 3) * kChunkBytes +
                              weight_slot(o % kTileRows, c & 3) * 16) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

__global__ void k_repack_sz(uint8_t* __restrict__ dst, const uint16_t* __restrict__ ss,
                            const uint32_t* __restrict__ sz, int out_f, int G, int row_offset, int inter) {
  const long long n = static_cast<long long>(out_f) * G;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i % G);
    const int so = static_cast<int>(i / G);
    const int o = physical_row(so + row_offset, inter);
    uint8_t* blk = dst + tile_group_offset(o, g, G);
    const int r = o % kTileRows;
    reinterpret_cast<uint16_t*>(blk + kTgScaleOff)[r] = ss[static_cast<size_t>(so) * G + g];
    const uint32_t zw = sz[static_cast<size_t>(so >> 3) * G + g];
    blk[kTgZpOff + r] = static_cast<uint8_t>((zw >> ((so & 7) * 4)) & 0xFu);
  }
}

// One thread per (row, 32-k chunk): 32 bf16 values out, 64 contiguous bytes.
__global__ void k_dequant_rows(uint16_t* __restrict__ dst, const uint8_t* __restrict__ stream, int row0,
                               int nrows, int K, int G) {
  const int C = K / 32;
  const long long n = static_cast<long long>(nrows) * C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % C);
    const int r = static_cast<int>(i / C);
    const int o = row0 + r;
    const int ro = o % kTileRows;
    const uint8_t* blk = stream + tile_group_offset(o, c >> 2, G);
    const uint4 q = *reinterpret_cast<const uint4*>(blk + (c & 3) * kChunkBytes + weight_slot(ro, c & 3) * 16);
    const float s = bf16_bits_to_float(reinterpret_cast<const uint16_t*>(blk + kTgScaleOff)[ro]);
    const float z = static_cast<float>(blk[kTgZpOff + ro]);
    const uint32_t in[4] = {q.x, q.y, q.z, q.w};
    uint4* d = reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * K + c * 32);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      uint16_t v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        v[k] = float_to_bf16_bits((static_cast<float>((in[w] >> (4 * nib_pos(k))) & 0xFu) - z) * s);
      d[w] = make_uint4(v[0] | (uint32_t(v[1]) << 16), v[2] | (uint32_t(v[3]) << 16),
                        v[4] | (uint32_t(v[5]) << 16), v[6] | (uint32_t(v[7]) << 16));
    }
  }
}

// A wait that nothing satisfies: the same bounded mbarrier wait the kernels use, on a barrier nobody
// arrives at. It gives up after `polls` tests, reports through the status word and the kernel returns.
__global__ void k_wait_timeout_selftest(int* status, uint32_t polls) {
  __shared__ uint64_t bar;
  const uint32_t bar_a = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(bar_a, 1);
    fence_mbar_init();
    if (!mbar_wait_bounded(bar_a, 0, polls)) atomicExch(status, W4A16_ETIMEOUT);
  }
}

int grid_for(long long n, int block) {
  long long g = (n + block - 1) / block;
  return static_cast<int>(g < 1 ? 1 : (g > 65535 * 16 ? 65535 * 16 : g));
}

}  // namespace

void note_weight_write(cudaStream_t st) {
  std::lock_guard<std::mutex> lk(g_ww_mu);
  for (cudaStream_t q : g_ww_streams)
    if (q == st) return;
  g_ww_streams.push_back(st);
  g_ww_count.store(static_cast<int>(g_ww_streams.size()), std::memory_order_release);
}
bool take_weight_write(cudaStream_t st) {
  if (g_ww_count.load(std::memory_order_relaxed) == 0) return false;
  std::lock_guard<std::mutex> lk(g_ww_mu);
  for (size_t i = 0; i < g_ww_streams.size(); ++i)
    if (g_ww_streams[i] == st) {
      g_ww_streams.erase(g_ww_streams.begin() + static_cast<long>(i));
      g_ww_count.store(static_cast<int>(g_ww_streams.size()), std::memory_order_release);
      return true;
    }
  return false;
}

int check_weights(const w4a16_weights_t* w) {
  W4_REQUIRE(w != nullptr, "weights: null struct");
  W4_REQUIRE(w->qweight && w->scale && w->zp, "weights: null buffer");
  W4_REQUIRE(w->group_size == kGroup, "weights: group_size %d unsupported (only 128)", w->group_size);
  W4_REQUIRE(w->out_f > 0 && w->out_f % kRowGranule == 0, "weights: out_f %d not a positive multiple of 16",
             w->out_f);
  W4_REQUIRE(w->in_f > 0 && w->in_f % kGroup == 0, "weights: in_f %d not a positive multiple of 128",
             w->in_f);
  W4_REQUIRE(w->num_groups == w->in_f / kGroup, "weights: num_groups %d != in_f/128", w->num_groups);
  W4_REQUIRE((reinterpret_cast<uintptr_t>(w->qweight) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(w->scale) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(w->zp) & 15) == 0,
             "weights: buffers must be 16-byte aligned");
  return W4A16_OK;
}

}  // namespace w4a16

using namespace w4a16;

extern "C" {

const char* w4a16_last_error(void) { return g_err; }

int w4a16_device_status(void) {
  int v = 0;
  W4_CUDA(cudaDeviceSynchronize());
  W4_CUDA(cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int)));
  if (v != 0) set_error("device status %d: a bounded device-side wait expired", v);
  return v;
}

int w4a16_device_status_clear(void) {
  const int zero = 0;
  W4_CUDA(cudaDeviceSynchronize());
  W4_CUDA(cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int)));
  return W4A16_OK;
}

int w4a16_selftest_wait_timeout(int polls, void* stream) {
  W4_REQUIRE(polls >= 1 && polls <= 4096, "selftest_wait_timeout: polls = %d outside [1,4096]", polls);
  const DeviceInfo* di = device_info();
  if (!di) return W4A16_ECUDA;
  k_wait_timeout_selftest<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(di->status, static_cast<uint32_t>(polls));
  W4_CUDA(cudaGetLastError());
  return W4A16_OK;
}

int w4a16_weights_alloc(w4a16_weights_t* w, int out_f, int in_f, int group_size, void* stream) {
  W4_REQUIRE(w != nullptr, "weights_alloc: null struct");
  W4_REQUIRE(group_size == kGroup, "weights_alloc: group_size %d unsupported (only 128)", group_size);
  W4_REQUIRE(out_f > 0 && out_f % kRowGranule == 0, "weights_alloc: out_f %d not a positive multiple of 16",
             out_f);
  W4_REQUIRE(in_f > 0 && in_f % kGroup == 0, "weights_alloc: in_f %d not a positive multiple of 128", in_f);
  memset(w, 0, sizeof *w);
  const int G = in_f / group_size;
  // The whole weight stream (int4 blocks with their scales and zero points interleaved per
  // 128-row x 128-k block) lives behind `qweight`; for out_f a multiple of 128 its size is exactly
  // the reference's total_bytes() = int4 + bf16 scales + one-byte zero points. `scale` and `zp` stay valid,
  // independently freeable allocations because the reference's callers cudaFree all three
  // pointers one by one (src/model/model.cu:111,204), but nothing is read through them.
  const size_t qb = stream_bytes(out_f, G);  // out_f rounded up to whole 128-row tiles
  const size_t sb = 256;
  const size_t zb = 256;
  void *q = nullptr, *s = nullptr, *z = nullptr;
  cudaError_t e = cudaMalloc(&q, qb);
  if (e == cudaSuccess) e = cudaMalloc(&s, sb);
  if (e == cudaSuccess) e = cudaMalloc(&z, zb);
  if (e != cudaSuccess) {
    cudaFree(q);
    cudaFree(s);
    cudaFree(z);
    return fail(W4A16_ECUDA, "weights_alloc(%d x %d): %s", out_f, in_f, cudaGetErrorString(e));
  }
  if (out_f % kTileRows != 0) {
    // rows of the last tile past out_f: zero scales, so they contribute nothing and are never stored.
    // On the caller's stream, so that it is ordered before the repack that follows on that stream.
    e = cudaMemsetAsync(q, 0, qb, static_cast<cudaStream_t>(stream));
    note_weight_write(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
      cudaFree(q);
      cudaFree(s);
      cudaFree(z);
      return fail(W4A16_ECUDA, "weights_alloc: %s", cudaGetErrorString(e));
    }
  }
  w->qweight = static_cast<uint32_t*>(q);
  w->scale = static_cast<uint16_t*>(s);
  w->zp = static_cast<uint8_t*>(z);
  w->out_f = out_f;
  w->in_f = in_f;
  w->group_size = group_size;
  w->num_groups = G;
  return W4A16_OK;
}

static int repack_rows(const w4a16_weights_t* w, int dst_row_offset, const uint32_t* packed, const uint16_t* scale,
                       const uint32_t* zp, int out_f, int inter, void* stream) {
  if (int rc = check_weights(w)) return rc;
  W4_REQUIRE(packed && scale && zp, "repack_into: null source tensor");
  W4_REQUIRE(out_f > 0 && out_f % kRowGranule == 0, "repack_into: out_f %d not a positive multiple of 16",
             out_f);
  W4_REQUIRE(dst_row_offset >= 0 && dst_row_offset % kRowGranule == 0,
             "repack_into: row offset %d not a multiple of 16", dst_row_offset);
  W4_REQUIRE(dst_row_offset + out_f <= w->out_f, "repack_into: rows [%d,%d) exceed out_f %d",
             dst_row_offset, dst_row_offset + out_f, w->out_f);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* stream_base = reinterpret_cast<uint8_t*>(w->qweight);
  const long long nq = static_cast<long long>(out_f) * (w->in_f / 32);
  k_repack_q<<<grid_for(nq, 256), 256, 0, st>>>(stream_base, packed, out_f, w->in_f / 8, w->num_groups,
                                                dst_row_offset, inter);
  const long long ns = static_cast<long long>(out_f) * w->num_groups;
  k_repack_sz<<<grid_for(ns, 256), 256, 0, st>>>(stream_base, scale, zp, out_f, w->num_groups, dst_row_offset, inter);
  W4_CUDA(cudaGetLastError());
  note_weight_write(st);
  return W4A16_OK;
}

int w4a16_repack_into(const w4a16_weights_t* w, int dst_row_offset, const uint32_t* packed,
                      const uint16_t* scale, const uint32_t* zp, int out_f, void* stream) {
  return repack_rows(w, dst_row_offset, packed, scale, zp, out_f, 0, stream);
}

int w4a16_repack_into_swiglu(const w4a16_weights_t* w, int dst_row_offset, const uint32_t* packed,
                             const uint16_t* scale, const uint32_t* zp, int out_f, int inter, void* stream) {
  W4_REQUIRE(w != nullptr && inter > 0 && 2 * inter == w->out_f,
             "repack_into_swiglu: inter = %d must be half of the container's rows", inter);
  return repack_rows(w, dst_row_offset, packed, scale, zp, out_f, inter, stream);
}

int w4a16_weights_free(w4a16_weights_t* w) {
  W4_REQUIRE(w != nullptr, "weights_free: null struct");
  cudaFree(w->qweight);
  cudaFree(w->scale);
  cudaFree(w->zp);
  memset(w, 0, sizeof *w);
  return W4A16_OK;
}

int w4a16_dequant_rows(uint16_t* dst, const w4a16_weights_t* w, int row0, int nrows, void* stream) {
  if (int rc = check_weights(w)) return rc;
  W4_REQUIRE(dst != nullptr && (reinterpret_cast<uintptr_t>(dst) & 15) == 0,
             "dequant_rows: dst null or not 16-byte aligned");
  W4_REQUIRE(row0 >= 0 && nrows >= 0 && row0 + nrows <= w->out_f, "dequant_rows: rows [%d,%d) outside [0,%d)",
             row0, row0 + nrows, w->out_f);
  if (nrows == 0) return W4A16_OK;
  const long long n = static_cast<long long>(nrows) * (w->in_f / 32);
  k_dequant_rows<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      dst, reinterpret_cast<const uint8_t*>(w->qweight), row0, nrows, w->in_f, w->num_groups);
  W4_CUDA(cudaGetLastError());
  return W4A16_OK;
}

}  // extern "C"
