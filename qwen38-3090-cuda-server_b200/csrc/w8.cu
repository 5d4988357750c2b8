// INT8 (W8A16) lm_head weights: the load-time quantiser into the private block layout,
// the container's free, and the row export that anchors bit-exactness of the format.
//
// Replaces quantize_w8a16 / k_quant_w8 and w8a16_free of the reference project
// (src/kernels/gemv_w4a16.cu:479-499,610-617). The launchers that multiply these weights
// (gemv_w8a16, gemm_small_w8a16) share the decode kernel and live in skinny.cu.
#include <cstring>

#include "common.cuh"

namespace w4a16 {
namespace {

// One warp per (row, group): lane l holds k = 4 l .. 4 l + 3 of the group's 128 values.
//   s = max|v| / 127 (stored rounded to bf16), q = clamp(rn(v * (127 / max|v|)), -127, 127)
// exactly as the reference's quantiser computes them (fp32 throughout, round to nearest even).
__global__ void k_quant_w8(uint8_t* __restrict__ dst, const uint16_t* __restrict__ src, int out_f, int in_f, int G) {
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(out_f) * G) return;
  const int g = static_cast<int>(wid % G);
  const int o = static_cast<int>(wid / G);
  const uint2 raw = *reinterpret_cast<const uint2*>(src + static_cast<size_t>(o) * in_f + g * kGroup + 4 * lane);
  const float v[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                      __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u)};
  float mx = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  const float s = mx / 127.0f;
  const float inv = (mx > 0.f) ? 127.0f / mx : 0.f;
  uint8_t* blk = dst + (static_cast<size_t>(o / kTileRows) * G + g) * kW8BlockBytes;
  const int r = o % kTileRows;
  if (lane == 0) reinterpret_cast<uint16_t*>(blk + kW8ScaleOff)[r] = float_to_bf16_bits(s);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int k = 4 * lane + i;
    int q = __float2int_rn(v[i] * inv);
    q = max(-127, min(127, q));
    const int j = (k & ~7) + w8_pos_of_k(k & 7);  // byte position inside the row's 128
    blk[(j >> 4) * kW8ChunkBytes + r * 16 + (j & 15)] = static_cast<uint8_t>(static_cast<int8_t>(q));
  }
}

// One thread per (row, k): plain row-major codes; one thread per (row, group): scales.
__global__ void k_w8_unpack_rows(int8_t* __restrict__ q, uint16_t* __restrict__ sc, const uint8_t* __restrict__ stream,
                                 int row0, int nrows, int K, int G) {
  const long long n = static_cast<long long>(nrows) * K;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int k = static_cast<int>(i % K);
    const int rr = static_cast<int>(i / K);
    const int o = row0 + rr, g = k / kGroup, kk = k % kGroup;
    const uint8_t* blk = stream + (static_cast<size_t>(o / kTileRows) * G + g) * kW8BlockBytes;
    const int r = o % kTileRows;
    const int j = (kk & ~7) + w8_pos_of_k(kk & 7);
    if (q) q[i] = static_cast<int8_t>(blk[(j >> 4) * kW8ChunkBytes + r * 16 + (j & 15)]);
    if (sc && kk == 0) sc[static_cast<size_t>(rr) * G + g] = reinterpret_cast<const uint16_t*>(blk + kW8ScaleOff)[r];
  }
}

}  // namespace

int check_w8(const w4a16_w8_weights_t* w) {
  W4_REQUIRE(w != nullptr, "w8 weights: null struct");
  W4_REQUIRE(w->qweight && w->scale, "w8 weights: null buffer");
  W4_REQUIRE(w->group_size == kGroup, "w8 weights: group_size %d unsupported (only 128)", w->group_size);
  W4_REQUIRE(w->out_f > 0 && w->out_f % kRowGranule == 0, "w8 weights: out_f %d not a positive multiple of 16",
             w->out_f);
  W4_REQUIRE(w->in_f > 0 && w->in_f % kGroup == 0, "w8 weights: in_f %d not a positive multiple of 128", w->in_f);
  W4_REQUIRE(w->num_groups == w->in_f / kGroup, "w8 weights: num_groups %d != in_f/128", w->num_groups);
  W4_REQUIRE((reinterpret_cast<uintptr_t>(w->qweight) & 15) == 0, "w8 weights: buffer must be 16-byte aligned");
  return W4A16_OK;
}

}  // namespace w4a16

using namespace w4a16;

extern "C" {

int w4a16_w8_quantize(w4a16_w8_weights_t* dst, const uint16_t* src, int out_f, int in_f, int group_size,
                      void* stream) {
  W4_REQUIRE(dst != nullptr, "w8_quantize: null struct");
  W4_REQUIRE(src != nullptr && (reinterpret_cast<uintptr_t>(src) & 7) == 0, "w8_quantize: src null or not 8-byte aligned");
  W4_REQUIRE(group_size == kGroup, "w8_quantize: group_size %d unsupported (only 128)", group_size);
  W4_REQUIRE(out_f > 0 && out_f % kRowGranule == 0, "w8_quantize: out_f %d not a positive multiple of 16", out_f);
  W4_REQUIRE(in_f > 0 && in_f % kGroup == 0, "w8_quantize: in_f %d not a positive multiple of 128", in_f);
  memset(dst, 0, sizeof *dst);
  const int G = in_f / kGroup;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t qb = w8_stream_bytes(out_f, G);
  void *q = nullptr, *s = nullptr;
  cudaError_t e = cudaMalloc(&q, qb);
  if (e == cudaSuccess) e = cudaMalloc(&s, 256);
  // rows of the last tile past out_f: zero codes and zero scales, ordered before the quantiser on its stream
  if (e == cudaSuccess && out_f % kTileRows != 0) e = cudaMemsetAsync(q, 0, qb, st);
  if (e != cudaSuccess) {
    cudaFree(q);
    cudaFree(s);
    return fail(W4A16_ECUDA, "w8_quantize(%d x %d): %s", out_f, in_f, cudaGetErrorString(e));
  }
  const long long threads = static_cast<long long>(out_f) * G * 32;
  k_quant_w8<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, st>>>(static_cast<uint8_t*>(q), src, out_f, in_f, G);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    cudaFree(q);
    cudaFree(s);
    return fail(W4A16_ECUDA, "w8_quantize: %s", cudaGetErrorString(e));
  }
  note_weight_write(st);
  dst->qweight = static_cast<int8_t*>(q);
  dst->scale = static_cast<uint16_t*>(s);
  dst->out_f = out_f;
  dst->in_f = in_f;
  dst->group_size = group_size;
  dst->num_groups = G;
  return W4A16_OK;
}

int w4a16_w8_free(w4a16_w8_weights_t* w) {
  W4_REQUIRE(w != nullptr, "w8_free: null struct");
  cudaFree(w->qweight);
  cudaFree(w->scale);
  memset(w, 0, sizeof *w);
  return W4A16_OK;
}

int w4a16_w8_unpack_rows(int8_t* q, uint16_t* scale, const w4a16_w8_weights_t* w, int row0, int nrows, void* stream) {
  if (int rc = check_w8(w)) return rc;
  W4_REQUIRE(q != nullptr || scale != nullptr, "w8_unpack_rows: both outputs are null");
  W4_REQUIRE(row0 >= 0 && nrows >= 0 && row0 + nrows <= w->out_f, "w8_unpack_rows: rows [%d,%d) outside [0,%d)", row0,
             row0 + nrows, w->out_f);
  if (nrows == 0) return W4A16_OK;
  const long long n = static_cast<long long>(nrows) * w->in_f;
  long long grid = (n + 255) / 256;
  if (grid > 65535 * 16) grid = 65535 * 16;
  k_w8_unpack_rows<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      q, scale, reinterpret_cast<const uint8_t*>(w->qweight), row0, nrows, w->in_f, w->num_groups);
  W4_CUDA(cudaGetLastError());
  return W4A16_OK;
}

}  // extern "C"
