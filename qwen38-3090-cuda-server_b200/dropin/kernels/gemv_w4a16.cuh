// Drop-in replacement for src/kernels/gemv_w4a16.cuh of the reference server.
//
// Same namespace, struct fields and launcher signatures as the reference header
// (src/kernels/gemv_w4a16.cuh:50-60,64-69,85-90,94-110,124-135,148-166,187-188), so that
// src/model, src/spec, src/draft and the reference's own gates compile against it
// unchanged. Every launcher is a thin inline shim over the C ABI of
// libw4a16_b200.so (include/w4a16_b200.h); a non-zero status becomes the
// reference's print-to-stderr-and-abort behaviour (src/kernels/gemv_w4a16.cu:9-10).
//
// Differences a caller can observe:
//   * the three weight buffers stay independent cudaFree-able allocations, but the
//     whole weight stream lives behind `qweight`; `scale` and `zp` are placeholders;
//   * gemm_small_w4a16 and gemm_mma_w4a16 are the same kernel;
//   * lm_head_argmax_w4a16 / lm_head_argmax_w8a16 are new: GEMV / skinny GEMM with the argmax fused in;
//   * W8A16Weights keeps both pointers as independent allocations, the int8 stream lives behind `qweight`;
//   * group_size must be 128 (the only size the served checkpoint uses).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "w4a16_b200.h"

namespace qwen {

struct W4A16Weights {
  uint32_t*      qweight = nullptr;
  __nv_bfloat16* scale   = nullptr;
  uint8_t*       zp      = nullptr;
  int out_f = 0, in_f = 0, group_size = 0, num_groups = 0;

  size_t qweight_bytes() const { return size_t(out_f) * in_f / 8 * sizeof(uint32_t); }
  size_t scale_bytes()   const { return size_t(out_f) * num_groups * sizeof(__nv_bfloat16); }
  size_t zp_bytes()      const { return size_t(out_f) * num_groups; }
  size_t total_bytes()   const { return qweight_bytes() + scale_bytes() + zp_bytes(); }
};

struct GemvScratch {
  float* xf      = nullptr;   // per-CTA (max, index) pairs of the fused argmax
  float* xgsum   = nullptr;   // split-tile arrival tickets (zero between calls)
  float* partial = nullptr;   // split-K partial tiles
  int    max_in = 0, max_groups = 0, max_out = 0, max_splits = 0, max_m = 1;
  size_t partial_elems = 0;
  size_t bytes() const {
    return size_t(max_splits) * 16 * 8 + (size_t(max_out) / 128 + 2) * 48 + 32 + partial_elems * 4;
  }
};

namespace detail {
static_assert(sizeof(W4A16Weights) == sizeof(w4a16_weights_t), "W4A16Weights must mirror w4a16_weights_t");
static_assert(sizeof(GemvScratch) == sizeof(w4a16_scratch_t), "GemvScratch must mirror w4a16_scratch_t");
inline w4a16_weights_t* cw(W4A16Weights& w) { return reinterpret_cast<w4a16_weights_t*>(&w); }
inline const w4a16_weights_t* cw(const W4A16Weights& w) { return reinterpret_cast<const w4a16_weights_t*>(&w); }
inline w4a16_scratch_t* cs(GemvScratch& s) { return reinterpret_cast<w4a16_scratch_t*>(&s); }
inline void check(int rc, const char* what) {
  if (rc != 0) {
    fprintf(stderr, "%s: %s (status %d)\n", what, w4a16_last_error(), rc);
    abort();
  }
}
}  // namespace detail

inline void awq_alloc_fused(W4A16Weights& dst, int total_out_f, int in_f, int group_size,
                            cudaStream_t stream = 0) {
  detail::check(w4a16_weights_alloc(detail::cw(dst), total_out_f, in_f, group_size, stream), "awq_alloc_fused");
}
inline void awq_repack_into(W4A16Weights& dst, int dst_row_offset, const uint32_t* src_packed,
                            const __nv_bfloat16* src_scale, const uint32_t* src_zp, int out_f,
                            cudaStream_t stream = 0) {
  detail::check(w4a16_repack_into(detail::cw(dst), dst_row_offset, src_packed,
                                  reinterpret_cast<const uint16_t*>(src_scale), src_zp, out_f, stream),
                "awq_repack_into");
}
inline void awq_repack(W4A16Weights& dst, const uint32_t* src_packed, const __nv_bfloat16* src_scale,
                       const uint32_t* src_zp, int out_f, int in_f, int group_size,
                       cudaStream_t stream = 0) {
  awq_alloc_fused(dst, out_f, in_f, group_size, stream);
  awq_repack_into(dst, 0, src_packed, src_scale, src_zp, out_f, stream);
}
inline void awq_free(W4A16Weights& w) { detail::check(w4a16_weights_free(detail::cw(w)), "awq_free"); }

inline void gemv_scratch_alloc(GemvScratch& s, int max_in, int max_out, int min_group, int max_m = 1) {
  detail::check(w4a16_scratch_alloc(detail::cs(s), max_in, max_out, min_group, max_m), "gemv_scratch_alloc");
}
inline void gemv_scratch_free(GemvScratch& s) { detail::check(w4a16_scratch_free(detail::cs(s)), "gemv_scratch_free"); }
// Aborts with a readable message if the scratch cannot serve an out_f-row, M-token call.
inline void gemv_partial_check(const GemvScratch& s, int /*splits*/, int out_f, int M) {
  detail::check(w4a16_scratch_check(reinterpret_cast<const w4a16_scratch_t*>(&s), out_f, M), "gemv_partial_check");
}
inline size_t gemv_scratch_bytes_for_m(const GemvScratch& s, int /*max_m*/) { return s.bytes(); }

inline void gemm_small_w4a16(__nv_bfloat16* y, const W4A16Weights& w, const __nv_bfloat16* x, int M,
                             GemvScratch& s, cudaStream_t stream = 0) {
  detail::check(w4a16_gemm_skinny(reinterpret_cast<uint16_t*>(y), detail::cw(w),
                                  reinterpret_cast<const uint16_t*>(x), M, detail::cs(s), stream),
                "gemm_small_w4a16");
}
inline void gemm_mma_w4a16(__nv_bfloat16* y, const W4A16Weights& w, const __nv_bfloat16* x, int M,
                           GemvScratch& s, cudaStream_t stream = 0) {
  detail::check(w4a16_gemm_skinny(reinterpret_cast<uint16_t*>(y), detail::cw(w),
                                  reinterpret_cast<const uint16_t*>(x), M, detail::cs(s), stream),
                "gemm_mma_w4a16");
}
inline void gemv_w4a16(__nv_bfloat16* y, const W4A16Weights& w, const __nv_bfloat16* x, GemvScratch& s,
                       cudaStream_t stream = 0) {
  detail::check(w4a16_gemv(y, 0, detail::cw(w), reinterpret_cast<const uint16_t*>(x), detail::cs(s), stream),
                "gemv_w4a16");
}
inline void gemv_w4a16_f32(float* y, const W4A16Weights& w, const __nv_bfloat16* x, GemvScratch& s,
                           cudaStream_t stream = 0) {
  detail::check(w4a16_gemv(y, 1, detail::cw(w), reinterpret_cast<const uint16_t*>(x), detail::cs(s), stream),
                "gemv_w4a16_f32");
}
inline int gemv_choose_splits(int out_f, int num_groups) { return w4a16_choose_splits(out_f, num_groups); }

// New: lm_head GEMV / skinny GEMM with the argmax fused in. ids[m] is what
// gemv/gemm -> bf16 logits -> argmax_rows would return (src/kernels/elementwise.cu:129-150):
// the largest bf16-rounded logit of row m, lowest index on ties. `logits` may be null.
inline void lm_head_argmax_w4a16(int32_t* ids, const W4A16Weights& w, const __nv_bfloat16* x, int M,
                                 GemvScratch& s, __nv_bfloat16* logits = nullptr, cudaStream_t stream = 0) {
  detail::check(w4a16_lm_head_argmax(ids, reinterpret_cast<uint16_t*>(logits), nullptr, 0, detail::cw(w),
                                     reinterpret_cast<const uint16_t*>(x), M, detail::cs(s), stream),
                "lm_head_argmax_w4a16");
}

// ---- INT8 g128 lm_head (src/kernels/gemv_w4a16.cuh:148-166) ----
struct W8A16Weights {
  int8_t*        qweight = nullptr;   // private int8 stream (codes and scales per 128-row x 128-k block)
  __nv_bfloat16* scale   = nullptr;   // placeholder allocation: freed by the caller like the reference's
  int out_f = 0, in_f = 0, group_size = 0, num_groups = 0;
  size_t total_bytes() const {
    return size_t(out_f) * in_f + size_t(out_f) * num_groups * 2;
  }
};

namespace detail {
static_assert(sizeof(W8A16Weights) == sizeof(w4a16_w8_weights_t), "W8A16Weights must mirror w4a16_w8_weights_t");
inline w4a16_w8_weights_t* cw8(W8A16Weights& w) { return reinterpret_cast<w4a16_w8_weights_t*>(&w); }
inline const w4a16_w8_weights_t* cw8(const W8A16Weights& w) { return reinterpret_cast<const w4a16_w8_weights_t*>(&w); }
}  // namespace detail

inline void quantize_w8a16(W8A16Weights& dst, const __nv_bfloat16* src, int out_f, int in_f, int group_size,
                           cudaStream_t stream = 0) {
  detail::check(w4a16_w8_quantize(detail::cw8(dst), reinterpret_cast<const uint16_t*>(src), out_f, in_f, group_size,
                                  stream),
                "quantize_w8a16");
}
inline void gemv_w8a16(__nv_bfloat16* y, const W8A16Weights& w, const __nv_bfloat16* x, GemvScratch& s,
                       cudaStream_t stream = 0) {
  detail::check(w4a16_w8_gemv(reinterpret_cast<uint16_t*>(y), detail::cw8(w), reinterpret_cast<const uint16_t*>(x),
                              detail::cs(s), stream),
                "gemv_w8a16");
}
inline void gemm_small_w8a16(__nv_bfloat16* y, const W8A16Weights& w, const __nv_bfloat16* x, int M, GemvScratch& s,
                             cudaStream_t stream = 0) {
  detail::check(w4a16_w8_gemm_skinny(reinterpret_cast<uint16_t*>(y), detail::cw8(w),
                                     reinterpret_cast<const uint16_t*>(x), M, detail::cs(s), stream),
                "gemm_small_w8a16");
}
inline void w8a16_free(W8A16Weights& w) { detail::check(w4a16_w8_free(detail::cw8(w)), "w8a16_free"); }
// New: the INT8 lm_head with the argmax fused in (same contract as lm_head_argmax_w4a16).
inline void lm_head_argmax_w8a16(int32_t* ids, const W8A16Weights& w, const __nv_bfloat16* x, int M,
                                 GemvScratch& s, __nv_bfloat16* logits = nullptr, cudaStream_t stream = 0) {
  detail::check(w4a16_w8_lm_head_argmax(ids, reinterpret_cast<uint16_t*>(logits), nullptr, 0, detail::cw8(w),
                                        reinterpret_cast<const uint16_t*>(x), M, detail::cs(s), stream),
                "lm_head_argmax_w8a16");
}

}  // namespace qwen
