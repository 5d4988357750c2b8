// Drop-in replacement for src/kernels/gemm_w4a16.cuh of the reference server
// (struct GemmWorkspace and the three launchers at src/kernels/gemm_w4a16.cuh:30-48).
// The prefill GEMM dequantises inside the tensor-core pipeline, so the workspace
// holds no bf16 weight tile and no cuBLAS handle is created; the fields stay so
// that callers which free `wbuf` themselves (src/model/model.cu:440-441) keep working.
#pragma once
#include "gemv_w4a16.cuh"

namespace qwen {

struct GemmWorkspace {
  __nv_bfloat16* wbuf = nullptr;
  size_t         bytes = 0;
  int            max_rows = 0;
  void*          cublas = nullptr;   // unused: kept for layout compatibility
};

namespace detail {
static_assert(sizeof(GemmWorkspace) == sizeof(w4a16_workspace_t), "GemmWorkspace must mirror w4a16_workspace_t");
inline w4a16_workspace_t* cws(GemmWorkspace& ws) { return reinterpret_cast<w4a16_workspace_t*>(&ws); }
}  // namespace detail

inline void gemm_workspace_alloc(GemmWorkspace& ws, size_t bytes) {
  detail::check(w4a16_workspace_alloc(detail::cws(ws), bytes), "gemm_workspace_alloc");
}
inline void gemm_workspace_free(GemmWorkspace& ws) {
  detail::check(w4a16_workspace_free(detail::cws(ws)), "gemm_workspace_free");
}
// C[M, out_f] = A[M, in_f] @ W^T, all row-major, A and C bf16, fp32 accumulate.
inline void gemm_w4a16(__nv_bfloat16* C, const W4A16Weights& w, const __nv_bfloat16* A, int M,
                       GemmWorkspace& ws, cudaStream_t stream = 0) {
  detail::check(w4a16_gemm_prefill(reinterpret_cast<uint16_t*>(C), detail::cw(w),
                                   reinterpret_cast<const uint16_t*>(A), M, detail::cws(ws), stream),
                "gemm_w4a16");
}
// Rows [row0,row0+nrows) of the weights as a plain row-major bf16 matrix.
inline void w4a16_dequant_rows(__nv_bfloat16* dst, const W4A16Weights& w, int row0, int nrows,
                               cudaStream_t stream = 0) {
  detail::check(::w4a16_dequant_rows(reinterpret_cast<uint16_t*>(dst), detail::cw(w), row0, nrows, stream),
                "w4a16_dequant_rows");
}

}  // namespace qwen
