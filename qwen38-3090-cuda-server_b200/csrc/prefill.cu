// Prefill W4A16 GEMM (placeholder until the tcgen05 kernel lands): workspace
// management only. gemm_prefill reports that it is not built yet.
#include <cstring>

#include "common.cuh"

using namespace w4a16;

extern "C" {

int w4a16_workspace_alloc(w4a16_workspace_t* ws, size_t bytes) {
  W4_REQUIRE(ws != nullptr, "workspace_alloc: null struct");
  memset(ws, 0, sizeof *ws);
  if (bytes < 4096) bytes = 4096;
  void* p = nullptr;
  W4_CUDA(cudaMalloc(&p, bytes));
  ws->wbuf = static_cast<uint16_t*>(p);
  ws->bytes = bytes;
  return W4A16_OK;
}

int w4a16_workspace_free(w4a16_workspace_t* ws) {
  W4_REQUIRE(ws != nullptr, "workspace_free: null struct");
  cudaFree(ws->wbuf);
  memset(ws, 0, sizeof *ws);
  return W4A16_OK;
}

int w4a16_gemm_prefill(uint16_t*, const w4a16_weights_t*, const uint16_t*, int, w4a16_workspace_t*, void*) {
  return fail(W4A16_EINVAL, "gemm_prefill: not built yet");
}

}  // extern "C"
