// Thin C-ABI wrapper that compiles the reference project's own host header
// (src/loader/w4a16_unpack.h) unchanged, from where it lies, so the oracle's
// restatement can be checked against the real thing. Built only where the
// reference checkout is present; the output goes to oracle/_ref/ and is never
// part of the product. No reference source is copied: the header is included
// by path (-I<reference root>).
#include <cstdint>
#include "src/loader/w4a16_unpack.h"

extern "C" {

__attribute__((visibility("default")))
void ref_unpack_q(const uint32_t* packed, int64_t N, int64_t K, int8_t* out) {
  for (int64_t o = 0; o < N; ++o)
    for (int64_t i = 0; i < K; ++i) out[o * K + i] = int8_t(qwen::w4_q(packed, K, o, i));
}

__attribute__((visibility("default")))
void ref_unpack_zp(const uint32_t* zp, int64_t N, int64_t G, int8_t* out) {
  for (int64_t o = 0; o < N; ++o)
    for (int64_t g = 0; g < G; ++g) out[o * G + g] = int8_t(qwen::w4_zp(zp, G, o, g));
}

// float(q - zp) * bf16_to_f32(scale), the expression tests/gate_dequant.cpp:70-77 checks.
__attribute__((visibility("default")))
void ref_dequant_f32(const uint32_t* packed, const uint16_t* scale, const uint32_t* zp,
                     int64_t N, int64_t K, int64_t group, float* out) {
  const int64_t G = K / group;
  for (int64_t o = 0; o < N; ++o)
    for (int64_t i = 0; i < K; ++i) {
      const int64_t g = i / group;
      uint32_t u = uint32_t(scale[o * G + g]) << 16;
      float s;
      __builtin_memcpy(&s, &u, 4);
      out[o * K + i] = float(qwen::w4_q(packed, K, o, i) - qwen::w4_zp(zp, G, o, g)) * s;
    }
}

}  // extern "C"
