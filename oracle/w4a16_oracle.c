/*
 * CPU oracle for the W4A16 (AWQ int4, group-quantised) matmul path.
 *
 * THIS IS TEST INFRASTRUCTURE. It is a plain-C restatement of the arithmetic
 * the reference server defines for this path, used only as the checker in
 * tests, in the smoke run and as the timed CPU baseline of the benchmark.
 * The product never calls it.
 *
 * Parity is pinned: the restatement is checked bit for bit against
 *   - the reference's own header src/loader/w4a16_unpack.h compiled as is,
 *   - the reference's dequant fixtures tests/fixtures/dequant (7 tensors),
 *   - compressed_tensors' pack_to_int32 / unpack_from_int32.
 *
 * Reference lines each function follows (paths inside the reference project):
 *   nibble order, w4_q, w4_zp ........ src/loader/w4a16_unpack.h:25-42
 *   fp32 dequant (q-zp)*s ............ tests/gate_dequant.cpp:70-77
 *   bf16 dequant, rounded once ....... src/kernels/gemm_w4a16.cu:26-36
 *   fp64 GEMV / GEMM check loop ...... tests/gate_gemv.cu:96-114, tests/gate_gemm.cu:73-90
 *   bf16 round-to-nearest-even ....... tests/gate_gemv.cu:24-29
 *   argmax, ties to lowest index ..... src/spec/spec.cu:128-136, src/kernels/elementwise.cu:129-150
 *   min/max int4 quantiser ........... src/model/model.cu:140-172
 *   symmetric int8 quantiser ......... src/kernels/gemv_w4a16.cu:479-499
 *   int8 GEMV / GEMM (s * sum q x) ... src/kernels/gemv_w4a16.cu:501-523,525-568
 *   rmsnorm, residual_add, swiglu .... src/kernels/elementwise.cu:8-49,162-171
 *
 * On-disk ("compressed-tensors pack-quantized") layout, all little endian:
 *   packed [N][K/8] u32 : element i of a row is bits [4(i%8), 4(i%8)+4) of word i/8
 *   scale  [N][G]   bf16
 *   zp     [N/8][G] u32 : row o, group g is nibble (o%8) of word [o/8][g]
 * The stored nibble is value+8 for both q and zp, so w = (q_nib - zp_nib) * s.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even; NaN stays NaN (quiet) */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t r = (u >> 16) & 1u;
  return (uint16_t)((u + 0x7fffu + r) >> 16);
}

static inline int32_t nib(const uint32_t* words, int64_t e) {
  return (int32_t)((words[e >> 3] >> ((e & 7) * 4)) & 0xFu) - 8;
}
static inline int32_t q_at(const uint32_t* packed, int64_t K, int64_t o, int64_t i) {
  return nib(packed + o * (K >> 3), i);
}
static inline int32_t zp_at(const uint32_t* zp, int64_t G, int64_t o, int64_t g) {
  return (int32_t)((zp[(o >> 3) * G + g] >> ((o & 7) * 4)) & 0xFu) - 8;
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Thread count of the timed baseline; a launcher may have exported OMP_NUM_THREADS=1. */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORACLE_API void oracle_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]);
}
ORACLE_API void oracle_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}

/* signed codes in [-8,7] */
ORACLE_API void oracle_unpack_q(const uint32_t* packed, int64_t N, int64_t K, int8_t* out) {
  for (int64_t o = 0; o < N; ++o)
    for (int64_t i = 0; i < K; ++i) out[o * K + i] = (int8_t)q_at(packed, K, o, i);
}
ORACLE_API void oracle_unpack_zp(const uint32_t* zp, int64_t N, int64_t G, int8_t* out) {
  for (int64_t o = 0; o < N; ++o)
    for (int64_t g = 0; g < G; ++g) out[o * G + g] = (int8_t)zp_at(zp, G, o, g);
}

/* rows [row0,row0+nrows) -> fp32 [nrows][K]:  float(q-zp) * float(scale) */
ORACLE_API void oracle_dequant_f32(const uint32_t* packed, const uint16_t* scale,
                                   const uint32_t* zp, int64_t N, int64_t K, int64_t group,
                                   int64_t row0, int64_t nrows, float* out) {
  (void)N;
  const int64_t G = K / group;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < nrows; ++r) {
    const int64_t o = row0 + r;
    for (int64_t i = 0; i < K; ++i) {
      const int64_t g = i / group;
      const float s = bf16_to_f32(scale[o * G + g]);
      out[r * K + i] = (float)(q_at(packed, K, o, i) - zp_at(zp, G, o, g)) * s;
    }
  }
}

/* the same value rounded once to bf16 */
ORACLE_API void oracle_dequant_bf16(const uint32_t* packed, const uint16_t* scale,
                                    const uint32_t* zp, int64_t N, int64_t K, int64_t group,
                                    int64_t row0, int64_t nrows, uint16_t* out) {
  (void)N;
  const int64_t G = K / group;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < nrows; ++r) {
    const int64_t o = row0 + r;
    for (int64_t i = 0; i < K; ++i) {
      const int64_t g = i / group;
      const float s = bf16_to_f32(scale[o * G + g]);
      out[r * K + i] = f32_to_bf16((float)(q_at(packed, K, o, i) - zp_at(zp, G, o, g)) * s);
    }
  }
}

/* Y[M][N] (fp64) = X[M][K] * W^T with every term double(q-zp)*double(s)*double(x),
 * accumulated in fp64 in ascending k: the parity reference.
 * rows == NULL: all N rows; else only the nrows listed rows, out is [M][nrows]. */
ORACLE_API void oracle_gemm_f64(const uint32_t* packed, const uint16_t* scale, const uint32_t* zp,
                                int64_t N, int64_t K, int64_t group, const uint16_t* x,
                                int64_t M, const int64_t* rows, int64_t nrows, double* out) {
  const int64_t G = K / group;
  const int64_t R = rows ? nrows : N;
#pragma omp parallel
  {
    double* w = (double*)malloc(sizeof(double) * (size_t)K);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < R; ++r) {
      const int64_t o = rows ? rows[r] : r;
      for (int64_t i = 0; i < K; ++i) {
        const int64_t g = i / group;
        w[i] = (double)(q_at(packed, K, o, i) - zp_at(zp, G, o, g)) *
               (double)bf16_to_f32(scale[o * G + g]);
      }
      for (int64_t m = 0; m < M; ++m) {
        const uint16_t* xm = x + m * K;
        double acc = 0.0;
        for (int64_t i = 0; i < K; ++i) acc += w[i] * (double)bf16_to_f32(xm[i]);
        out[m * R + r] = acc;
      }
    }
    free(w);
  }
}

/* Dequant-then-fp32-matmul: the weight row is expanded to fp32 (q-zp)*s, then
 * dotted with each activation row in fp32. Sixteen fixed partial sums (k mod 16)
 * are combined in a fixed tree, so the result does not depend on thread count.
 * This is the timed CPU baseline. out is fp32 [M][N]. */
ORACLE_API void oracle_gemm_f32(const uint32_t* packed, const uint16_t* scale, const uint32_t* zp,
                                int64_t N, int64_t K, int64_t group, const uint16_t* x,
                                int64_t M, float* out) {
  const int64_t G = K / group;
  float* xf = (float*)malloc(sizeof(float) * (size_t)(M * K));
  for (int64_t i = 0; i < M * K; ++i) xf[i] = bf16_to_f32(x[i]);
#pragma omp parallel
  {
    float* w = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
    for (int64_t o = 0; o < N; ++o) {
      const uint32_t* pw = packed + o * (K >> 3);
      for (int64_t g = 0; g < G; ++g) {
        const float s = bf16_to_f32(scale[o * G + g]);
        const int32_t z = zp_at(zp, G, o, g);
        for (int64_t t = g * group / 8; t < (g + 1) * group / 8; ++t) {
          const uint32_t word = pw[t];
          for (int p = 0; p < 8; ++p)
            w[t * 8 + p] = (float)((int32_t)((word >> (4 * p)) & 0xFu) - 8 - z) * s;
        }
      }
      for (int64_t m = 0; m < M; ++m) {
        const float* xm = xf + m * K;
        float a[16];
        for (int j = 0; j < 16; ++j) a[j] = 0.f;
        for (int64_t i = 0; i < K; i += 16)
          for (int j = 0; j < 16; ++j) a[j] += w[i + j] * xm[i + j];
        for (int j = 0; j < 8; ++j) a[j] += a[j + 8];
        for (int j = 0; j < 4; ++j) a[j] += a[j + 4];
        out[m * N + o] = (a[0] + a[2]) + (a[1] + a[3]);
      }
    }
    free(w);
  }
  free(xf);
}

/* ids[m] = argmax over n of bf16 logits[m][n]; strict '>' keeps the lowest index.
 * A NaN logit never wins (comparison false), as in the reference. */
ORACLE_API void oracle_argmax_bf16(const uint16_t* logits, int64_t M, int64_t N, int32_t* ids) {
  for (int64_t m = 0; m < M; ++m) {
    float best = -3.402823466e+38f;
    int32_t bi = 0;
    for (int64_t n = 0; n < N; ++n) {
      const float v = bf16_to_f32(logits[m * N + n]);
      if (v > best) { best = v; bi = (int32_t)n; }
    }
    ids[m] = bi;
  }
}

/* lm_head with argmax: logits = bf16(fp64-accumulated dot), ids as above.
 * Also returns the bf16 logits (may be NULL) and, per row, the gap between the
 * best and second-best logit in bf16 ulps of the best (gap_ulps, may be NULL),
 * so a test can tell a real mismatch from a tie. */
ORACLE_API void oracle_lm_head_argmax(const uint32_t* packed, const uint16_t* scale,
                                      const uint32_t* zp, int64_t N, int64_t K, int64_t group,
                                      const uint16_t* x, int64_t M, int32_t* ids,
                                      uint16_t* logits_out, double* gap_ulps) {
  double* y = (double*)malloc(sizeof(double) * (size_t)(M * N));
  uint16_t* lg = logits_out ? logits_out : (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(M * N));
  oracle_gemm_f64(packed, scale, zp, N, K, group, x, M, NULL, 0, y);
  for (int64_t i = 0; i < M * N; ++i) lg[i] = f32_to_bf16((float)y[i]);
  oracle_argmax_bf16(lg, M, N, ids);
  if (gap_ulps) {
    for (int64_t m = 0; m < M; ++m) {
      const float best = bf16_to_f32(lg[m * N + ids[m]]);
      float second = -3.402823466e+38f;
      for (int64_t n = 0; n < N; ++n)
        if (n != ids[m]) { const float v = bf16_to_f32(lg[m * N + n]); if (v > second) second = v; }
      int e;
      frexpf(fabsf(best) > 0.f ? fabsf(best) : 1e-30f, &e);
      const double ulp = ldexp(1.0, e - 8); /* bf16: 8 significant bits */
      gap_ulps[m] = ((double)best - (double)second) / ulp;
    }
  }
  if (!logits_out) free(lg);
  free(y);
}

/* Asymmetric min/max int4 quantiser of a bf16 [rows][cols] matrix into the
 * on-disk layout: s=(hi-lo)/15 (1e-8 if not >0), z=clamp(rn(-lo/s),0,15),
 * q=clamp(rn(v*(1/s))+z,0,15). zp must be zero-filled by the caller (it is OR-ed). */
ORACLE_API void oracle_quant_i4(const uint16_t* src, int64_t rows, int64_t cols, int64_t group,
                                uint32_t* packed, uint16_t* scale, uint32_t* zp) {
  const int64_t G = cols / group;
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t g = 0; g < G; ++g) {
      const int64_t base = r * cols + g * group;
      float lo = 1e30f, hi = -1e30f;
      for (int64_t i = 0; i < group; ++i) {
        const float v = bf16_to_f32(src[base + i]);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
      }
      float s = (hi - lo) / 15.0f;
      if (!(s > 0.f)) s = 1e-8f;
      int z = (int)nearbyintf(-lo / s);
      z = z < 0 ? 0 : (z > 15 ? 15 : z);
      scale[r * G + g] = f32_to_bf16(s);
      zp[(r >> 3) * G + g] |= (uint32_t)z << ((r & 7) * 4);
      const float inv = 1.0f / s;
      for (int64_t i = 0; i < group; i += 8) {
        uint32_t w = 0;
        for (int k = 0; k < 8; ++k) {
          int q = (int)nearbyintf(bf16_to_f32(src[base + i + k]) * inv) + z;
          q = q < 0 ? 0 : (q > 15 ? 15 : q);
          w |= (uint32_t)q << (4 * k);
        }
        packed[r * (cols / 8) + (g * group + i) / 8] = w;
      }
    }
  }
}

/* ---- INT8 g128 symmetric lm_head variant (W8A16) ----
 * Quantiser: per (row, group) mx = max|v|, s = mx/127 stored as bf16, inv = mx>0 ? 127/mx : 0,
 * q = clamp(rn(v*inv), -127, 127); fp32 throughout. q is plain row-major int8 [rows][cols],
 * scale bf16 [rows][G] (the reference's 32-row interleave is a private layout, not part of
 * the arithmetic). */
ORACLE_API void oracle_quant_w8(const uint16_t* src, int64_t rows, int64_t cols, int64_t group,
                                int8_t* q, uint16_t* scale) {
  const int64_t G = cols / group;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t g = 0; g < G; ++g) {
      const int64_t base = r * cols + g * group;
      float mx = 0.f;
      for (int64_t i = 0; i < group; ++i) mx = fmaxf(mx, fabsf(bf16_to_f32(src[base + i])));
      const float s = mx / 127.0f;
      const float inv = (mx > 0.f) ? 127.0f / mx : 0.f;
      scale[r * G + g] = f32_to_bf16(s);
      for (int64_t i = 0; i < group; ++i) {
        int v = (int)nearbyintf(bf16_to_f32(src[base + i]) * inv);
        v = v < -127 ? -127 : (v > 127 ? 127 : v);
        q[base + i] = (int8_t)v;
      }
    }
  }
}

/* Y[M][N] (fp64) = X[M][K] * W^T with W = double(q) * double(bf16 scale), ascending k.
 * rows == NULL: all N rows; else only the listed rows, out is [M][nrows]. */
ORACLE_API void oracle_gemm_w8_f64(const int8_t* q, const uint16_t* scale, int64_t N, int64_t K,
                                   int64_t group, const uint16_t* x, int64_t M, const int64_t* rows,
                                   int64_t nrows, double* out) {
  const int64_t G = K / group;
  const int64_t R = rows ? nrows : N;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < R; ++r) {
    const int64_t o = rows ? rows[r] : r;
    for (int64_t m = 0; m < M; ++m) {
      const uint16_t* xm = x + m * K;
      double acc = 0.0;
      for (int64_t g = 0; g < G; ++g) {
        const double s = (double)bf16_to_f32(scale[o * G + g]);
        for (int64_t i = g * group; i < (g + 1) * group; ++i)
          acc += (double)q[o * K + i] * s * (double)bf16_to_f32(xm[i]);
      }
      out[m * R + r] = acc;
    }
  }
}

/* ---- the elementwise neighbours of a linear layer (fp32 arithmetic, bf16 in and out) ----
 * rmsnorm: 256 threads per row; thread t sums x[i]^2 over i = t, t+256, ... in fp32, a shuffle tree adds
 * the 32 lanes of a warp (offsets 16, 8, 4, 2, 1), thread 0 adds the 8 warp sums in order;
 * inv = rsqrt(sum / dim + eps); out = bf16(x * inv * (1 + w)). The summation order is restated exactly;
 * rsqrtf is the correctly rounded 1/sqrt here (the device instruction may differ in the last place). */
ORACLE_API void oracle_rmsnorm(const uint16_t* x, const uint16_t* w, int64_t rows, int64_t dim, float eps,
                               uint16_t* out) {
  for (int64_t r = 0; r < rows; ++r) {
    const uint16_t* xr = x + r * dim;
    float part[256];
    for (int t = 0; t < 256; ++t) {
      float a = 0.f;
      for (int64_t i = t; i < dim; i += 256) {
        const float v = bf16_to_f32(xr[i]);
        a += v * v;
      }
      part[t] = a;
    }
    float warp[8];
    for (int wv = 0; wv < 8; ++wv) {
      float l[32];
      for (int j = 0; j < 32; ++j) l[j] = part[wv * 32 + j];
      for (int sft = 16; sft > 0; sft >>= 1)
        for (int j = 0; j < 32; ++j) l[j] = l[j] + (j + sft < 32 ? l[j + sft] : l[j]);  /* shfl_down: lane 0 is exact */
      warp[wv] = l[0];
    }
    float t = 0.f;
    for (int wv = 0; wv < 8; ++wv) t += warp[wv];
    const float inv = (float)(1.0 / sqrt((double)(t / (float)dim + eps)));
    for (int64_t i = 0; i < dim; ++i)
      out[r * dim + i] = f32_to_bf16(bf16_to_f32(xr[i]) * inv * (1.0f + bf16_to_f32(w[i])));
  }
}

/* out[i] = bf16(float(out[i]) + float(x[i])) */
ORACLE_API void oracle_residual_add(uint16_t* out, const uint16_t* x, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(bf16_to_f32(out[i]) + bf16_to_f32(x[i]));
}

/* fused [rows][2 inter] = [gate | up] -> out [rows][inter] = bf16(g / (1 + exp(-g)) * u), fp32 */
ORACLE_API void oracle_swiglu(const uint16_t* fused, int64_t rows, int64_t inter, uint16_t* out) {
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < inter; ++i) {
      const float g = bf16_to_f32(fused[r * 2 * inter + i]);
      const float u = bf16_to_f32(fused[r * 2 * inter + inter + i]);
      out[r * inter + i] = f32_to_bf16((g / (1.f + expf(-g))) * u);
    }
}
