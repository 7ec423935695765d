/*
 * CPU oracle for the W4A32 quantized linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of mllm-advanced's W4A32 linear
 * (int4 group-32 weights with bf16 per-group scales, activations quantized on the fly
 * to asymmetric int8 per row, int8 x int4 block dot products, fp32 output).  It is the
 * checker the CUDA path is compared against; nothing the library ships may call it.
 *
 * Parity status: PINNED.  Each function is checked (tests/test_oracle.py) against
 *  - the reference's own scalar code for this path compiled from its sources in place
 *    (oracle/_ref/libkai_ref.so, built by oracle/Makefile from
 *    tests/Arm/KaiLinearTest.hpp), on the reference fixture (M=1, K=N=1024,
 *    srand 4568 / 4572) and on ragged shapes, bit for bit; and
 *  - golden vectors committed under tests/golden/ that were produced by that build.
 * What stays unpinned (no reference test covers it, and Arm KleidiAI, which holds the
 * production kernels, is an un-vendored submodule): the position of the bias add and the
 * bf16 rounding mode inside KleidiAI.  Both are stated below where they are chosen.
 *
 * Reference anchors (paths relative to the reference project root):
 *   weight quantization + nibble layout  mllm/Backends/Arm/Kernels/kai_linear.cpp:220-291
 *                                        (identical copy tests/Arm/KaiLinearTest.hpp:232-298)
 *   bf16 casts                           tests/Arm/KaiLinearTest.hpp:133-149
 *   activation quantization              tests/Arm/KaiLinearTest.hpp:163-230
 *   block matmul                         tests/Arm/KaiLinearTest.hpp:311-385
 *   stride helpers                       tests/Arm/KaiLinearTest.hpp:300-309
 *
 * Build with -ffp-contract=off: the accumulation "acc += (float)iacc * scale" must be a
 * separate multiply and add, as the reference's scalar code compiles to on x86-64.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ---- helpers: tests/Arm/KaiLinearTest.hpp:300-309 ---- */
static size_t roundup_sz(size_t a, size_t b) { return ((a + b - 1) / b) * b; }
ORACLE_API size_t oracle_num_blocks_per_row(size_t k, size_t bl) { return roundup_sz(k, bl) / bl; }
ORACLE_API size_t oracle_rhs_native_stride(size_t k) { return roundup_sz(k, 2) / 2; }
ORACLE_API size_t oracle_rhs_scale_stride(size_t k, size_t bl) {
  return oracle_num_blocks_per_row(k, bl) * sizeof(uint16_t);
}
/* bytes per quantized activation row: k int8 + float recip-scale + int32 offset
 * (tests/Arm/KaiLinearTest.hpp:164) */
ORACLE_API size_t oracle_lhs_row_stride(size_t k) { return k + sizeof(float) + sizeof(int32_t); }

/* ---- bf16 <-> f32: tests/Arm/KaiLinearTest.hpp:133-149 ----
 * scale_mode 0: truncate (bits >> 16), what the reference's test does without
 *               __ARM_FEATURE_BF16 and what its published build flags select.
 * scale_mode 1: round to nearest even (the bfcvt variant), offered as an option.
 * scale_mode 2: IEEE fp16 (round to nearest even) - the BASELINE configs' wording. */
ORACLE_API uint16_t oracle_cast_bf16_f32(float f32, int scale_mode) {
  uint32_t bits;
  memcpy(&bits, &f32, sizeof(bits));
  if (scale_mode == 1) {
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x40u); /* NaN */
    uint32_t lsb = (bits >> 16) & 1u;
    bits += 0x7fffu + lsb;
  }
  return (uint16_t)(bits >> 16);
}

ORACLE_API float oracle_cast_f32_bf16(uint16_t bf16) {
  const uint32_t bits = ((uint32_t)bf16) << 16;
  float f32;
  memcpy(&f32, &bits, sizeof(f32));
  return f32;
}

/* IEEE binary16 -> f32, for scale_mode 2. */
ORACLE_API float oracle_cast_f32_f16(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400u));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, sizeof(f));
  return f;
}

/* f32 -> IEEE binary16, round to nearest even, for scale_mode 2. */
ORACLE_API uint16_t oracle_cast_f16_f32(float f) {
  uint32_t x;
  memcpy(&x, &f, sizeof(x));
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
  if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* overflows to inf after rounding */
  if (x < 0x33000001u) return (uint16_t)sign;              /* rounds to zero */
  int32_t e = (int32_t)(x >> 23) - 127;
  uint32_t m = (x & 0x7fffffu) | 0x800000u;
  uint32_t shift, half;
  if (e < -14) {
    shift = (uint32_t)(13 + (-14 - e));
    uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u);
    half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | q);
  }
  uint32_t q = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3ffu);
  uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
  return (uint16_t)(sign | q);
}

ORACLE_API float oracle_scale_to_f32(uint16_t s, int scale_mode) {
  return scale_mode == 2 ? oracle_cast_f32_f16(s) : oracle_cast_f32_bf16(s);
}

/* ---- weight quantization: mllm/Backends/Arm/Kernels/kai_linear.cpp:220-291 ----
 * Per row, per block of `bl` along K: take the element of largest magnitude keeping its
 * sign (strict <, first maximum wins); scale = max / -8; quantize with the un-rounded fp32
 * reciprocal, round half away from zero, clamp to [-8, 7]; store q+8 as a nibble, even k
 * in the low half of byte k/2, odd k in the high half; store the scale as 2 bytes. */
ORACLE_API void oracle_quant_nxk_qs4c32_f32(size_t n, size_t k, size_t bl, const float* rhs_f32,
                                            uint8_t* rhs_qs4c32, uint16_t* rhs_scales,
                                            int scale_mode) {
  const size_t num_blocks_row = oracle_num_blocks_per_row(k, bl);
  const size_t stride = oracle_rhs_native_stride(k);
  memset(rhs_qs4c32, 0, n * stride);
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (size_t row = 0; row < n; ++row) {
    const float* src = rhs_f32 + row * k;
    uint16_t* scales = rhs_scales + row * num_blocks_row;
    for (size_t blk = 0; blk < num_blocks_row; ++blk) {
      float amax = 0.0f, max = 0.0f;
      for (size_t b = 0; b < bl; ++b) {
        const size_t k_idx = blk * bl + b;
        if (k_idx >= k) break;
        const float v = src[k_idx];
        const float av = fabsf(v);
        if (amax < av) { amax = av; max = v; }
      }
      const float scale = (float)((double)max / -8.0);
      const float recip = scale ? 1.0f / scale : 0.0f;
      scales[blk] = scale_mode == 2 ? oracle_cast_f16_f32(scale) : oracle_cast_bf16_f32(scale, scale_mode);
      for (size_t i = 0; i < bl; ++i) {
        const size_t k_idx = blk * bl + i;
        if (k_idx >= k) break;
        int32_t q = (int32_t)roundf(src[k_idx] * recip);
        q = q < -8 ? -8 : q;
        q = q > 7 ? 7 : q;
        const uint8_t u = (uint8_t)(q + 8);
        const size_t addr = k_idx / 2 + row * stride;
        if ((k_idx % 2) == 0) rhs_qs4c32[addr] = u;
        else rhs_qs4c32[addr] |= (uint8_t)(u << 4);
      }
    }
  }
}

/* ---- activation quantization: tests/Arm/KaiLinearTest.hpp:163-230 ----
 * Per row: asymmetric int8 with one scale and one zero point.  Row layout in `lhs_qa8dx`:
 * { float recip_scale; int32 neg_zero_point; int8 q[k] }.  Note the two rounding rules:
 * round() (half away from zero) for the values, lrintf (half to even) for the zero point. */
ORACLE_API void oracle_quant_qa8dx_f32(size_t m, size_t k, const float* lhs_f32, int8_t* lhs_qa8dx) {
  const size_t dst_stride = oracle_lhs_row_stride(k);
  for (size_t row = 0; row < m; ++row) {
    const float* src = lhs_f32 + row * k;
    float max0 = -FLT_MAX, min0 = FLT_MAX;
    for (size_t i = 0; i < k; ++i) {
      const float v = src[i];
      max0 = v < max0 ? max0 : v; /* std::max(src, max0) */
      min0 = min0 < v ? min0 : v; /* std::min(src, min0) */
    }
    const float qmin = (float)INT8_MIN, qmax = (float)INT8_MAX;
    const float rmin0 = min0 < 0.0f ? min0 : 0.0f; /* std::min(0.0f, min0) */
    const float rmax0 = 0.0f < max0 ? max0 : 0.0f; /* std::max(0.0f, max0) */
    const float scale0 = rmin0 == rmax0 ? 1.f : (qmax - qmin) / (rmax0 - rmin0);
    const float recip_scale0 = scale0 ? 1.0f / scale0 : 0.0f;
    const float descaled_min0 = rmin0 * scale0;
    const float descaled_max0 = rmax0 * scale0;
    const float zp_from_min_error0 = qmin + descaled_min0;
    const float zp_from_max_error0 = qmax + descaled_max0;
    float zero_point0 = zp_from_min_error0 + zp_from_max_error0 > 0 ? qmin - descaled_min0
                                                                    : qmax - descaled_max0;
    zero_point0 = zero_point0 < qmin ? qmin : zero_point0; /* std::max(zp, qmin) */
    zero_point0 = qmax < zero_point0 ? qmax : zero_point0; /* std::min(zp, qmax) */
    const int32_t nudged_zero_point0 = (int32_t)lrintf(zero_point0);

    int8_t* dst = lhs_qa8dx + row * dst_stride;
    const int32_t neg_zp = -nudged_zero_point0;
    memcpy(dst, &recip_scale0, sizeof(float));
    memcpy(dst + sizeof(float), &neg_zp, sizeof(int32_t));
    dst += sizeof(float) + sizeof(int32_t);
    for (size_t i = 0; i < k; ++i) {
      int32_t v = (int32_t)roundf(src[i] * scale0);
      v += nudged_zero_point0;
      v = v < INT8_MIN ? INT8_MIN : v;
      v = v > INT8_MAX ? INT8_MAX : v;
      dst[i] = (int8_t)v;
    }
  }
}

/* ---- block matmul: tests/Arm/KaiLinearTest.hpp:311-385 ----
 * dst[m,n] = clamp( lhs_scale[m] * sum_blocks( (float)( sum_{k in block} (a_q + a_off) * (u - 8) )
 *                                              * scale[n, block] ) (+ bias[n]) )
 * The int32 block sums are exact; the fp32 accumulation runs over blocks in K order with a
 * separate multiply and add.  The bias add (absent from the reference's test, which passes no
 * bias; the production add sits inside KleidiAI) is placed after the lhs_scale multiply and
 * before the clamp: "unpinned", chosen by convention. */
static void matmul_rows(size_t row_begin, size_t row_end, size_t n, size_t k, size_t bl,
                        const int8_t* lhs_qa8dx, const uint8_t* rhs_qs4c32,
                        const uint16_t* scales, int scale_mode, const float* bias, float* dst_f32,
                        float scalar_min, float scalar_max, int parallel) {
  const size_t num_blocks_row = oracle_num_blocks_per_row(k, bl);
  const size_t lhs_stride = oracle_lhs_row_stride(k);
  const size_t rhs_stride = oracle_rhs_native_stride(k);
  (void)parallel;
  for (size_t row = row_begin; row < row_end; ++row) {
    const int8_t* lhs_row = lhs_qa8dx + row * lhs_stride;
    float lhs_scale;
    int32_t lhs_offset;
    memcpy(&lhs_scale, lhs_row, sizeof(float));
    memcpy(&lhs_offset, lhs_row + sizeof(float), sizeof(int32_t));
    const int8_t* lhs_q = lhs_row + sizeof(float) + sizeof(int32_t);
#ifdef _OPENMP
#pragma omp parallel for schedule(static) if (parallel)
#endif
    for (size_t col = 0; col < n; ++col) {
      float main_acc = 0.0f;
      const uint8_t* rhs_row = rhs_qs4c32 + col * rhs_stride;
      for (size_t blk = 0; blk < num_blocks_row; ++blk) {
        const float rhs_scale = oracle_scale_to_f32(scales[blk + col * num_blocks_row], scale_mode);
        int32_t iacc = 0;
        for (size_t i = 0; i < bl; ++i) {
          const size_t k_idx = blk * bl + i;
          if (k_idx >= k) break;
          const int32_t lhs_v = (int32_t)lhs_q[k_idx];
          const uint8_t byte = rhs_row[k_idx / 2];
          const int32_t rhs_v = (k_idx % 2) == 0 ? ((int32_t)(byte & 0x0F)) - 8 : ((int32_t)(byte >> 4)) - 8;
          iacc += lhs_v * rhs_v;
          iacc += lhs_offset * rhs_v;
        }
        main_acc += (float)iacc * rhs_scale;
      }
      main_acc = main_acc * lhs_scale;
      if (bias) main_acc = main_acc + bias[col];
      main_acc = main_acc < scalar_min ? scalar_min : main_acc; /* std::max(acc, min) */
      main_acc = scalar_max < main_acc ? scalar_max : main_acc; /* std::min(acc, max) */
      dst_f32[row * n + col] = main_acc;
    }
  }
}

ORACLE_API void oracle_matmul_f32_qa8dx_qs4c32(size_t m, size_t n, size_t k, size_t bl,
                                               const int8_t* lhs_qa8dx, const uint8_t* rhs_qs4c32,
                                               const uint16_t* scales, int scale_mode,
                                               const float* bias, float* dst_f32, float scalar_min,
                                               float scalar_max) {
  matmul_rows(0, m, n, k, bl, lhs_qa8dx, rhs_qs4c32, scales, scale_mode, bias, dst_f32, scalar_min,
              scalar_max, 1);
}

/* Whole forward of one linear on already-quantized weights: activation quantization of every row
 * (single pass, as the reference does before its parallel region,
 * mllm/Backends/Arm/Kernels/kai_linear.cpp:358-362) followed by the block matmul.
 * `workspace` must hold m * oracle_lhs_row_stride(k) bytes. */
ORACLE_API void oracle_linear_w4a32(size_t m, size_t n, size_t k, const float* x, const uint8_t* rhs_qs4c32,
                                    const uint16_t* scales, int scale_mode, const float* bias,
                                    float* y, void* workspace) {
  oracle_quant_qa8dx_f32(m, k, x, (int8_t*)workspace);
  oracle_matmul_f32_qa8dx_qs4c32(m, n, k, 32, (const int8_t*)workspace, rhs_qs4c32, scales, scale_mode,
                                 bias, y, -FLT_MAX, FLT_MAX);
}

/* glibc rand()-based generator of the reference fixture's inputs
 * (tests/Arm/KaiLinearTest.hpp:154-161): srand(seed), then (float)(rand()/RAND_MAX)*2-1. */
#include <stdlib.h>
ORACLE_API void oracle_fill_uniform_random(size_t count, float* dst, unsigned seed) {
  srand(seed);
  for (size_t i = 0; i < count; ++i) dst[i] = (float)((double)rand() / RAND_MAX) * 2 - 1;
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
