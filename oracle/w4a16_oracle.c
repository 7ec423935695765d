/*
 * CPU oracle for the W4A16 sibling of the quantized linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * Restates, in plain C, mllm-advanced's KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk: asymmetric int4
 * weights in groups of 32 along K with an fp32 scale and an fp32 "zero" term per group,
 * activations quantized on the fly to symmetric int8 per 32-element block with an fp32 scale
 * per block, fp16 output.  Nothing the library ships may call it.
 *
 * Parity status: PARITY UNPINNED.
 *  - The weight quantization follows the reference's own scalar code line by line
 *    (mllm/Backends/Arm/Kernels/kai_linear.cpp:710-817).  That file cannot be compiled on x86-64
 *    (arm_neon.h, KleidiAI headers, an inline `fcvtns`), so it is restated, not executed.
 *  - The activation quantization (kai_run_lhs_quant_pack_qsi8d32pscalef32_f32_neon / _f16_neon,
 *    call sites kai_linear.cpp:863,913) and the block matmul (the
 *    kai_matmul_clamp_f16_qsi8d32p_qai4c32p ukernels, call site kai_linear.cpp:886-895,936-945)
 *    live in Arm KleidiAI, an un-vendored submodule (.gitmodules; pinned commit not recorded in
 *    the tree).  They are restated from the format names and the published scalar algorithm:
 *    per block amax/127 scale, round half away from zero; per block
 *    a_scale * (w_scale * int_dot + w_zero * int_sum), fp32 accumulation in K order, bias added
 *    last, clamp, one rounding to fp16.
 *  - The reference's only test for this path (tests/Arm/KaiLinearTest.hpp:479-594, M=32, K=N=64)
 *    compares against a dense fp16 product with 1e-2 relative tolerance and stores no output
 *    vectors; tests/test_w4a16.py reproduces its inputs and reports how this oracle does on it.
 *
 * Build with -ffp-contract=off.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

uint16_t oracle_cast_f16_f32(float f);  /* w4a32_oracle.c */
float oracle_cast_f32_f16(uint16_t h);

static size_t a16_roundup(size_t a, size_t b) { return ((a + b - 1) / b) * b; }
static size_t a16_blocks(size_t k, size_t bl) { return a16_roundup(k, bl) / bl; }
static size_t a16_native_stride(size_t k) { return a16_roundup(k, 2) / 2; }

/* kai_linear.hpp:194-198: `fcvtns` = round to nearest, ties to even, to int32. */
static int32_t a16_round_nearest(float v) { return (int32_t)lrintf(v); }

/* kai_linear.cpp:710-817.  rhs_f32: [n,k] row-major.  Outputs:
 *   rhs_qai4c32 [n][ceil(k/2)]: byte j of a row = (u[2j] << 4) | u[2j+1], u = q + 8  (":807-816": the
 *                               halves are swapped at the end, so the EVEN k sits in the HIGH half)
 *   rhs_scales  [n][blocks]   : scale = 1 / inv_scale
 *   rhs_zeros   [n][blocks]   : (-zero_point) * scale, so that w ~ (u - 8) * scale + zero
 * zero_point itself (before the rescale of ":797-805") is returned in zp_out when not NULL. */
ORACLE_API void oracle_w4a16_quant_nxk_qai4c32_f32(size_t n, size_t k, size_t bl, const float* rhs_f32,
                                                   uint8_t* rhs_qai4c32, float* rhs_zeros, float* rhs_scales,
                                                   int32_t* zp_out) {
  const size_t nb = a16_blocks(k, bl);
  const size_t stride = a16_native_stride(k);
  memset(rhs_qai4c32, 0, n * stride);
  for (size_t row = 0; row < n; ++row) {
    const float* src = rhs_f32 + row * k;
    for (size_t b = 0; b < nb; ++b) {
      float mn = FLT_MAX, mx = -FLT_MAX;
      for (size_t i = 0; i < bl; ++i) {
        const size_t x = b * bl + i;
        if (x >= k) break;
        const float v = src[x];
        mn = v < mn ? v : mn; /* std::min(a, b) returns b when b < a */
        mx = mx < v ? v : mx; /* std::max(a, b) returns b when a < b */
      }
      if (mn > 0) mn = 0;
      if (mx < 0) mx = 0;
      const float inv_scale = mx != mn ? (7.0f - -8.0f) / (mx - mn) : 1.0f;
      const float scale = 1.0f / inv_scale;
      const float scaled_min = mn / scale;
      const float scaled_max = mx / scale;
      const float zero_point_f =
          -(scaled_min + -8.0f) < scaled_max + 7.0f ? scaled_min - -8.0f : scaled_max - 7.0f;
      const int32_t zero_point = -a16_round_nearest(zero_point_f);
      if (zp_out) zp_out[row * nb + b] = zero_point;
      rhs_scales[row * nb + b] = scale;
      /* ":765" stores the integer as float, ":797-805" then rescales it */
      rhs_zeros[row * nb + b] = (-(float)zero_point) * scale;
      for (size_t i = 0; i < bl; ++i) {
        const size_t x = b * bl + i;
        if (x >= k) break;
        const float this_inv_scale = scale != 0 ? 1.0f / scale : 0.0f;
        int32_t q = a16_round_nearest(src[x] * this_inv_scale) + zero_point;
        q = q < -8 ? -8 : q;
        q = q > 7 ? 7 : q;
        const uint8_t u = (uint8_t)(q + 8);
        uint8_t* dst = rhs_qai4c32 + x / 2 + row * stride;
        if ((x % 2) == 0) *dst = u; /* low half first ... */
        else *dst |= (uint8_t)(u << 4);
      }
    }
  }
  for (size_t i = 0; i < n * stride; ++i) { /* ... then the halves are swapped */
    const uint8_t v = rhs_qai4c32[i];
    rhs_qai4c32[i] = (uint8_t)(((v & 0x0F) << 4) | (v >> 4));
  }
}

/* Activation quantization, format qsi8d32p + fp32 scale (restated; see the header):
 * per row and block of `bl`: amax = max |x|, scale = amax / 127, recip = scale ? 1/scale : 0,
 * q = (int8) clamp(roundf(x * recip), -127, 127).  a_q: [m][blocks*bl] (zero padded), a_s: [m][blocks]. */
ORACLE_API void oracle_w4a16_quant_lhs_f32(size_t m, size_t k, size_t bl, const float* lhs, int8_t* a_q,
                                           float* a_s) {
  const size_t nb = a16_blocks(k, bl);
  memset(a_q, 0, m * nb * bl);
  for (size_t row = 0; row < m; ++row) {
    for (size_t b = 0; b < nb; ++b) {
      float amax = 0.0f;
      for (size_t i = 0; i < bl && b * bl + i < k; ++i) {
        const float a = fabsf(lhs[row * k + b * bl + i]);
        amax = a > amax ? a : amax;
      }
      const float scale = amax / 127.0f;
      const float recip = scale ? 1.0f / scale : 0.0f;
      a_s[row * nb + b] = scale;
      for (size_t i = 0; i < bl && b * bl + i < k; ++i) {
        float r = roundf(lhs[row * k + b * bl + i] * recip);
        r = r < -127.0f ? -127.0f : r;
        r = r > 127.0f ? 127.0f : r;
        a_q[(row * nb + b) * bl + i] = (int8_t)r;
      }
    }
  }
}

/* y[m,n] = fp16( clamp( sum_b a_s[m,b] * ( s[n,b] * (float)dot_b + z[n,b] * (float)sum_b ) + bias[n] ) )
 * dot_b = sum_{k in b} a_q[m,k] * (u[n,k] - 8), sum_b = sum_{k in b} a_q[m,k]; fp32, blocks in K order. */
ORACLE_API void oracle_w4a16_matmul(size_t m, size_t n, size_t k, size_t bl, const int8_t* a_q, const float* a_s,
                                    const uint8_t* rhs_qai4c32, const float* rhs_scales, const float* rhs_zeros,
                                    const float* bias, uint16_t* dst_f16, float clamp_min, float clamp_max) {
  const size_t nb = a16_blocks(k, bl);
  const size_t stride = a16_native_stride(k);
#pragma omp parallel for schedule(static)
  for (size_t row = 0; row < m; ++row) {
    for (size_t col = 0; col < n; ++col) {
      float acc = 0.0f;
      for (size_t b = 0; b < nb; ++b) {
        int32_t dot = 0, sum = 0;
        for (size_t i = 0; i < bl && b * bl + i < k; ++i) {
          const size_t x = b * bl + i;
          const uint8_t byte = rhs_qai4c32[col * stride + x / 2];
          const int32_t u = (x % 2) == 0 ? (byte >> 4) : (byte & 0x0F);
          const int32_t a = a_q[(row * nb + b) * bl + i];
          dot += a * (u - 8);
          sum += a;
        }
        const float t = rhs_scales[col * nb + b] * (float)dot + rhs_zeros[col * nb + b] * (float)sum;
        acc += a_s[row * nb + b] * t;
      }
      if (bias) acc += bias[col];
      acc = acc < clamp_min ? clamp_min : acc;
      acc = acc > clamp_max ? clamp_max : acc;
      dst_f16[row * n + col] = oracle_cast_f16_f32(acc);
    }
  }
}

/* The whole forward on fp32 activations (fp16 activations are widened to fp32 by the caller, which is
 * exact).  ws: m * blocks * (bl + 4) bytes. */
ORACLE_API void oracle_linear_w4a16(size_t m, size_t n, size_t k, const float* x, const uint8_t* rhs_qai4c32,
                                    const float* rhs_scales, const float* rhs_zeros, const float* bias,
                                    uint16_t* y_f16, void* ws) {
  const size_t nb = a16_blocks(k, 32);
  float* a_s = (float*)ws;
  int8_t* a_q = (int8_t*)(a_s + m * nb);
  oracle_w4a16_quant_lhs_f32(m, k, 32, x, a_q, a_s);
  oracle_w4a16_matmul(m, n, k, 32, a_q, a_s, rhs_qai4c32, rhs_scales, rhs_zeros, bias, y_f16, -65504.0f, 65504.0f);
}

/* Inputs of the reference fixture (tests/Arm/KaiLinearTest.hpp:486-502): fp32 as in the W4A32 fixture;
 * the fp16 overload rounds rand()/RAND_MAX to fp16 FIRST, then computes *2-1 in fp16. */
ORACLE_API void oracle_w4a16_fill_uniform_random_f16(size_t count, uint16_t* dst, unsigned seed) {
  srand(seed);
  for (size_t i = 0; i < count; ++i) {
    const uint16_t h = oracle_cast_f16_f32((float)((double)rand() / RAND_MAX));
    const float two = oracle_cast_f32_f16(oracle_cast_f16_f32(oracle_cast_f32_f16(h) * 2.0f));
    dst[i] = oracle_cast_f16_f32(two - 1.0f);
  }
}
