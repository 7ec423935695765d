// Builds the reference's own scalar code for the W4A32 path into a C-callable library.
// TEST INFRASTRUCTURE ONLY (validates oracle/w4a32_oracle.c and generates tests/golden/).
//
// The functions exported here are the protected members of the reference's gtest fixture
// KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_Test (tests/Arm/KaiLinearTest.hpp:127-477), compiled
// from that header where it lies in the reference tree; nothing is copied.  The header's Arm-only
// includes are satisfied by the declaration-only stand-ins under oracle/ref_shim/.
#include <cfloat>
#include <cstring>
#include "tests/Arm/KaiLinearTest.hpp"

namespace {
struct Exposed : public KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_Test {
  using Base = KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_Test;
  using Base::cast_bf16_f32;
  using Base::cast_f32_bf16;
  using Base::fill_uniform_random;
  using Base::quant_nxk_qs4c32_f32;
  using Base::ref_matmul_mxn_mxk_nxk_f32_qa8dx_qs4c32;
  using Base::ref_quant_qa8dx_f32;
};
Exposed& fixture() {
  static Exposed f;
  return f;
}
}  // namespace

extern "C" {
__attribute__((visibility("default"))) uint16_t kairef_cast_bf16_f32(float v) { return fixture().cast_bf16_f32(v); }
__attribute__((visibility("default"))) float kairef_cast_f32_bf16(uint16_t v) { return fixture().cast_f32_bf16(v); }
__attribute__((visibility("default"))) void kairef_fill_uniform_random(size_t rows, size_t cols, float* dst, size_t seed) {
  fixture().fill_uniform_random(rows, cols, dst, seed);
}
__attribute__((visibility("default"))) void kairef_quant_nxk_qs4c32_f32(size_t n, size_t k, size_t bl, const float* rhs,
                                                                      uint8_t* q, uint16_t* scales) {
  fixture().quant_nxk_qs4c32_f32(n, k, bl, rhs, q, scales);
}
__attribute__((visibility("default"))) void kairef_quant_qa8dx_f32(size_t m, size_t k, const float* lhs, int8_t* out) {
  fixture().ref_quant_qa8dx_f32(m, k, lhs, out);
}
__attribute__((visibility("default"))) void kairef_matmul(size_t m, size_t n, size_t k, size_t bl, const int8_t* lhs,
                                                        const uint8_t* rhs, const uint16_t* scales, float* dst) {
  fixture().ref_matmul_mxn_mxk_nxk_f32_qa8dx_qs4c32(m, n, k, bl, lhs, rhs, scales, dst, -FLT_MAX, FLT_MAX);
}
}
