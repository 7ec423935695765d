// Stand-in for mllm/Backends/Arm/Kernels/kai_linear.hpp, which needs <arm_neon.h> and the
// un-vendored KleidiAI headers.  Declarations only (no definitions): the fixtures in
// tests/Arm/KaiLinearTest.hpp hold these objects as members and call them from methods the
// oracle build never instantiates.  Shapes of the declarations follow
// mllm/Backends/Arm/Kernels/kai_linear.hpp:57-118 and :186-232.
#pragma once
#include <cstddef>
#include <cstdint>
#include "mllm/Core/DataTypes.hpp"
// Arm's float16_t, as a storage-only stand-in that computes through float (the fp16 fixtures
// that use it are compiled but never run by the oracle build).
struct float16_t {
  _Float16 v;
  float16_t() = default;
  float16_t(float f) : v((_Float16)f) {}
  float16_t(double f) : v((_Float16)f) {}
  float16_t(int f) : v((_Float16)f) {}
  operator float() const { return (float)v; }
  float16_t& operator+=(float o) { v = (_Float16)((float)v + o); return *this; }
};
#include <fmt/core.h>
template<>
struct fmt::formatter<float16_t> : fmt::formatter<float> {
  template<typename Ctx>
  auto format(const float16_t& h, Ctx& ctx) const { return fmt::formatter<float>::format((float)h, ctx); }
};
namespace mllm::arm {
struct KaiLinear_fp16_fp16_fp16p_mxk_kxn {
  size_t pack_rhs_size(int K, int N);
  void pack_rhs_offline(float16_t* out, const float16_t* rhs, const float16_t* bias, int K, int N);
  void matmul(float16_t* dst, const float16_t* lhs, const float16_t* rhs, int M, int K, int N);
};
struct KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk {
  enum class Tiles : uint8_t { qai8dxp1x8_qsi4c32p4x8_1x4x32 };
  size_t workspace_size(int M, int K, Tiles t);
  size_t quant_pack_rhs_size(int N, int K, Tiles t);
  void quant_pack_rhs_offline(uint8_t* out, const float* rhs, const float* bias, int N, int K, Tiles t);
  void matmul(float* dst, const float* lhs, const uint8_t* packed, void* ws, int M, int K, int N, Tiles t);
};
struct KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk {
  enum class Tiles : uint8_t { qsi8d32p1x8_qai4c32p4x8_1x4 , qsi8d32p4x8_qai4c32p4x8_8x4_i8mm, qsi8d32p4x4_qai4c32p4x4_8x4, qsi8d32p1x4_qai4c32p4x4_1x4 };
  size_t workspace_size(int M, int K, mllm::DataTypes dt, Tiles t);
  size_t quant_pack_rhs_size(int N, int K, Tiles t);
  void quant_pack_rhs_offline(uint8_t* out, const float* rhs, const float* bias, int K, int N, Tiles t);
  void matmul(float16_t* dst, const float16_t* lhs, const uint8_t* packed, void* ws, int M, int K, int N, Tiles t);
};
}  // namespace mllm::arm
