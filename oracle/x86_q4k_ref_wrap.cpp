// C-callable wrapper around the reference's X86 int4 kernels, used only as the timed
// "reference CPU path" beside the GPU numbers (bench.py).  TEST/BENCH INFRASTRUCTURE ONLY.
//
// The reference's X86 backend has no LinearOp; its int4 arithmetic is the ggml-derived
// Q4_K x Q8_K dot product (mllm/Backends/X86/Kernels/quants.cpp:83-225,
// vec_dot_q4_k_q8_k_avx2.cpp:70-147, vec_dot_q4_k_q8_k_avx512f.cpp).  This is a DIFFERENT int4
// format from the Arm W4A32 path (256-element super-blocks, 6-bit sub-scales and mins), so it is
// a throughput baseline, never a parity oracle.  The GEMV below follows the harness pattern of
// benchmarks/Backend/X86/GemvOps.cpp:9-48: quantize the weight rows once, quantize each activation
// row per call, one vec_dot per output element; rows are spread over OpenMP threads.
#include <cstdint>
#include <cstdlib>
#include <vector>
#include <omp.h>
#include "mllm/Backends/X86/Kernels/quants.hpp"
#include "mllm/Backends/X86/Kernels/vec_dot_q4_k_q8_k_avx2.hpp"
#include "mllm/Backends/X86/Kernels/vec_dot_q4_k_q8_k_avx512f.hpp"

#define API extern "C" __attribute__((visibility("default")))

API size_t x86ref_q4k_row_bytes(int K) { return (size_t)(K / 256) * sizeof(mllm::block_q4_k_t); }
API size_t x86ref_q8k_row_bytes(int K) { return (size_t)(K / 256) * sizeof(mllm::block_q8_k_t); }
API int x86ref_has_avx512(void) {
#if defined(__AVX512F__)
  return 1;
#else
  return 0;
#endif
}

// W: fp32 [N, K] row-major -> N rows of Q4_K super-blocks (untimed set-up).
API void x86ref_quantize_weights(const float* W, int N, int K, void* out) {
  const size_t rb = x86ref_q4k_row_bytes(K);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    mllm::X86::quantize_row_q4_k((mllm::block_q4_k_t*)((char*)out + n * rb), W + (size_t)n * K, K);
}

// y[M,N] = x[M,K] . Wq^T ; activation rows are quantized to Q8_K inside the call.
// variant 0 = AVX2 kernel, 1 = AVX-512 kernel (only if compiled in).
API int x86ref_linear(const float* x, const void* Wq, float* y, int M, int N, int K, int threads, int variant,
                      void* q8_workspace) {
  if (K % 256 != 0) return 1;
  const size_t rb = x86ref_q4k_row_bytes(K);
  const size_t xb = x86ref_q8k_row_bytes(K);
  if (threads <= 0) threads = omp_get_max_threads();
  for (int m = 0; m < M; ++m)
    mllm::X86::quantize_row_q8_k((char*)q8_workspace + m * xb, x + (size_t)m * K, K);
#pragma omp parallel for schedule(static) num_threads(threads) collapse(1)
  for (int n = 0; n < N; ++n) {
    const auto* wrow = (const mllm::block_q4_k_t*)((const char*)Wq + n * rb);
    for (int m = 0; m < M; ++m) {
      const auto* xrow = (const mllm::block_q8_k_t*)((const char*)q8_workspace + m * xb);
      float c = 0.f;
#if defined(__AVX512F__)
      if (variant == 1) mllm::X86::vec_dot_q4_k_q8_k_avx512f(&c, wrow, xrow, K);
      else
#endif
        mllm::X86::vec_dot_q4_k_q8_k_avx2(&c, wrow, xrow, K);
      y[(size_t)m * N + n] = c;
    }
  }
  return 0;
}
API int x86ref_max_threads(void) { return omp_get_max_threads(); }
