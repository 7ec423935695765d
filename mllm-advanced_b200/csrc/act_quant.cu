// Dynamic per-row int8 activation quantization as stand-alone kernels:
//  - act_quant_reflayout_kernel: the reference's row layout {float recip, int32 -zp, int8 q[k]}
//    (tests/Arm/KaiLinearTest.hpp:163-230 of the reference project), used by parity tests.
//  - act_quant_ws_kernel: the GEMM workspace: int8 [M][K_pad] in natural k order + row headers.
// The M <= 4 GEMV path does this inside the GEMV kernel instead (see gemv.cu).
#include "device_common.cuh"

namespace mllmb200 {

// grid = M rows, block = 256
__global__ void __launch_bounds__(256) act_quant_reflayout_kernel(const float* __restrict__ x, int k, int ldx,
                                                                  uint8_t* __restrict__ out) {
  __shared__ float scratch[64];
  const int m = blockIdx.x;
  const float* row = x + (size_t)m * ldx;
  float mn, mx;
  block_row_minmax(row, k, scratch, mn, mx);
  const ActQuantParams p = act_quant_params(mn, mx);
  uint8_t* dst = out + (size_t)m * (k + 8);
  if (threadIdx.x == 0) {
    // rows are k+8 bytes apart, so the header is not always 4-byte aligned: store bytewise
    const uint32_t rbits = __float_as_uint(p.recip_scale);
    const uint32_t obits = (uint32_t)(-p.nzp);
    for (int i = 0; i < 4; ++i) {
      dst[i] = (uint8_t)(rbits >> (8 * i));
      dst[4 + i] = (uint8_t)(obits >> (8 * i));
    }
  }
  for (int i = threadIdx.x; i < k; i += blockDim.x) dst[8 + i] = (uint8_t)(int8_t)act_quant_value(row[i], p);
}

// grid = M rows, block = 256.  a_q: int8 [M][k_pad] (k_pad = groups*32, padding = 0);
// hdr: [M] {float lhs_scale, int32 a_off}.
__global__ void __launch_bounds__(256) act_quant_ws_kernel(const float* __restrict__ x, int k, int ldx, int k_pad,
                                                           int8_t* __restrict__ a_q, float2* __restrict__ hdr) {
  __shared__ float scratch[64];
  const int m = blockIdx.x;
  const float* row = x + (size_t)m * ldx;
  float mn, mx;
  block_row_minmax(row, k, scratch, mn, mx);
  const ActQuantParams p = act_quant_params(mn, mx);
  if (threadIdx.x == 0) hdr[m] = make_float2(p.recip_scale, __int_as_float(-p.nzp));
  uint32_t* dst = reinterpret_cast<uint32_t*>(a_q + (size_t)m * k_pad);
  for (int w = threadIdx.x; w < (k_pad >> 2); w += blockDim.x) {
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kk = 4 * w + j;
      const int q = kk < k ? act_quant_value(row[kk], p) : 0;
      packed |= ((uint32_t)q & 0xFFu) << (8 * j);
    }
    dst[w] = packed;
  }
}

}  // namespace mllmb200
