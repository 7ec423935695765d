// SIMT (dp4a) W4A32 GEMM: the any-shape path (any M, K, N, including K not a multiple of 32).
// It reads the quantized activations from the workspace written by act_quant_ws_kernel and the
// weights straight from the tile layout.  One CTA = one 32-row weight panel x 32 activation rows;
// each of the 4 warps owns 8 activation rows, lane = weight row.  Every group sum is an exact
// int32 and the fp32 accumulation runs over the K-groups in order, as in the reference's scalar
// code (tests/Arm/KaiLinearTest.hpp:338-377); only the zero-point term is taken out of the
// integer sum (see gemv.cu).  The tcgen05 kernel (gemm_tc.cu) is the fast path for large M.
#include "device_common.cuh"

namespace mllmb200 {

constexpr int kSimtRowsPerWarp = 8;
constexpr int kSimtWarps = 4;
constexpr int kSimtMTile = kSimtRowsPerWarp * kSimtWarps;

// nibble word -> two words of signed int8 in natural k order
__device__ __forceinline__ void unpack_word_signed(uint32_t w, int& k0123, int& k4567) {
  const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
  uint32_t a = __byte_perm(lo, hi, 0x5140);  // k0 k1 k2 k3
  uint32_t b = __byte_perm(lo, hi, 0x7362);  // k4 k5 k6 k7
  // u - 8 per byte: flip bit 3 (4-bit two's complement) and sign-extend into the high half-byte
  const uint32_t sa = (~a) & 0x08080808u, sb = (~b) & 0x08080808u;
  k0123 = (int)((a ^ 0x08080808u) | (sa * 0x1Eu));
  k4567 = (int)((b ^ 0x08080808u) | (sb * 0x1Eu));
}

__global__ void __launch_bounds__(kSimtWarps * 32) w4a32_gemm_simt_kernel(
    const int8_t* __restrict__ a_q, const float2* __restrict__ a_hdr, const uint8_t* __restrict__ tiled,
    float* __restrict__ y, int m, int k_pad, int n, int ldy, int num_groups, size_t zsum_off, size_t bias_off) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int panel = blockIdx.x;
  const int m0 = blockIdx.y * kSimtMTile + warp * kSimtRowsPerWarp;
  if (m0 >= m) return;
  const TiledHeader* hdr = reinterpret_cast<const TiledHeader*>(tiled);
  const uint32_t scale_mode = hdr->scale_mode;
  const uint8_t* cells = tiled + sizeof(TiledHeader) + (size_t)panel * num_groups * kCellBytes;
  float acc[kSimtRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kSimtRowsPerWarp; ++i) acc[i] = 0.0f;
  for (int b = 0; b < num_groups; ++b) {
    const uint8_t* cell = cells + (size_t)b * kCellBytes;
    const uint4 wq = *reinterpret_cast<const uint4*>(cell + lane * 16);
    const float s = decode_scale(*reinterpret_cast<const uint16_t*>(cell + kCellNibbleBytes + lane * 2), scale_mode);
    int w[8];
    unpack_word_signed(wq.x, w[0], w[1]);
    unpack_word_signed(wq.y, w[2], w[3]);
    unpack_word_signed(wq.z, w[4], w[5]);
    unpack_word_signed(wq.w, w[6], w[7]);
#pragma unroll
    for (int i = 0; i < kSimtRowsPerWarp; ++i) {
      const int mm = min(m0 + i, m - 1);
      const int4* ap = reinterpret_cast<const int4*>(a_q + (size_t)mm * k_pad + b * kGroup);
      const int4 a0 = __ldg(ap), a1 = __ldg(ap + 1);
      int iacc = 0;
      iacc = __dp4a(a0.x, w[0], iacc);
      iacc = __dp4a(a0.y, w[1], iacc);
      iacc = __dp4a(a0.z, w[2], iacc);
      iacc = __dp4a(a0.w, w[3], iacc);
      iacc = __dp4a(a1.x, w[4], iacc);
      iacc = __dp4a(a1.y, w[5], iacc);
      iacc = __dp4a(a1.z, w[6], iacc);
      iacc = __dp4a(a1.w, w[7], iacc);
      acc[i] = fmaf((float)iacc, s, acc[i]);
    }
  }
  const int n_pad = panel * kPanelRows + lane;
  const float zs = reinterpret_cast<const float*>(tiled + zsum_off)[n_pad];
  const float bs = reinterpret_cast<const float*>(tiled + bias_off)[n_pad];
  if (n_pad < n) {
#pragma unroll
    for (int i = 0; i < kSimtRowsPerWarp; ++i) {
      const int mm = m0 + i;
      if (mm < m) {
        const float2 h = a_hdr[mm];
        float v = fmaf((float)__float_as_int(h.y), zs, acc[i]);
        v = fmaf(v, h.x, bs);
        y[(size_t)mm * ldy + n_pad] = clamp_flt_max(v);
      }
    }
  }
}

cudaError_t launch_w4a32_gemm_simt(const int8_t* a_q, const float2* a_hdr, const void* tiled, float* y, int m, int k,
                                   int n, int ldy, cudaStream_t stream) {
  const int num_groups = (k + kGroup - 1) / kGroup;
  const int num_panels = (n + kPanelRows - 1) / kPanelRows;
  const TiledHeader th = make_tiled_header(n, k, 0, 0);
  const int my = (m + kSimtMTile - 1) / kSimtMTile;
  if (my > 65535) return cudaErrorInvalidValue;
  dim3 grid((unsigned)num_panels, (unsigned)my, 1);
  w4a32_gemm_simt_kernel<<<grid, kSimtWarps * 32, 0, stream>>>(a_q, a_hdr, static_cast<const uint8_t*>(tiled), y, m,
                                                               num_groups * kGroup, n, ldy, num_groups, th.zsum_off,
                                                               th.bias_off);
  return cudaGetLastError();
}

}  // namespace mllmb200
