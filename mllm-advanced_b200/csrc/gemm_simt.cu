// SIMT (dp4a) W4A32 GEMM: the any-shape path (any M, K, N, including K not a multiple of 32).
// It reads the quantized activation records written by act_quant_records_kernel and the
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

__global__ void __launch_bounds__(kSimtWarps * 32) w4a32_gemm_simt_kernel(
    const uint8_t* __restrict__ a_rec, const float2* __restrict__ a_hdr, const uint8_t* __restrict__ tiled,
    float* __restrict__ y, int m, int n, int k, int ldy, int num_groups, size_t zsum_off, size_t bias_off) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (!tiled_header_ok_cta(tiled, n, k)) return;  // before the first byte of the matrix is read
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
    const int lo0 = (int)(wq.x & 0x0F0F0F0Fu), hi0 = (int)((wq.x >> 4) & 0x0F0F0F0Fu);
    const int lo1 = (int)(wq.y & 0x0F0F0F0Fu), hi1 = (int)((wq.y >> 4) & 0x0F0F0F0Fu);
    const int lo2 = (int)(wq.z & 0x0F0F0F0Fu), hi2 = (int)((wq.z >> 4) & 0x0F0F0F0Fu);
    const int lo3 = (int)(wq.w & 0x0F0F0F0Fu), hi3 = (int)((wq.w >> 4) & 0x0F0F0F0Fu);
#pragma unroll
    for (int i = 0; i < kSimtRowsPerWarp; ++i) {
      const int mm = min(m0 + i, m - 1);
      const uint8_t* rec = a_rec + ((size_t)mm * num_groups + b) * kActRecordBytes;
      const int4 alo = __ldg(reinterpret_cast<const int4*>(rec));
      const int4 ahi = __ldg(reinterpret_cast<const int4*>(rec + 16));
      int ia = __ldg(reinterpret_cast<const int*>(rec + 32));
      int ib = 0;
      ia = __dp4a(alo.x, lo0, ia);
      ib = __dp4a(ahi.x, hi0, ib);
      ia = __dp4a(alo.y, lo1, ia);
      ib = __dp4a(ahi.y, hi1, ib);
      ia = __dp4a(alo.z, lo2, ia);
      ib = __dp4a(ahi.z, hi2, ib);
      ia = __dp4a(alo.w, lo3, ia);
      ib = __dp4a(ahi.w, hi3, ib);
      acc[i] = fmaf((float)(ia + ib), s, acc[i]);
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

cudaError_t launch_w4a32_gemm_simt(const uint8_t* a_rec, const float2* a_hdr, const void* tiled, float* y, int m, int k,
                                   int n, int ldy, cudaStream_t stream) {
  const int num_groups = (k + kGroup - 1) / kGroup;
  const int num_panels = (n + kPanelRows - 1) / kPanelRows;
  const TiledHeader th = make_tiled_header(n, k, 0, 0);
  const int my = (m + kSimtMTile - 1) / kSimtMTile;
  if (my > 65535) return cudaErrorInvalidValue;
  dim3 grid((unsigned)num_panels, (unsigned)my, 1);
  w4a32_gemm_simt_kernel<<<grid, kSimtWarps * 32, 0, stream>>>(a_rec, a_hdr, static_cast<const uint8_t*>(tiled), y, m, n,
                                                               k, ldy, num_groups, th.zsum_off, th.bias_off);
  return cudaGetLastError();
}

}  // namespace mllmb200
