// Host side of the W4A16 part of the C ABI: weight quantization and its pre-pack blob.
// Arithmetic follows mllm/Backends/Arm/Kernels/kai_linear.cpp:710-817 (reference project paths):
// per row and group of 32, min/max including 0, scale = 1 / (15 / (max - min)), zero point by
// round-to-nearest-even (the reference's `fcvtns`), nibble q + 8 with the even k in the high half.
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/mllmb200.h"
#include "layout_a16.h"

using namespace mllmb200;

namespace {

inline int32_t round_nearest_even(float v) { return (int32_t)std::lrintf(v); }

// One row of kai_linear.cpp:729-795 plus the rescale of ":797-805" and the half swap of ":807-816".
void quant_row_a16(const float* src, int k, uint8_t* nib, float* scales, float* zeros) {
  const int nb = (int)blob_num_blocks(k);
  std::memset(nib, 0, blob_nibble_stride(k));
  for (int b = 0; b < nb; ++b) {
    float mn = FLT_MAX, mx = -FLT_MAX;
    const int k0 = b * kGroup, k1 = std::min(k, k0 + kGroup);
    for (int i = k0; i < k1; ++i) {
      mn = std::min(mn, src[i]);
      mx = std::max(mx, src[i]);
    }
    if (mn > 0) mn = 0;
    if (mx < 0) mx = 0;
    const float inv_scale = mx != mn ? (7.0f - -8.0f) / (mx - mn) : 1.0f;
    const float scale = 1.0f / inv_scale;
    const float scaled_min = mn / scale, scaled_max = mx / scale;
    const float zero_point_f = -(scaled_min + -8.0f) < scaled_max + 7.0f ? scaled_min - -8.0f : scaled_max - 7.0f;
    const int32_t zero_point = -round_nearest_even(zero_point_f);
    scales[b] = scale;
    zeros[b] = (-(float)zero_point) * scale;
    const float this_inv_scale = scale != 0 ? 1.0f / scale : 0.0f;
    for (int i = k0; i < k1; ++i) {
      int32_t q = round_nearest_even(src[i] * this_inv_scale) + zero_point;
      q = std::min(std::max(q, -8), 7);
      const uint8_t u = (uint8_t)(q + 8);
      if ((i & 1) == 0) nib[i / 2] |= (uint8_t)(u << 4);
      else nib[i / 2] |= u;
    }
  }
}

int check_shape_a16(int n, int k) {
  if (n <= 0 || k <= 0) return MLLMB200_INVALID_ARG;
  const double bytes = (double)n * ((k + 1) / 2 + blob_num_blocks(k) * 8 + 4) + 64;
  if (bytes >= 2147483648.0) return MLLMB200_UNSUPPORTED;  // tensor sizes are int32 in the reference
  return MLLMB200_OK;
}

}  // namespace

extern "C" {

int mllmb200_w4a16_prepack_size(int N, int K, int has_bias, size_t* bytes) {
  if (!bytes) return MLLMB200_INVALID_ARG;
  if (int st = check_shape_a16(N, K)) return st;
  *bytes = make_blob_header_a16(N, K, has_bias).total_bytes;
  return MLLMB200_OK;
}

int mllmb200_w4a16_blob_offsets(int N, int K, int has_bias, size_t* nibbles_off, size_t* scales_off,
                                size_t* zeros_off, size_t* bias_off) {
  if (int st = check_shape_a16(N, K)) return st;
  const BlobHeader h = make_blob_header_a16(N, K, has_bias);
  if (nibbles_off) *nibbles_off = h.nibbles_off;
  if (scales_off) *scales_off = h.scales_off;
  if (zeros_off) *zeros_off = a16_zeros_off(h);
  if (bias_off) *bias_off = h.bias_off;
  return MLLMB200_OK;
}

int mllmb200_w4a16_quant_prepack(const float* W, const float* bias, int N, int K, void* blob) {
  if (!W || !blob) return MLLMB200_INVALID_ARG;
  if (int st = check_shape_a16(N, K)) return st;
  const BlobHeader h = make_blob_header_a16(N, K, bias != nullptr);
  uint8_t* base = (uint8_t*)blob;
  std::memset(base, 0, h.total_bytes);
  std::memcpy(base, &h, sizeof(h));
  uint8_t* nib = base + h.nibbles_off;
  float* sc = (float*)(base + h.scales_off);
  float* zr = (float*)(base + a16_zeros_off(h));
  const size_t ns = blob_nibble_stride(K), nb = blob_num_blocks(K);
  unsigned nt = std::max(1u, std::min(std::thread::hardware_concurrency(), 16u));
  if ((size_t)N * K < (1u << 18)) nt = 1;
  std::vector<std::thread> pool;
  auto work = [&](int r0, int r1) {
    for (int r = r0; r < r1; ++r) quant_row_a16(W + (size_t)r * K, K, nib + r * ns, sc + r * nb, zr + r * nb);
  };
  const int per = (N + (int)nt - 1) / (int)nt;
  for (unsigned t = 1; t < nt; ++t) {
    const int r0 = std::min(N, (int)t * per), r1 = std::min(N, r0 + per);
    if (r0 < r1) pool.emplace_back(work, r0, r1);
  }
  work(0, std::min(N, per));
  for (auto& t : pool) t.join();
  if (bias) std::memcpy(base + h.bias_off, bias, (size_t)N * 4);
  return MLLMB200_OK;
}

int mllmb200_w4a16_blob_info(const void* blob, size_t blob_bytes, int* N, int* K, int* has_bias) {
  if (!blob || blob_bytes < sizeof(BlobHeader)) return MLLMB200_BAD_BLOB;
  BlobHeader h;
  std::memcpy(&h, blob, sizeof(h));
  if (h.magic != kBlobMagic || h.version != kBlobVersion || h.group != (uint32_t)kGroup || h.layout != kBlobLayoutA16)
    return MLLMB200_BAD_BLOB;
  if (h.n == 0 || h.k == 0) return MLLMB200_BAD_BLOB;
  const BlobHeader e = make_blob_header_a16((int)h.n, (int)h.k, (int)h.has_bias);
  if (e.scales_off != h.scales_off || e.bias_off != h.bias_off || e.total_bytes != h.total_bytes ||
      blob_bytes < h.total_bytes)
    return MLLMB200_BAD_BLOB;
  if (N) *N = (int)h.n;
  if (K) *K = (int)h.k;
  if (has_bias) *has_bias = (int)h.has_bias;
  return MLLMB200_OK;
}

}  // extern "C"
