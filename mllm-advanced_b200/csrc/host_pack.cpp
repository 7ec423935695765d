// Host side of the C ABI: weight quantization and the pre-pack blob.
// Arithmetic follows mllm/Backends/Arm/Kernels/kai_linear.cpp:220-291 (reference project paths)
// and must stay bit-identical to it; tests compare against the CPU oracle.
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/mllmb200.h"
#include "layout.h"

using namespace mllmb200;

namespace {

inline uint16_t f32_to_bf16_trunc(float f) {
  uint32_t b;
  std::memcpy(&b, &f, 4);
  return (uint16_t)(b >> 16);
}
inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t b;
  std::memcpy(&b, &f, 4);
  if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x40u);
  b += 0x7fffu + ((b >> 16) & 1u);
  return (uint16_t)(b >> 16);
}
inline uint16_t f32_to_f16_rne(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0u));
  if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
  if (x < 0x33000001u) return (uint16_t)sign;
  const int32_t e = (int32_t)(x >> 23) - 127;
  const uint32_t m = (x & 0x7fffffu) | 0x800000u;
  if (e < -14) {
    const uint32_t shift = (uint32_t)(13 + (-14 - e));
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | q);
  }
  uint32_t q = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3ffu);
  const uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
  return (uint16_t)(sign | q);
}
inline uint16_t encode_scale(float s, int mode) {
  switch (mode) {
    case MLLMB200_SCALE_BF16_RNE: return f32_to_bf16_rne(s);
    case MLLMB200_SCALE_FP16: return f32_to_f16_rne(s);
    default: return f32_to_bf16_trunc(s);
  }
}

// One row of kai_linear.cpp:236-289.
void quant_row(const float* src, int k, uint8_t* nib, uint16_t* scales, int mode) {
  const int nb = (int)blob_num_blocks(k);
  std::memset(nib, 0, blob_nibble_stride(k));
  for (int b = 0; b < nb; ++b) {
    float amax = 0.0f, mx = 0.0f;
    const int k0 = b * kGroup, k1 = std::min(k, k0 + kGroup);
    for (int i = k0; i < k1; ++i) {
      const float v = src[i], a = std::fabs(v);
      if (amax < a) { amax = a; mx = v; }
    }
    const float scale = (float)((double)mx / -8.0);
    const float recip = scale ? 1.0f / scale : 0.0f;
    scales[b] = encode_scale(scale, mode);
    for (int i = k0; i < k1; ++i) {
      int32_t q = (int32_t)std::round(src[i] * recip);
      q = std::max(q, -8);
      q = std::min(q, 7);
      const uint8_t u = (uint8_t)(q + 8);
      if ((i & 1) == 0) nib[i / 2] = u;
      else nib[i / 2] |= (uint8_t)(u << 4);
    }
  }
}

int check_shape(int n, int k) {
  if (n <= 0 || k <= 0) return MLLMB200_INVALID_ARG;
  // single blobs stay below 2 GiB: the reference keeps tensor sizes in int32
  // (mllm/Backends/Arm/Passes/KaiQuantizationPass.cpp:167).
  const double bytes = (double)n * ((k + 1) / 2 + blob_num_blocks(k) * 2 + 4) + 64;
  if (bytes >= 2147483648.0) return MLLMB200_UNSUPPORTED;
  return MLLMB200_OK;
}

}  // namespace

extern "C" {

int mllmb200_w4a32_prepack_size(int N, int K, int has_bias, size_t* bytes) {
  if (!bytes) return MLLMB200_INVALID_ARG;
  if (int st = check_shape(N, K)) return st;
  *bytes = make_blob_header(N, K, 0, has_bias).total_bytes;
  return MLLMB200_OK;
}

int mllmb200_w4a32_blob_offsets(int N, int K, int has_bias, size_t* nibbles_off, size_t* scales_off,
                                size_t* bias_off) {
  if (int st = check_shape(N, K)) return st;
  const BlobHeader h = make_blob_header(N, K, 0, has_bias);
  if (nibbles_off) *nibbles_off = h.nibbles_off;
  if (scales_off) *scales_off = h.scales_off;
  if (bias_off) *bias_off = h.bias_off;
  return MLLMB200_OK;
}

int mllmb200_w4a32_quant_prepack(const float* W, const float* bias, int N, int K, int scale_mode, void* blob) {
  if (!W || !blob) return MLLMB200_INVALID_ARG;
  if (scale_mode < 0 || scale_mode > 2) return MLLMB200_INVALID_ARG;
  if (int st = check_shape(N, K)) return st;
  const BlobHeader h = make_blob_header(N, K, scale_mode, bias != nullptr);
  uint8_t* base = (uint8_t*)blob;
  std::memset(base, 0, h.total_bytes);
  std::memcpy(base, &h, sizeof(h));
  uint8_t* nib = base + h.nibbles_off;
  uint16_t* sc = (uint16_t*)(base + h.scales_off);
  const size_t ns = blob_nibble_stride(K), nb = blob_num_blocks(K);
  // rows are independent: spread them over host threads (the reference runs this loop on one).
  unsigned nt = std::max(1u, std::min(std::thread::hardware_concurrency(), 16u));
  if ((size_t)N * K < (1u << 18)) nt = 1;
  std::vector<std::thread> pool;
  auto work = [&](int r0, int r1) {
    for (int r = r0; r < r1; ++r) quant_row(W + (size_t)r * K, K, nib + r * ns, sc + r * nb, scale_mode);
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

int mllmb200_w4a32_prepack_from_quantized(const uint8_t* nibbles, const uint16_t* scales, const float* bias,
                                          int N, int K, int scale_mode, void* blob) {
  if (!nibbles || !scales || !blob) return MLLMB200_INVALID_ARG;
  if (scale_mode < 0 || scale_mode > 2) return MLLMB200_INVALID_ARG;
  if (int st = check_shape(N, K)) return st;
  const BlobHeader h = make_blob_header(N, K, scale_mode, bias != nullptr);
  uint8_t* base = (uint8_t*)blob;
  std::memset(base, 0, h.total_bytes);
  std::memcpy(base, &h, sizeof(h));
  std::memcpy(base + h.nibbles_off, nibbles, (size_t)N * blob_nibble_stride(K));
  std::memcpy(base + h.scales_off, scales, (size_t)N * blob_num_blocks(K) * 2);
  if (bias) std::memcpy(base + h.bias_off, bias, (size_t)N * 4);
  return MLLMB200_OK;
}

int mllmb200_w4a32_blob_info(const void* blob, size_t blob_bytes, int* N, int* K, int* scale_mode, int* has_bias) {
  if (!blob || blob_bytes < sizeof(BlobHeader)) return MLLMB200_BAD_BLOB;
  BlobHeader h;
  std::memcpy(&h, blob, sizeof(h));
  if (h.magic != kBlobMagic || h.version != kBlobVersion || h.group != (uint32_t)kGroup || h.layout != 0)
    return MLLMB200_BAD_BLOB;
  if (h.n == 0 || h.k == 0 || h.scale_mode > 2) return MLLMB200_BAD_BLOB;
  const BlobHeader e = make_blob_header((int)h.n, (int)h.k, (int)h.scale_mode, (int)h.has_bias);
  if (e.nibbles_off != h.nibbles_off || e.scales_off != h.scales_off || e.bias_off != h.bias_off ||
      e.total_bytes != h.total_bytes || blob_bytes < h.total_bytes)
    return MLLMB200_BAD_BLOB;
  if (N) *N = (int)h.n;
  if (K) *K = (int)h.k;
  if (scale_mode) *scale_mode = (int)h.scale_mode;
  if (has_bias) *has_bias = (int)h.has_bias;
  return MLLMB200_OK;
}

const char* mllmb200_status_str(int status) {
  switch (status) {
    case MLLMB200_OK: return "ok";
    case MLLMB200_INVALID_ARG: return "invalid argument";
    case MLLMB200_UNSUPPORTED: return "unsupported shape or mode";
    case MLLMB200_CUDA_ERROR: return "CUDA runtime error";
    case MLLMB200_TIMEOUT: return "device-side wait timed out";
    case MLLMB200_BAD_BLOB: return "pre-pack blob header mismatch";
    case MLLMB200_TOO_LARGE: return "request exceeds a fixed capacity";
    default: return "unknown status";
  }
}

int mllmb200_version(void) { return 100; }

}  // extern "C"
