// Data layouts of the W4A16 sibling path (asymmetric int4 weights with an fp32 scale and an fp32 zero
// term per group of 32, per-block int8 activations, fp16 output).
#pragma once
#include "layout.h"

namespace mllmb200 {

constexpr uint32_t kBlobLayoutA16 = 1;           // BlobHeader.layout of a W4A16 blob
constexpr uint32_t kTiledMagicA16 = 0x3631424Du;  // 'MB16'

// ---- pre-pack blob ----
//   header  BlobHeader (layout = 1, scale_mode = 0)
//   nibbles u8  [N][ceil(K/2)]  byte j = (u[2j] << 4) | u[2j+1], u = q + 8   (the reference's final "s0s1" order)
//   scales  f32 [N][ceil(K/32)]
//   zeros   f32 [N][ceil(K/32)] = -zero_point * scale
//   bias    f32 [N]             only when has_bias
// BlobHeader.scales_off points at the scales; the zeros follow them (16-byte aligned), then the bias.
inline size_t a16_zeros_off(const BlobHeader& h) {
  return align_up(h.scales_off + (size_t)h.n * blob_num_blocks((int)h.k) * 4, 16);
}
inline BlobHeader make_blob_header_a16(int n, int k, int has_bias) {
  BlobHeader h{};
  h.magic = kBlobMagic;
  h.version = kBlobVersion;
  h.n = (uint32_t)n;
  h.k = (uint32_t)k;
  h.group = kGroup;
  h.scale_mode = 0;
  h.has_bias = has_bias ? 1u : 0u;
  h.layout = kBlobLayoutA16;
  h.nibbles_off = sizeof(BlobHeader);
  h.scales_off = align_up(h.nibbles_off + (size_t)n * blob_nibble_stride(k), 16);
  h.bias_off = align_up(a16_zeros_off(h) + (size_t)n * blob_num_blocks(k) * 4, 16);
  h.total_bytes = align_up(h.bias_off + (has_bias ? (size_t)n * 4 : 0), 16);
  return h;
}

// ---- device tile layout ----
// Panels of 32 rows; for panel p and K-group b a 768-byte cell:
//   nibbles: 32 rows x 16 bytes (byte j of a row: k = 2j in the LOW half, 2j+1 in the high half, value q + 8)
//   scales : 32 rows x fp32
//   zeros  : 32 rows x fp32
// cells ordered [panel][group]; then bias[n] (fp32 per padded row, 0 when absent).
// Padding rows and padding k hold nibble 8, scale 0 and zero 0.
constexpr int kCellBytesA16 = kCellNibbleBytes + kPanelRows * 4 + kPanelRows * 4;  // 768

struct TiledHeaderA16 {
  uint32_t magic, version, n, k, num_groups, num_panels, has_bias, reserved;
  uint64_t cells_off, bias_off, total_bytes;
  uint64_t reserved2;
  uint32_t max_weight_bits;  // fp32 bits of max over the matrix of 8 |scale| + |zero| (>= any |weight|); written by the repack
  uint8_t pad[256 - 32 - 32 - 4];
};
static_assert(sizeof(TiledHeaderA16) == 256, "tiled header is 256 bytes");

inline TiledHeaderA16 make_tiled_header_a16(int n, int k, int has_bias) {
  TiledHeaderA16 h{};
  h.magic = kTiledMagicA16;
  h.version = 1;
  h.n = (uint32_t)n;
  h.k = (uint32_t)k;
  h.num_groups = (uint32_t)blob_num_blocks(k);
  h.num_panels = (uint32_t)((n + kPanelRows - 1) / kPanelRows);
  h.has_bias = has_bias ? 1u : 0u;
  h.cells_off = sizeof(TiledHeaderA16);
  h.bias_off = h.cells_off + (size_t)h.num_panels * h.num_groups * kCellBytesA16;
  h.total_bytes = align_up(h.bias_off + (size_t)h.num_panels * kPanelRows * 4, 256);
  return h;
}

// ---- quantized activations ----
// Per K-group b and activation row m a 48-byte record, ordered [group][row] (the rows of a tile are contiguous):
//   words 0..3 : int8 a_q for k = 8i+{0,2,4,6}  (matches the low half-bytes of nibble word i)
//   words 4..7 : int8 a_q for k = 8i+{1,3,5,7}  (matches the high half-bytes)
//   word  8    : sum_{k in b} a_q[k]            (int32)
//   word  9    : the block's scale              (fp32)
//   words 10,11: unused
constexpr int kActRecordBytesA16 = 48;

}  // namespace mllmb200
