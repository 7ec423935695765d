// Data layouts shared by host packing code and device kernels.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace mllmb200 {

constexpr uint32_t kBlobMagic = 0x5732424Du;   // 'MB2W' little-endian
constexpr uint32_t kBlobVersion = 1;
constexpr uint32_t kTiledMagic = 0x5432424Du;  // 'MB2T'
constexpr int kGroup = 32;                      // K elements per scale group

// ---- pre-pack blob (host side, stored in .mllm parameter files) ----
struct BlobHeader {
  uint32_t magic, version, n, k, group, scale_mode, has_bias, layout;
  uint64_t nibbles_off, scales_off, bias_off, total_bytes;
};
static_assert(sizeof(BlobHeader) == 64, "blob header is 64 bytes");

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline size_t blob_nibble_stride(int k) { return (size_t)(k + 1) / 2; }
inline size_t blob_num_blocks(int k) { return (size_t)(k + kGroup - 1) / kGroup; }

inline BlobHeader make_blob_header(int n, int k, int scale_mode, int has_bias) {
  BlobHeader h{};
  h.magic = kBlobMagic;
  h.version = kBlobVersion;
  h.n = (uint32_t)n;
  h.k = (uint32_t)k;
  h.group = kGroup;
  h.scale_mode = (uint32_t)scale_mode;
  h.has_bias = has_bias ? 1u : 0u;
  h.layout = 0;
  h.nibbles_off = sizeof(BlobHeader);
  h.scales_off = align_up(h.nibbles_off + (size_t)n * blob_nibble_stride(k), 16);
  h.bias_off = align_up(h.scales_off + (size_t)n * blob_num_blocks(k) * 2, 16);
  h.total_bytes = align_up(h.bias_off + (has_bias ? (size_t)n * 4 : 0), 16);
  return h;
}

// ---- device tile layout ----
// Rows are grouped into panels of 32.  For panel p and K-group b the "cell" holds
//   nibbles: 32 rows x 16 bytes  (row r at byte r*16; byte j = k 2j (low half) and 2j+1 (high half), value q+8)
//   scales : 32 rows x 2 bytes
// = 576 bytes, cells ordered [panel][group].  A warp reads one cell with one 16-byte load per lane,
// every byte of it used; a CTA's share of a panel is one contiguous byte range, so it moves with a
// few bulk copies.  Padding rows (N not a multiple of 32) and padding k (K not a multiple of 32)
// hold nibble 8 (= weight 0) and scale 0.
// After the cells: zsum[n] = sum_b scale[n,b] * sum_{k in b} (u[n,k]-8)   (fp32, per padded row)
//                  bias[n]                                                 (fp32, 0 when absent)
constexpr int kPanelRows = 32;
constexpr int kCellNibbleBytes = kPanelRows * 16;
constexpr int kCellScaleBytes = kPanelRows * 2;
constexpr int kCellBytes = kCellNibbleBytes + kCellScaleBytes;  // 576

struct TiledHeader {
  uint32_t magic, version, n, k, num_groups, num_panels, scale_mode, has_bias;
  uint64_t cells_off, zsum_off, bias_off, total_bytes;
  uint32_t max_scale_bits;  // fp32 bits of the largest |group scale| of the matrix (written by the repack kernel)
  uint8_t pad[256 - 32 - 32 - 4];
};
static_assert(sizeof(TiledHeader) == 256, "tiled header is 256 bytes");

inline TiledHeader make_tiled_header(int n, int k, int scale_mode, int has_bias) {
  TiledHeader h{};
  h.magic = kTiledMagic;
  h.version = 1;
  h.n = (uint32_t)n;
  h.k = (uint32_t)k;
  h.num_groups = (uint32_t)blob_num_blocks(k);
  h.num_panels = (uint32_t)((n + kPanelRows - 1) / kPanelRows);
  h.scale_mode = (uint32_t)scale_mode;
  h.has_bias = has_bias ? 1u : 0u;
  h.cells_off = sizeof(TiledHeader);
  h.zsum_off = h.cells_off + (size_t)h.num_panels * h.num_groups * kCellBytes;
  h.bias_off = h.zsum_off + (size_t)h.num_panels * kPanelRows * 4;
  h.total_bytes = align_up(h.bias_off + (size_t)h.num_panels * kPanelRows * 4, 256);
  return h;
}

// ---- quantized activation workspace (GEMM path) ----
// Per activation row m and K-group b a 48-byte record:
//   words 0..3 : int8 a_q for k = 8i+{0,2,4,6}   (i = word index; matches the low half-bytes of nibble word i)
//   words 4..7 : int8 a_q for k = 8i+{1,3,5,7}   (matches the high half-bytes)
//   word  8    : -8 * sum_{k in b} a_q[k]        (turns the unsigned-nibble dot product into the signed one)
//   words 9..11: unused
// Padding k (beyond K) holds a_q = 0.  Then per row {float lhs_scale, int32 a_off}.
constexpr int kActRecordBytes = 48;

}  // namespace mllmb200
