// Device repacker: reference pre-pack layout (row-major nibbles + per-group scales + bias, see
// layout.h / mllm/Backends/Arm/Kernels/kai_linear.cpp:276-287 of the reference project) into
// the 32-row-panel tile layout the GEMV/GEMM kernels stream, and its inverse.
#include "device_common.cuh"

namespace mllmb200 {

__device__ unsigned int g_device_status = 0;

// One thread per (row in shard, K-group): moves the group's 16 nibble bytes and its scale.
__global__ void repack_cells_kernel(const uint8_t* __restrict__ nibbles, const uint16_t* __restrict__ scales,
                                    int k, int row_begin, int row_count, int num_groups, int num_panels,
                                    uint8_t* __restrict__ cells) {
  const long long total = (long long)num_panels * num_groups * kPanelRows;
  const size_t nib_stride = (size_t)(k + 1) / 2;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(idx % kPanelRows);
    const long long cell = idx / kPanelRows;
    const int b = (int)(cell % num_groups);
    const int p = (int)(cell / num_groups);
    const int row = p * kPanelRows + r;  // row inside the shard
    uint32_t w[4] = {0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};
    uint16_t s = 0;
    if (row < row_count) {
      const size_t src_row = (size_t)(row_begin + row);
      const uint8_t* src = nibbles + src_row * nib_stride + (size_t)b * 16;
      const int valid_k = min(kGroup, k - b * kGroup);  // elements of this group that exist
      const int full_bytes = valid_k >> 1;
      if (valid_k == kGroup && ((reinterpret_cast<uintptr_t>(src) & 15u) == 0)) {
        const uint4 v = *reinterpret_cast<const uint4*>(src);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
      } else {
        uint8_t* wb = reinterpret_cast<uint8_t*>(w);
        for (int j = 0; j < full_bytes; ++j) wb[j] = src[j];
        if (valid_k & 1) wb[full_bytes] = (uint8_t)((src[full_bytes] & 0x0F) | 0x80);  // unused half = weight 0
      }
      s = scales[src_row * num_groups + b];
    }
    uint8_t* dst = cells + (size_t)cell * kCellBytes;
    *reinterpret_cast<uint4*>(dst + r * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint16_t*>(dst + kCellNibbleBytes + r * 2) = s;
  }
}

// One warp per padded row: zsum[row] = sum_b scale[row,b] * sum_{k in b}(u-8), accumulated in fp64 in
// a fixed order, rounded once to fp32; and the bias copy.
__global__ void repack_rowdata_kernel(const uint8_t* __restrict__ cells, const float* __restrict__ bias_src,
                                      int row_begin, int row_count, int num_groups, int num_panels,
                                      uint32_t scale_mode, float* __restrict__ zsum, float* __restrict__ bias_dst,
                                      unsigned int* __restrict__ max_scale_bits) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int padded_rows = num_panels * kPanelRows;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < padded_rows;
       row += gridDim.x * warps_per_block) {
    const int p = row / kPanelRows, r = row % kPanelRows;
    double acc = 0.0;
    float smax = 0.0f;  // largest finite |scale| of the row (the fp16 tensor-core path scales by a power of two from it)
    for (int b = lane; b < num_groups; b += 32) {
      const uint8_t* cell = cells + ((size_t)p * num_groups + b) * kCellBytes;
      const uint4 v = *reinterpret_cast<const uint4*>(cell + r * 16);
      const uint32_t raw = *reinterpret_cast<const uint16_t*>(cell + kCellNibbleBytes + r * 2);
      const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
      int sum = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = ws[i] & 0x0F0F0F0Fu, hi = (ws[i] >> 4) & 0x0F0F0F0Fu;
        sum = __dp4a((int)lo, 0x01010101, sum);
        sum = __dp4a((int)hi, 0x01010101, sum);
      }
      sum -= 8 * kGroup;
      const float s = decode_scale(raw, scale_mode);
      acc += (double)s * (double)sum;
      if (fabsf(s) <= 3.402823466e+38f) smax = fmaxf(smax, fabsf(s));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      acc += __shfl_xor_sync(0xffffffffu, acc, o);
      smax = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, o));
    }
    if (lane == 0) {
      if (max_scale_bits != nullptr && row < row_count) atomicMax(max_scale_bits, __float_as_uint(smax));  // non-negative floats order as integers
      zsum[row] = (float)acc;
      bias_dst[row] = (bias_src != nullptr && row < row_count) ? bias_src[row_begin + row] : 0.0f;
    }
  }
}

// Inverse mapping: tile layout -> blob sections for `row_count` rows.
__global__ void unpack_cells_kernel(const uint8_t* __restrict__ cells, int k, int row_count, int num_groups,
                                    int num_panels, uint8_t* __restrict__ nibbles, uint16_t* __restrict__ scales) {
  const long long total = (long long)num_panels * num_groups * kPanelRows;
  const size_t nib_stride = (size_t)(k + 1) / 2;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(idx % kPanelRows);
    const long long cell = idx / kPanelRows;
    const int b = (int)(cell % num_groups);
    const int p = (int)(cell / num_groups);
    const int row = p * kPanelRows + r;
    if (row >= row_count) continue;
    const uint8_t* src = cells + (size_t)cell * kCellBytes;
    const uint8_t* wb = src + r * 16;
    uint8_t* dst = nibbles + (size_t)row * nib_stride + (size_t)b * 16;
    const int valid_k = min(kGroup, k - b * kGroup);
    const int full_bytes = valid_k >> 1;
    for (int j = 0; j < full_bytes; ++j) dst[j] = wb[j];
    if (valid_k & 1) dst[full_bytes] = (uint8_t)(wb[full_bytes] & 0x0F);  // the reference leaves the unused half 0
    scales[(size_t)row * num_groups + b] = *reinterpret_cast<const uint16_t*>(src + kCellNibbleBytes + r * 2);
  }
}

__global__ void unpack_bias_kernel(const float* __restrict__ bias_src, int row_count, float* __restrict__ bias_dst) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < row_count; i += gridDim.x * blockDim.x)
    bias_dst[i] = bias_src[i];
}

}  // namespace mllmb200
