// Dynamic per-row int8 activation quantization (reference project:
// tests/Arm/KaiLinearTest.hpp:163-230; production call site
// mllm/Backends/Arm/Kernels/kai_linear.cpp:358-362), as kernels of their own:
//  - act_quant_records_kernel: what the GEMV and the SIMT GEMM consume - per row and K-group a
//    48-byte record {4 words a_q for even k, 4 words a_q for odd k, -8 * sum(a_q), pad} (the byte
//    order the nibble unpack produces, see layout.h) plus one {lhs_scale, a_off} header per row.
//    With `m8_pad > 0` the same kernel writes instead what the tcgen05 GEMM consumes as its B
//    operand: [K-group][row/8][256-byte block], a block being 8 rows x 32 int8 in the canonical
//    K-major core-matrix layout (two 128-byte core matrices, k in the same permuted order).
//  - act_quant_reflayout_kernel: the reference's row layout {float recip, int32 -zp, int8 q[k]},
//    used by the parity tests.
// One CTA per activation row.  The row is read once from global memory and kept in registers
// between the min/max pass and the quantization pass.
#include "device_common.cuh"

namespace mllmb200 {

constexpr int kQuantThreads = 512;
constexpr int kQuantItemsPerThread = 4;  // 8-value items kept in registers: covers K <= 16384

// records: [M][num_groups] x 48 bytes; hdr: [M] {float lhs_scale, int32 a_off (bit pattern)}.
__global__ void __launch_bounds__(kQuantThreads) act_quant_records_kernel(const float* __restrict__ x, int k, int ldx,
                                                                          int num_groups, uint8_t* __restrict__ records,
                                                                          float2* __restrict__ hdr, int use_pdl,
                                                                          int m8_pad) {
  __shared__ float scratch[64];
  if (use_pdl) {
    pdl_launch_dependents();  // the GEMV behind us may start fetching its weights
    pdl_wait_prior();         // x may be the output of the kernel before us
  }
  const int m = blockIdx.x, tid = threadIdx.x;
  const float* row = x + (size_t)m * ldx;
  const int num_items = num_groups * 4;  // item = 8 consecutive k
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
  float v[kQuantItemsPerThread][8];
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
#pragma unroll
  for (int it = 0; it < kQuantItemsPerThread; ++it) {
    const int item = tid + it * kQuantThreads;
    const int k0 = item * 8;
    if (item < num_items && k0 < k) {
      if (vec && k0 + 8 <= k) {
        const float4 a = *reinterpret_cast<const float4*>(row + k0);
        const float4 b = *reinterpret_cast<const float4*>(row + k0 + 4);
        v[it][0] = a.x; v[it][1] = a.y; v[it][2] = a.z; v[it][3] = a.w;
        v[it][4] = b.x; v[it][5] = b.y; v[it][6] = b.z; v[it][7] = b.w;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          mn = fminf(mn, v[it][j]);
          mx = fmaxf(mx, v[it][j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const bool in = k0 + j < k;
          v[it][j] = in ? row[k0 + j] : 0.0f;
          if (in) {
            mn = fminf(mn, v[it][j]);
            mx = fmaxf(mx, v[it][j]);
          }
        }
      }
    }
  }
  // rows longer than the register window: finish the min/max from memory
  for (int kk = kQuantItemsPerThread * kQuantThreads * 8 + tid; kk < k; kk += kQuantThreads) {
    mn = fminf(mn, row[kk]);
    mx = fmaxf(mx, row[kk]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const int warp = tid >> 5, lane = tid & 31;
  if (lane == 0) {
    scratch[warp] = mn;
    scratch[32 + warp] = mx;
  }
  __syncthreads();
  mn = lane < kQuantThreads / 32 ? scratch[lane] : 3.402823466e+38f;
  mx = lane < kQuantThreads / 32 ? scratch[32 + lane] : -3.402823466e+38f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const ActQuantParams p = act_quant_params(mn, mx);
  if (tid == 0) hdr[m] = make_float2(p.recip_scale, __int_as_float(-p.nzp));

  uint8_t* out = records + (size_t)m * num_groups * kActRecordBytes;
  // Packs one 8-value item into its record.  Called by every thread of a warp together (the quad
  // shuffles need full warps); `valid` masks the stores.
  auto emit = [&](int item, bool valid, const int (&q8)[8]) {
    const uint32_t lo = ((uint32_t)q8[0] & 0xFFu) | (((uint32_t)q8[2] & 0xFFu) << 8) |
                        (((uint32_t)q8[4] & 0xFFu) << 16) | (((uint32_t)q8[6] & 0xFFu) << 24);
    const uint32_t hi = ((uint32_t)q8[1] & 0xFFu) | (((uint32_t)q8[3] & 0xFFu) << 8) |
                        (((uint32_t)q8[5] & 0xFFu) << 16) | (((uint32_t)q8[7] & 0xFFu) << 24);
    int s = q8[0] + q8[1] + q8[2] + q8[3] + q8[4] + q8[5] + q8[6] + q8[7];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (valid) {
      const int g = item >> 2, i = item & 3;
      if (m8_pad > 0) {
        uint8_t* blk = records + ((size_t)g * m8_pad + (m >> 3)) * 256;
        *reinterpret_cast<uint2*>(blk + (i >> 1) * 128 + (m & 7) * 16 + (i & 1) * 8) = make_uint2(lo, hi);
      } else {
        uint32_t* rec = reinterpret_cast<uint32_t*>(out + (size_t)g * kActRecordBytes);
        rec[i] = lo;
        rec[4 + i] = hi;
        if (i == 0) *reinterpret_cast<uint4*>(rec + 8) = make_uint4((uint32_t)(-8 * s), 0u, 0u, 0u);
      }
    }
  };
  // items held in registers (trip count is a compile-time constant: full warps at the shuffles)
#pragma unroll
  for (int it = 0; it < kQuantItemsPerThread; ++it) {
    const int item = tid + it * kQuantThreads;
    if (it * kQuantThreads >= num_items) break;  // uniform over the CTA
    const bool valid = item < num_items;
    const int k0 = item * 8;
    int q8[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q8[j] = (valid && k0 + j < k) ? act_quant_value(v[it][j], p) : 0;
    emit(item, valid, q8);
  }
  // rows longer than the register window: the rest comes from memory (uniform trip count)
  for (int base = kQuantItemsPerThread * kQuantThreads; base < num_items; base += kQuantThreads) {
    const int item = base + tid;
    const bool valid = item < num_items;
    const int k0 = item * 8;
    int q8[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q8[j] = (valid && k0 + j < k) ? act_quant_value(row[k0 + j], p) : 0;
    emit(item, valid, q8);
  }
}

// The tcgen05 GEMM's B operand: [K-group][row/8][256-byte block], a block = 8 rows x 32 int8 as two
// 128-byte core matrices (row r at byte r*16 of each).  One CTA quantizes 8 consecutive rows, one
// warp per row, so that every 256-byte block is written whole by one CTA (a one-row-per-CTA kernel
// scatters 8-byte pieces 16 KB apart and was measured at 545 us for M=512, K=8192).
// Pass 1: coalesced read of the row for min/max; pass 2: lane = K-group, 32 consecutive floats each.
// Four warps share a row (each scans a quarter of it; the partial min/max meet in shared memory).
// grid = ceil(M/8), block = 1024 (8 rows x 4 warps).
constexpr int kBlocksWarpsPerRow = 4;
__global__ void __launch_bounds__(8 * kBlocksWarpsPerRow * 32) act_quant_blocks_kernel(
    const float* __restrict__ x, int m_total, int k, int ldx, int num_groups, int m8_pad, uint8_t* __restrict__ blocks,
    float2* __restrict__ hdr) {
  __shared__ float s_mm[8][kBlocksWarpsPerRow][2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = warp & 7, part = warp >> 3;
  const int m = blockIdx.x * 8 + r;
  const bool live = m < m_total;  // padding rows are never read back
  const float* row = x + (size_t)(live ? m : 0) * ldx;
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
  if (live) {
    const int stride = 32 * kBlocksWarpsPerRow, first = part * 32 + lane;
    if (vec) {
      const float4* r4 = reinterpret_cast<const float4*>(row);
      for (int i = first; i < (k >> 2); i += stride) {
        const float4 v = r4[i];
        mn = fminf(mn, fminf(fminf(v.x, v.y), fminf(v.z, v.w)));
        mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
      }
      for (int i = (k & ~3) + first; i < k; i += stride) {
        mn = fminf(mn, row[i]);
        mx = fmaxf(mx, row[i]);
      }
    } else {
      for (int i = first; i < k; i += stride) {
        mn = fminf(mn, row[i]);
        mx = fmaxf(mx, row[i]);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0) {
    s_mm[r][part][0] = mn;
    s_mm[r][part][1] = mx;
  }
  __syncthreads();
  if (!live) return;
#pragma unroll
  for (int q = 0; q < kBlocksWarpsPerRow; ++q) {
    mn = fminf(mn, s_mm[r][q][0]);
    mx = fmaxf(mx, s_mm[r][q][1]);
  }
  const ActQuantParams p = act_quant_params(mn, mx);
  if (lane == 0 && part == 0) hdr[m] = make_float2(p.recip_scale, __int_as_float(-p.nzp));
  // one thread per (K-group, 16-byte K chunk): twice the parallelism of one thread per group
  for (int it = part * 32 + lane; it < num_groups * 2; it += 32 * kBlocksWarpsPerRow) {
    const int g = it >> 1, c = it & 1;
    const int k0 = g * kGroup + c * 16;
    uint32_t w[4];  // lo hi lo hi: the chunk's 16 elements in the order the nibble masks produce
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float f[8];
      if (vec && k0 + i * 8 + 8 <= k) {
        const float4 a = *reinterpret_cast<const float4*>(row + k0 + i * 8);
        const float4 b = *reinterpret_cast<const float4*>(row + k0 + i * 8 + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = (k0 + i * 8 + j < k) ? row[k0 + i * 8 + j] : 0.0f;
      }
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t q = (k0 + i * 8 + j < k) ? ((uint32_t)act_quant_value(f[j], p) & 0xFFu) : 0u;
        if (j & 1) hi |= q << (8 * (j >> 1));
        else lo |= q << (8 * (j >> 1));
      }
      w[2 * i] = lo;
      w[2 * i + 1] = hi;
    }
    uint8_t* blk = blocks + ((size_t)g * m8_pad + (m >> 3)) * 256 + (m & 7) * 16;
    *reinterpret_cast<uint4*>(blk + c * 128) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

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

// The same for the fp16 tensor-core path (gemm_tcf16.cu): the zero-point-corrected values a_q + a_off
// are written as fp16 (exact) in 512-byte canonical K-major blocks [group][row / 8]: 4 chunks of 128 bytes, chunk c =
// 8 rows x 16 bytes holding k = 8c + {0,4,1,5,2,6,3,7} - the order in which the weight side's
// nibble unpack (two nibbles 16 bits apart per half2) produces its elements.
constexpr int kF16RowsPerCta = 4;   // rows 4i .. 4i+3 sit side by side in a block: 64-byte pieces
constexpr int kF16WarpsPerRow = 8;
__global__ void __launch_bounds__(kF16RowsPerCta * kF16WarpsPerRow * 32) act_quant_blocks_f16_kernel(
    const float* __restrict__ x, int m_total, int k, int ldx, int num_groups, int m8_pad, uint8_t* __restrict__ blocks,
    float2* __restrict__ hdr, int use_pdl, int* __restrict__ clear_ints, int clear_count) {
  __shared__ float s_mm[kF16RowsPerCta][kF16WarpsPerRow][2];
  if (use_pdl) {
    // x may be the previous kernel's output, and that kernel may still be reading the blocks this one overwrites:
    // nothing happens before it has finished; the kernel behind this one may set itself up meanwhile
    pdl_launch_dependents();
    pdl_wait_prior();
  }
  // the K-split counters of the GEMM behind this kernel (it reads them only after this grid has finished)
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i < clear_count; i += blockDim.x) clear_ints[i] = 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = warp & (kF16RowsPerCta - 1), part = warp / kF16RowsPerCta;
  const int m = blockIdx.x * kF16RowsPerCta + r;
  const bool live = m < m_total;
  const float* row = x + (size_t)(live ? m : 0) * ldx;
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
  if (live) {
    const int stride = 32 * kF16WarpsPerRow, first = part * 32 + lane;
    if (vec) {
      const float4* r4 = reinterpret_cast<const float4*>(row);
      for (int i = first; i < (k >> 2); i += stride) {
        const float4 v = r4[i];
        mn = fminf(mn, fminf(fminf(v.x, v.y), fminf(v.z, v.w)));
        mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
      }
      for (int i = (k & ~3) + first; i < k; i += stride) {
        mn = fminf(mn, row[i]);
        mx = fmaxf(mx, row[i]);
      }
    } else {
      for (int i = first; i < k; i += stride) {
        mn = fminf(mn, row[i]);
        mx = fmaxf(mx, row[i]);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0) {
    s_mm[r][part][0] = mn;
    s_mm[r][part][1] = mx;
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < kF16WarpsPerRow; ++q) {
    mn = fminf(mn, s_mm[r][q][0]);
    mx = fmaxf(mx, s_mm[r][q][1]);
  }
  const ActQuantParams p = act_quant_params(mn, mx);
  if (live && lane == 0 && part == 0) hdr[m] = make_float2(p.recip_scale, __int_as_float(-p.nzp));
  // padding rows (m >= m_total, inside the padded tile) are written as zeros: the tensor core reads them.
  // One thread per (K-group, 8-element chunk): 4 x the parallelism of one thread per group.
  for (int it = part * 32 + lane; it < num_groups * 4; it += 32 * kF16WarpsPerRow) {
    const int g = it >> 2, c = it & 3;
    const int kc = g * kGroup + c * 8;
    uint8_t* blk = blocks + ((size_t)g * m8_pad + (m >> 3)) * 512 + (m & 7) * 16;
    float f[8];
    if (live && vec && kc + 8 <= k) {
      const float4 a = *reinterpret_cast<const float4*>(row + kc);
      const float4 b = *reinterpret_cast<const float4*>(row + kc + 4);
      f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
    } else {
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) f[jj] = (live && kc + jj < k) ? row[kc + jj] : 0.0f;
    }
    __align__(16) __half h[8];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      // a_q + a_off (= a_q - zero point), |.| <= 255: exact in fp16, and exactly the factor the reference
      // multiplies the weight with, so no zero-point correction term (and none of its cancellation) is left
      const int q = (live && kc + jj < k) ? act_quant_value(f[jj], p) - p.nzp : 0;
      const int pos = (jj < 4) ? 2 * jj : 2 * (jj - 4) + 1;  // chunk order {0,4,1,5,2,6,3,7}
      h[pos] = __int2half_rn(q);
    }
    *reinterpret_cast<uint4*>(blk + c * 128) = *reinterpret_cast<const uint4*>(h);
  }
}

cudaError_t launch_act_quant_blocks_f16(const float* x, int m, int m_pad, int k, int ldx, uint8_t* blocks, float2* hdr,
                                        cudaStream_t stream, int use_pdl, int* clear_ints, int clear_count) {
  const int num_groups = (k + kGroup - 1) / kGroup;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(m_pad / kF16RowsPerCta), 1, 1);
  cfg.blockDim = dim3(kF16RowsPerCta * kF16WarpsPerRow * 32, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  if (use_pdl) {
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, act_quant_blocks_f16_kernel, x, m, k, ldx, num_groups, m_pad / 8, blocks, hdr, use_pdl,
                            clear_ints, clear_ints != nullptr ? clear_count : 0);
}

// m8_pad == 0: 48-byte records; m8_pad > 0: canonical 256-byte blocks with m8_pad blocks per K-group.
cudaError_t launch_act_quant_records(const float* x, int m, int k, int ldx, uint8_t* records, float2* hdr, int use_pdl,
                                     int m8_pad, cudaStream_t stream) {
  const int num_groups = (k + kGroup - 1) / kGroup;
  if (m8_pad > 0) {
    act_quant_blocks_kernel<<<(m + 7) / 8, 8 * kBlocksWarpsPerRow * 32, 0, stream>>>(x, m, k, ldx, num_groups, m8_pad, records, hdr);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)m, 1, 1);
  cfg.blockDim = dim3(kQuantThreads, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  if (use_pdl) {
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, act_quant_records_kernel, x, k, ldx, num_groups, records, hdr, use_pdl, m8_pad);
}

}  // namespace mllmb200
