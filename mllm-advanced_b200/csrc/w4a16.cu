// W4A16 sibling of the quantized linear: asymmetric int4 weights (fp32 scale + fp32 zero term per group of
// 32), activations quantized per 32-element block to symmetric int8 with an fp32 scale, fp16 output.
// Stands in for KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk (reference project:
// mllm/Backends/Arm/Kernels/kai_linear.cpp:680-951):
//   y[m,n] = fp16( clamp( sum_b a_s[m,b] * ( s[n,b] * float(dot_b) + z[n,b] * float(sum_b) ) + bias[n] ) )
//   dot_b = sum_{k in b} a_q[m,k] * (u[n,k] - 8),  sum_b = sum_{k in b} a_q[m,k]
// Kernels here: the repack (blob -> 768-byte cells), and three ways through the product, chosen by M in
// launch_w4a16_linear:
//   a16_gemv_fused_kernel            M <= 4 on small matrices: one launch, quantization inside, cluster K-split
//   a16_act_quant_kernel + a16_linear_kernel (+ a16_finish_kernel)   48-byte records, dp4a, any M
//   a16_act_quant_blocks_f16_kernel + the tcgen05 fp16 GEMM of gemm_tcf16.cu (A16 instantiation)   M >= 64
// In the dp4a kernels a CTA owns one 32-row panel (lane = output row) and its 8 warps split the K groups.
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/mllmb200.h"
#include "device_common.cuh"
#include "layout_a16.h"

namespace cg = cooperative_groups;

namespace mllmb200 {

// ------------------------------------------------------------------ repack
// One warp per (panel, group) cell, lane = row of the panel.
__global__ void a16_repack_cells_kernel(const uint8_t* __restrict__ nib, const float* __restrict__ scales,
                                        const float* __restrict__ zeros, int k, int row_begin, int row_count,
                                        int num_groups, int num_panels, uint8_t* __restrict__ cells,
                                        unsigned int* __restrict__ max_weight_bits) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= num_panels * num_groups) return;
  const int panel = warp / num_groups, g = warp % num_groups;
  const int r = panel * kPanelRows + lane;
  const bool row_ok = r < row_count;
  const size_t stride = (size_t)(k + 1) / 2;
  const size_t src_row = (size_t)(row_begin + r);
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kk = g * kGroup + (i * 4 + j) * 2;  // even k of this byte
      uint32_t lo = 8, hi = 8;                       // padding: weight 0
      if (row_ok && kk < k) {
        const uint32_t b = nib[src_row * stride + (size_t)(kk >> 1)];
        lo = b >> 4;  // the blob keeps the even k in the high half
        if (kk + 1 < k) hi = b & 15u;
      }
      word |= (lo | (hi << 4)) << (8 * j);
    }
    w[i] = word;
  }
  uint8_t* cell = cells + (size_t)warp * kCellBytesA16;
  reinterpret_cast<uint4*>(cell)[lane] = make_uint4(w[0], w[1], w[2], w[3]);
  float s = 0.0f, z = 0.0f;
  if (row_ok) {
    s = scales[src_row * num_groups + g];
    z = zeros[src_row * num_groups + g];
  }
  reinterpret_cast<float*>(cell + kCellNibbleBytes)[lane] = s;
  reinterpret_cast<float*>(cell + kCellNibbleBytes + kPanelRows * 4)[lane] = z;
  // 8 |s| + |z| bounds every |weight| of the group; the tensor-core path scales the matrix by it
  float bound = fmaf(8.0f, fabsf(s), fabsf(z));
  if (!(bound < 3.0e38f)) bound = 0.0f;  // inf / nan scales are not used for the range
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) bound = fmaxf(bound, __shfl_xor_sync(0xffffffffu, bound, o));
  if (lane == 0 && bound > 0.0f) atomicMax(max_weight_bits, __float_as_uint(bound));  // positive floats order as their bits
}

__global__ void a16_repack_bias_kernel(const float* __restrict__ bias, int row_begin, int row_count, int padded,
                                       float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < padded) out[i] = (bias && i < row_count) ? bias[row_begin + i] : 0.0f;
}

// ------------------------------------------------------------------ activation quantization
// grid (ceil(groups / 32), M), 256 threads: a warp takes 4 groups, 8 lanes per group, 4 consecutive k per lane.
template <typename T>
__device__ __forceinline__ float a16_load(const T* p);
template <>
__device__ __forceinline__ float a16_load<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float a16_load<__half>(const __half* p) { return __half2float(*p); }

template <typename T>
__global__ void __launch_bounds__(256) a16_act_quant_kernel(const T* __restrict__ x, int k, int ldx, int num_groups,
                                                            uint8_t* __restrict__ recs) {
  const int m = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = blockIdx.x * 32 + warp * 4 + (lane >> 3);
  const int j = lane & 7;  // which 4 of the group's 32 elements
  const T* row = x + (size_t)m * ldx;
  float v[4];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int kk = g * kGroup + j * 4 + i;
    v[i] = (g < num_groups && kk < k) ? a16_load<T>(row + kk) : 0.0f;
    amax = fmaxf(amax, fabsf(v[i]));
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = __fdiv_rn(amax, 127.0f);
  const float recip = scale != 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
  int q[4], sum = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float r = roundf(__fmul_rn(v[i], recip));  // half away from zero
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    q[i] = (int)r;
    sum += q[i];
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  // this lane: k = 4j..4j+3 of the group -> even k {0,2} and odd k {1,3} halves of word j/2 and word 4 + j/2
  const uint32_t ev = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[2] & 0xff) << 8);
  const uint32_t od = (uint32_t)(q[1] & 0xff) | ((uint32_t)(q[3] & 0xff) << 8);
  const uint32_t ev_p = __shfl_xor_sync(0xffffffffu, ev, 1), od_p = __shfl_xor_sync(0xffffffffu, od, 1);
  if (g >= num_groups) return;
  uint32_t* rec = reinterpret_cast<uint32_t*>(recs + ((size_t)g * gridDim.y + m) * kActRecordBytesA16);  // [group][row]
  if ((j & 1) == 0) rec[j >> 1] = ev | (ev_p << 16);
  else rec[4 + (j >> 1)] = od_p | (od << 16);
  if (j == 0) {
    rec[8] = (uint32_t)sum;
    rec[9] = __float_as_uint(scale);
  }
}

// The same quantization for the tensor-core path: the de-quantized values a_q * a_s, rounded once to fp16,
// in the 512-byte K-major operand blocks [group][row / 8] of gemm_tcf16.cu (4 chunks of 8 rows x 16 bytes,
// chunk c = k 8c + {0,4,1,5,2,6,3,7}).  One CTA per (padded) row, one thread per 8-element chunk; the four
// chunk threads of a group sit in adjacent lanes.  Padding rows are written as zeros.
template <typename T>
__global__ void __launch_bounds__(256) a16_act_quant_blocks_f16_kernel(const T* __restrict__ x, int m_total, int k,
                                                                       int ldx, int num_groups, int m8_pad,
                                                                       uint8_t* __restrict__ blocks) {
  const int m = blockIdx.x;
  const bool live = m < m_total;
  const T* row = x + (size_t)(live ? m : 0) * ldx;
  const int items = num_groups * 4;
  for (int base = 0; base < items; base += 256) {  // uniform trip count: the shuffles below need whole warps
    const int it = base + threadIdx.x;
    const bool valid = it < items;
    const int g = it >> 2, c = it & 3, kc = g * kGroup + c * 8;
    float f[8], amax = 0.0f;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      f[jj] = (valid && live && kc + jj < k) ? a16_load<T>(row + kc + jj) : 0.0f;
      amax = fmaxf(amax, fabsf(f[jj]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float scale = __fdiv_rn(amax, 127.0f);
    const float recip = scale != 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
    __align__(16) __half h[8];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const float q = fminf(fmaxf(roundf(__fmul_rn(f[jj], recip)), -127.0f), 127.0f);
      const int pos = (jj < 4) ? 2 * jj : 2 * (jj - 4) + 1;
      h[pos] = __float2half_rn(__fmul_rn(q, scale));
    }
    if (valid)
      *reinterpret_cast<uint4*>(blocks + ((size_t)g * m8_pad + (m >> 3)) * 512 + (m & 7) * 16 + c * 128) =
          *reinterpret_cast<const uint4*>(h);
  }
}

// ------------------------------------------------------------------ linear
__device__ __forceinline__ int a16_dot(const uint4& nw, const uint4& r0, const uint4& r1) {
  int d = 0;
  d = __dp4a((int)(nw.x & 0x0F0F0F0Fu), (int)r0.x, d);
  d = __dp4a((int)(nw.y & 0x0F0F0F0Fu), (int)r0.y, d);
  d = __dp4a((int)(nw.z & 0x0F0F0F0Fu), (int)r0.z, d);
  d = __dp4a((int)(nw.w & 0x0F0F0F0Fu), (int)r0.w, d);
  d = __dp4a((int)((nw.x >> 4) & 0x0F0F0F0Fu), (int)r1.x, d);
  d = __dp4a((int)((nw.y >> 4) & 0x0F0F0F0Fu), (int)r1.y, d);
  d = __dp4a((int)((nw.z >> 4) & 0x0F0F0F0Fu), (int)r1.z, d);
  d = __dp4a((int)((nw.w >> 4) & 0x0F0F0F0Fu), (int)r1.w, d);
  return d;
}

struct A16Cell {
  uint4 nw;
  float s, z;
};
__device__ __forceinline__ A16Cell a16_load_cell(const uint8_t* cell, int lane) {
  A16Cell c;
  c.nw = __ldg(reinterpret_cast<const uint4*>(cell) + lane);
  c.s = __ldg(reinterpret_cast<const float*>(cell + kCellNibbleBytes) + lane);
  c.z = __ldg(reinterpret_cast<const float*>(cell + kCellNibbleBytes + kPanelRows * 4) + lane);
  return c;
}

// grid (panels, ceil(M / MT), ksplit), 256 threads.  partial == nullptr: finish here (bias, clamp, fp16).
template <int MT>
__global__ void __launch_bounds__(256) a16_linear_kernel(const uint8_t* __restrict__ tiled,
                                                         const uint8_t* __restrict__ recs, int m, int k, int n,
                                                         int groups_per_slice, __half* __restrict__ y, int ldy,
                                                         float* __restrict__ partial, int n_pad) {
  __shared__ float red[8][MT][32];
  __shared__ uint4 s_rec[8][MT * 3];  // per warp: the MT records of the group it works on
  const TiledHeaderA16* hdr = reinterpret_cast<const TiledHeaderA16*>(tiled);
  if (hdr->magic != kTiledMagicA16 || hdr->n != (uint32_t)n || hdr->k != (uint32_t)k) {
    if (threadIdx.x == 0) atomicOr(&g_device_status, kDevStatusBadHeader);
    return;
  }
  const int nb = (int)hdr->num_groups;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int panel = blockIdx.x, m0 = blockIdx.y * MT;
  const int g_begin = blockIdx.z * groups_per_slice;
  const int g_end = min(nb, g_begin + groups_per_slice);
  const uint8_t* cells = tiled + hdr->cells_off + (size_t)panel * nb * kCellBytesA16;

  float acc[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i) acc[i] = 0.0f;

  // The records of a group are laid out [group][row]: the MT rows of this tile are MT * 48 contiguous bytes,
  // fetched by the warp with one coalesced load (two for MT = 16) and re-read from shared memory as broadcasts.
  constexpr int kRecVecs = MT * 3;                       // 16-byte pieces per (group, row tile)
  constexpr int kRecLoads = (kRecVecs + 31) / 32;
  const int rows_here = min(MT, m - m0);
  auto load_recs = [&](int gg, uint4 (&r)[kRecLoads]) {
    const uint4* src = reinterpret_cast<const uint4*>(recs + ((size_t)gg * m + m0) * kActRecordBytesA16);
#pragma unroll
    for (int q = 0; q < kRecLoads; ++q) {
      const int idx = q * 32 + lane;
      r[q] = idx < rows_here * 3 ? __ldg(src + idx) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  int g = g_begin + warp;
  A16Cell cur;
  uint4 rcur[kRecLoads];
  if (g < g_end) {
    cur = a16_load_cell(cells + (size_t)g * kCellBytesA16, lane);
    load_recs(g, rcur);
  }
  for (; g < g_end; g += 8) {
    A16Cell nxt = cur;
    uint4 rnxt[kRecLoads];
#pragma unroll
    for (int q = 0; q < kRecLoads; ++q) rnxt[q] = rcur[q];
    if (g + 8 < g_end) {
      nxt = a16_load_cell(cells + (size_t)(g + 8) * kCellBytesA16, lane);
      load_recs(g + 8, rnxt);
    }
    __syncwarp();  // the previous group's reads of s_rec are done
#pragma unroll
    for (int q = 0; q < kRecLoads; ++q)
      if (q * 32 + lane < kRecVecs) s_rec[warp][q * 32 + lane] = rcur[q];
    __syncwarp();
#pragma unroll
    for (int i = 0; i < MT; ++i) {  // rows beyond M hold zero records: they add 0
      const uint4 r0 = s_rec[warp][i * 3], r1 = s_rec[warp][i * 3 + 1], r2 = s_rec[warp][i * 3 + 2];
      const int asum = (int)r2.x;
      const int dot = a16_dot(cur.nw, r0, r1) - 8 * asum;
      const float t = fmaf(cur.s, (float)dot, cur.z * (float)asum);
      acc[i] = fmaf(__uint_as_float(r2.y), t, acc[i]);
    }
    cur = nxt;
#pragma unroll
    for (int q = 0; q < kRecLoads; ++q) rcur[q] = rnxt[q];
  }
#pragma unroll
  for (int i = 0; i < MT; ++i) red[warp][i][lane] = acc[i];
  __syncthreads();
  const int col = panel * kPanelRows;
  for (int idx = threadIdx.x; idx < MT * 32; idx += 256) {
    const int i = idx >> 5, l = idx & 31, row = m0 + i;
    if (row >= m) continue;
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w][i][l];
    if (partial) {
      partial[((size_t)blockIdx.z * m + row) * n_pad + col + l] = s;
    } else if (col + l < n) {
      const float* bias = reinterpret_cast<const float*>(tiled + hdr->bias_off);
      s += bias[col + l];
      s = fminf(fmaxf(s, -65504.0f), 65504.0f);
      y[(size_t)row * ldy + col + l] = __float2half_rn(s);
    }
  }
}

// M <= 4: ONE launch per linear.  The per-block activation quantization has no row-wide dependency (unlike the
// W4A32 path's per-row min/max), so every CTA quantizes the activations of its own K slice into shared memory
// first (a version in which each warp quantized the group it was about to use, with shuffles for the record
// words, spent ~800 cycles per group in dependent shuffles: 0.70 ms for the grouped 28-layer step).  K is split over the CTAs of a thread-block cluster (gridDim.z = cluster size <= 8); their
// partial sums meet in the first CTA's pass over distributed shared memory, in rank order (deterministic).
// Up to four matrices that read the same activations (q/k/v, gate/up) ride in one launch, their panels side
// by side along gridDim.x.
constexpr int kA16MaxProblems = 4;
struct A16Problem {
  const uint8_t* tiled;
  __half* y;
  int n, ldy, panel_begin;
};
struct A16Group {
  A16Problem p[kA16MaxProblems];
  int count;
};

template <int MT, typename T>
__global__ void __launch_bounds__(256) a16_gemv_fused_kernel(const A16Group grp, const T* __restrict__ x, int ldx, int m,
                                                             int k, int groups_per_slice) {
  __shared__ float red[8][MT][32];
  __shared__ float sum[MT][32];
  extern __shared__ uint4 s_rec[];  // [MT][groups_per_slice] records of 3 x 16 bytes
  cg::cluster_group cluster = cg::this_cluster();
  int pi = 0;
#pragma unroll
  for (int i = 1; i < kA16MaxProblems; ++i)
    if (i < grp.count && (int)blockIdx.x >= grp.p[i].panel_begin) pi = i;
  const uint8_t* __restrict__ tiled = grp.p[pi].tiled;
  __half* __restrict__ y = grp.p[pi].y;
  const int n = grp.p[pi].n, ldy = grp.p[pi].ldy;
  const TiledHeaderA16* hdr = reinterpret_cast<const TiledHeaderA16*>(tiled);
  // the CTAs of a cluster share blockIdx.x, hence the matrix: the early exit is taken by all of them or none
  if (hdr->magic != kTiledMagicA16 || hdr->n != (uint32_t)n || hdr->k != (uint32_t)k) {
    if (threadIdx.x == 0) atomicOr(&g_device_status, kDevStatusBadHeader);
    return;
  }
  const int nb = (int)hdr->num_groups;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int panel = (int)blockIdx.x - grp.p[pi].panel_begin;
  const int g_begin = blockIdx.z * groups_per_slice;
  const int g_end = min(nb, g_begin + groups_per_slice);
  const uint8_t* cells = tiled + hdr->cells_off + (size_t)panel * nb * kCellBytesA16;

  float acc[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i) acc[i] = 0.0f;
  int g = g_begin + warp;
  A16Cell cur;
  // Under programmatic dependent launch the weights (never written by a kernel) are fetched while the
  // previous kernel of the stream drains; the activations, which it may have produced, only after it is done.
  pdl_launch_dependents();
  if (g < g_end) cur = a16_load_cell(cells + (size_t)g * kCellBytesA16, lane);
  pdl_wait_prior();

  // Phase 1: the CTA quantizes the activations of its K slice once, into 48-byte records in shared memory
  // (8 lanes per group, 4 consecutive k per lane - the arithmetic of a16_act_quant_kernel).
  const int gcount = g_end - g_begin;
  for (int base = 0; base < gcount; base += 32) {  // uniform trip count: whole warps take part in the shuffles
    const int gi = base + warp * 4 + (lane >> 3), j = lane & 7;
    const int kk0 = (g_begin + gi) * kGroup + j * 4;
    float vv[MT][4];  // all rows' loads are issued before the first dependent shuffle
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int t = 0; t < 4; ++t)
        vv[i][t] = (gi < gcount && i < m && kk0 + t < k) ? a16_load<T>(x + (size_t)i * ldx + kk0 + t) : 0.0f;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      float v[4], amax = 0.0f;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        v[t] = vv[i][t];
        amax = fmaxf(amax, fabsf(v[t]));
      }
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float scale = __fdiv_rn(amax, 127.0f);
      const float recip = scale != 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
      int q[4], asum = 0;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        q[t] = (int)fminf(fmaxf(roundf(__fmul_rn(v[t], recip)), -127.0f), 127.0f);
        asum += q[t];
      }
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) asum += __shfl_xor_sync(0xffffffffu, asum, o);
      const uint32_t ev = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[2] & 0xff) << 8);
      const uint32_t od = (uint32_t)(q[1] & 0xff) | ((uint32_t)(q[3] & 0xff) << 8);
      const uint32_t ev_p = __shfl_xor_sync(0xffffffffu, ev, 1), od_p = __shfl_xor_sync(0xffffffffu, od, 1);
      if (gi < gcount) {
        uint32_t* rec = reinterpret_cast<uint32_t*>(s_rec + ((size_t)i * groups_per_slice + gi) * 3);
        if ((j & 1) == 0) rec[j >> 1] = ev | (ev_p << 16);
        else rec[4 + (j >> 1)] = od_p | (od << 16);
        if (j == 0) {
          rec[8] = (uint32_t)asum;
          rec[9] = __float_as_uint(scale);
        }
      }
    }
  }
  __syncthreads();

  // Phase 2: lane = output row, the warps take the slice's groups in turn; records come back as broadcasts.
  for (; g < g_end; g += 8) {
    A16Cell nxt = cur;
    if (g + 8 < g_end) nxt = a16_load_cell(cells + (size_t)(g + 8) * kCellBytesA16, lane);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const uint4* rec = s_rec + ((size_t)i * groups_per_slice + (g - g_begin)) * 3;
      const uint4 r0 = rec[0], r1 = rec[1], r2 = rec[2];
      const int asum = (int)r2.x;
      const int dot = a16_dot(cur.nw, r0, r1) - 8 * asum;
      const float t = fmaf(cur.s, (float)dot, cur.z * (float)asum);
      acc[i] = fmaf(__uint_as_float(r2.y), t, acc[i]);
    }
    cur = nxt;
  }
#pragma unroll
  for (int i = 0; i < MT; ++i) red[warp][i][lane] = acc[i];
  __syncthreads();
  if (threadIdx.x < MT * 32) {
    const int i = threadIdx.x >> 5;
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w][i][lane];
    sum[i][lane] = s;
  }
  cluster.sync();  // every CTA's sums are written
  if (cluster.block_rank() == 0 && threadIdx.x < MT * 32) {
    const int i = threadIdx.x >> 5, col = panel * kPanelRows + lane;
    float s = sum[i][lane];
    for (unsigned r = 1; r < cluster.num_blocks(); ++r) s += *cluster.map_shared_rank(&sum[i][lane], r);
    if (i < m && col < n) {
      s += reinterpret_cast<const float*>(tiled + hdr->bias_off)[col];
      s = fminf(fmaxf(s, -65504.0f), 65504.0f);
      y[(size_t)i * ldy + col] = __float2half_rn(s);
    }
  }
  cluster.sync();  // the other CTAs' shared memory stays alive until it has been read
}

__global__ void a16_finish_kernel(const float* __restrict__ partial, const uint8_t* __restrict__ tiled, int slices,
                                  int m, int n, int n_pad, __half* __restrict__ y, int ldy) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
  if (col >= n) return;
  const TiledHeaderA16* hdr = reinterpret_cast<const TiledHeaderA16*>(tiled);
  float s = 0.0f;
  for (int z = 0; z < slices; ++z) s += partial[((size_t)z * m + row) * n_pad + col];
  s += reinterpret_cast<const float*>(tiled + hdr->bias_off)[col];
  s = fminf(fmaxf(s, -65504.0f), 65504.0f);
  y[(size_t)row * ldy + col] = __float2half_rn(s);
}

// ------------------------------------------------------------------ host side
static inline int a16_mt(int m) { return m >= 16 ? 16 : m >= 8 ? 8 : m >= 4 ? 4 : m >= 2 ? 2 : 1; }

// K slices: enough CTAs for two per SM when the (panel, row-tile) grid is small; a slice keeps >= 8 groups.
int a16_slices(int m, int k, int n) {
  const int nb = (int)blob_num_blocks(k), panels = (n + kPanelRows - 1) / kPanelRows;
  const int mt = a16_mt(m), ctas = panels * ((m + mt - 1) / mt);
  if (ctas >= 148) return 1;
  int s = (296 + ctas - 1) / ctas;
  s = min(s, max(1, nb / 8));
  return min(s, 8);
}

// gemm_tcf16.cu
int w4a16_gemm_tcf16_tile(int m, int n);
int w4a16_gemm_tcf16_tile_grouped(int m, int count, const int* n);
cudaError_t launch_w4a16_gemm_tcf16_grouped(const uint8_t*, int, int, int, const void* const*, void* const*, const int*,
                                            const int*, cudaStream_t);
cudaError_t launch_w4a16_gemm_tcf16(const uint8_t*, const void*, void*, int, int, int, int, cudaStream_t);

// The tensor-core path (fp16 operands, one rounding each) for large M; otherwise the exact-integer dp4a kernel.
// Measured (us per linear, dp4a vs tensor-core path incl. its quantization): 1536 -> 8960: M = 32 18 / 19, M = 48
// 24 / 20; 8192 -> 28672: M = 16 120 / 136, M = 24 212 / 137; 8960 -> 1536 (12 weight tiles): M = 63 40 / 76;
// 1536 -> 1536: M = 63 10.5 / 18.  With few weight tiles the tensor-core kernel needs several row tiles to pay.
bool w4a16_tensor_path(int m, int n, int kernel) {
  if (kernel == 4) return m >= 8;
  return kernel == 0 && (m >= 128 || (m >= 32 && n >= 8192));
}

size_t a16_workspace_bytes(int m, int k, int n) {
  const size_t rec = align_up((size_t)m * blob_num_blocks(k) * kActRecordBytesA16, 256);
  const int s = a16_slices(m, k, n);
  const size_t n_pad = (size_t)((n + kPanelRows - 1) / kPanelRows) * kPanelRows;
  const size_t simt = rec + (s > 1 ? align_up((size_t)s * m * n_pad * 4, 256) : 0);
  // operand blocks of the tensor-core path: 64 bytes per row and K-group, rows padded to its widest tile
  const size_t blk = m >= 8 ? align_up((size_t)((m + 255) / 256 * 256) * blob_num_blocks(k) * 64, 256) : 0;
  return simt > blk ? simt : blk;
}

template <int MT>
static cudaError_t a16_launch_mt(const uint8_t* tiled, const uint8_t* recs, int m, int k, int n, __half* y, int ldy,
                                 float* partial, int slices, cudaStream_t st) {
  const int nb = (int)blob_num_blocks(k), panels = (n + kPanelRows - 1) / kPanelRows;
  const int gps = (nb + slices - 1) / slices;
  dim3 grid(panels, (m + MT - 1) / MT, slices);
  a16_linear_kernel<MT><<<grid, 256, 0, st>>>(tiled, recs, m, k, n, gps, y, ldy, slices > 1 ? partial : nullptr,
                                              panels * kPanelRows);
  return cudaGetLastError();
}

template <int MT, typename T>
static cudaError_t a16_launch_fused(const A16Group& grp, int panels, const void* x, int ldx, int m, int k, bool pdl,
                                    cudaStream_t st) {
  const int nb = (int)blob_num_blocks(k);
  int slices = (296 + panels - 1) / panels;  // two CTAs per SM where K allows; a slice keeps >= 8 groups
  slices = max(1, min(min(slices, nb / 8), 8));
  const int gps = (nb + slices - 1) / slices;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)panels, 1, (unsigned)slices);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = st;
  const size_t rec_bytes = (size_t)MT * gps * kActRecordBytesA16;
  if (rec_bytes > 160 * 1024) return cudaErrorInvalidConfiguration;  // not reachable under the size rule of this kernel
  static bool configured[64] = {};  // function attributes are per device
  if (rec_bytes > 48 * 1024 - sizeof(float) * (8 * MT * 32 + MT * 32)) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (!(dev >= 0 && dev < 64 && configured[dev])) {
      e = cudaFuncSetAttribute(a16_gemv_fused_kernel<MT, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(160 * 1024));
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
  }
  cfg.dynamicSmemBytes = rec_bytes;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)slices;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, a16_gemv_fused_kernel<MT, T>, grp, static_cast<const T*>(x), ldx, m, k, gps);
}

// The size rule of the single-launch kernel: small enough that launches, not bytes, set the time.  Every CTA
// repeats the quantization of its K slice for all M rows, which costs more than a second launch on large
// matrices and at M > 1 (measured per linear, fused vs records + dp4a: M = 1 wins from 1536 x 256 (3.7 vs 5.4 us)
// to 8192 x 8192 (17.6 vs 24.5) and ties at 28672 x 8192; M = 4 wins only at 1536 x 256 (5.0 vs 5.6) and loses at
// 1536 x 1536 (9.7 vs 6.2)).
static bool a16_fused_ok(int m, long long weights) {
  return m == 1 ? weights <= (128ll << 20) : (m <= 4 && weights * m <= (2ll << 20));
}

static cudaError_t a16_dispatch_fused(const A16Group& grp, int panels, const void* x, int x_dtype, int ldx, int m, int k,
                                      bool pdl, cudaStream_t st) {
  if (x_dtype == 1) {
    if (m == 1) return a16_launch_fused<1, __half>(grp, panels, x, ldx, m, k, pdl, st);
    if (m == 2) return a16_launch_fused<2, __half>(grp, panels, x, ldx, m, k, pdl, st);
    return a16_launch_fused<4, __half>(grp, panels, x, ldx, m, k, pdl, st);
  }
  if (m == 1) return a16_launch_fused<1, float>(grp, panels, x, ldx, m, k, pdl, st);
  if (m == 2) return a16_launch_fused<2, float>(grp, panels, x, ldx, m, k, pdl, st);
  return a16_launch_fused<4, float>(grp, panels, x, ldx, m, k, pdl, st);
}

cudaError_t launch_w4a16_linear(const void* x, int x_dtype, const void* tiled, void* y, void* ws, int m, int k, int n,
                                int ldx, int ldy, int kernel_and_flags, cudaStream_t st);

// Several matrices on the same activations: one launch of the single-launch kernel when the group as a whole
// passes its size rule, else one forward per matrix (the workspace is reused: the stream orders them).
cudaError_t launch_w4a16_linear_grouped(const void* x, int x_dtype, int m, int k, int ldx, int count,
                                        const void* const* tiled, void* const* y, const int* n, const int* ldy, void* ws,
                                        int flags, cudaStream_t st) {
  long long weights = 0;
  for (int i = 0; i < count; ++i) weights += (long long)n[i] * k;
  if (count <= kA16MaxProblems && a16_fused_ok(m, weights)) {
    A16Group grp = {};
    int panels = 0;
    for (int i = 0; i < count; ++i) {
      grp.p[i].tiled = static_cast<const uint8_t*>(tiled[i]);
      grp.p[i].y = static_cast<__half*>(y[i]);
      grp.p[i].n = n[i];
      grp.p[i].ldy = ldy[i];
      grp.p[i].panel_begin = panels;
      panels += (n[i] + kPanelRows - 1) / kPanelRows;
    }
    grp.count = count;
    return a16_dispatch_fused(grp, panels, x, x_dtype, ldx, m, k, (flags & 0x100) != 0, st);
  }
  long long n_sum = 0;
  for (int i = 0; i < count; ++i) n_sum += n[i];
  if (count <= 4 && w4a16_tensor_path(m, (int)(n_sum > 0x7fffffff ? 0x7fffffff : n_sum), 0)) {
    // one quantization into operand blocks and ONE tensor-core launch for the whole group
    const int nb = (int)blob_num_blocks(k);
    const int nt = w4a16_gemm_tcf16_tile_grouped(m, count, n), m_pad = (m + nt - 1) / nt * nt;
    uint8_t* blocks = static_cast<uint8_t*>(ws);
    if (x_dtype == 1)
      a16_act_quant_blocks_f16_kernel<__half><<<m_pad, 256, 0, st>>>(static_cast<const __half*>(x), m, k, ldx, nb, m_pad / 8, blocks);
    else
      a16_act_quant_blocks_f16_kernel<float><<<m_pad, 256, 0, st>>>(static_cast<const float*>(x), m, k, ldx, nb, m_pad / 8, blocks);
    const cudaError_t qe = cudaGetLastError();
    if (qe != cudaSuccess) return qe;
    return launch_w4a16_gemm_tcf16_grouped(blocks, m, k, count, tiled, y, n, ldy, st);
  }
  for (int i = 0; i < count; ++i) {
    const cudaError_t e = launch_w4a16_linear(x, x_dtype, tiled[i], y[i], ws, m, k, n[i], ldx, ldy[i], flags & 0x100, st);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t launch_w4a16_linear(const void* x, int x_dtype, const void* tiled, void* y, void* ws, int m, int k, int n,
                                int ldx, int ldy, int kernel_and_flags, cudaStream_t st) {
  const int kernel = kernel_and_flags & 0xff;
  const bool pdl = (kernel_and_flags & 0x100) != 0;  // only the single-launch kernel takes part
  const int nb = (int)blob_num_blocks(k);
  uint8_t* recs = static_cast<uint8_t*>(ws);
  if (kernel == 0 && a16_fused_ok(m, (long long)n * k)) {  // one launch: quantization inside, K split over a cluster
    A16Group grp = {};
    grp.p[0].tiled = static_cast<const uint8_t*>(tiled);
    grp.p[0].y = static_cast<__half*>(y);
    grp.p[0].n = n;
    grp.p[0].ldy = ldy;
    grp.p[0].panel_begin = 0;
    grp.count = 1;
    return a16_dispatch_fused(grp, (n + kPanelRows - 1) / kPanelRows, x, x_dtype, ldx, m, k, pdl, st);
  }
  if (w4a16_tensor_path(m, n, kernel)) {
    const int nt = w4a16_gemm_tcf16_tile(m, n), m_pad = (m + nt - 1) / nt * nt;
    if (x_dtype == 1)
      a16_act_quant_blocks_f16_kernel<__half><<<m_pad, 256, 0, st>>>(static_cast<const __half*>(x), m, k, ldx, nb, m_pad / 8, recs);
    else
      a16_act_quant_blocks_f16_kernel<float><<<m_pad, 256, 0, st>>>(static_cast<const float*>(x), m, k, ldx, nb, m_pad / 8, recs);
    const cudaError_t qe = cudaGetLastError();
    if (qe != cudaSuccess) return qe;
    return launch_w4a16_gemm_tcf16(recs, tiled, y, m, k, n, ldy, st);
  }
  float* partial =
      reinterpret_cast<float*>(recs + align_up((size_t)m * nb * kActRecordBytesA16, 256));
  dim3 qgrid((nb + 31) / 32, m);
  if (x_dtype == 1) a16_act_quant_kernel<__half><<<qgrid, 256, 0, st>>>(static_cast<const __half*>(x), k, ldx, nb, recs);
  else a16_act_quant_kernel<float><<<qgrid, 256, 0, st>>>(static_cast<const float*>(x), k, ldx, nb, recs);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int slices = a16_slices(m, k, n);
  const uint8_t* t = static_cast<const uint8_t*>(tiled);
  __half* yh = static_cast<__half*>(y);
  switch (a16_mt(m)) {
    case 16: e = a16_launch_mt<16>(t, recs, m, k, n, yh, ldy, partial, slices, st); break;
    case 8: e = a16_launch_mt<8>(t, recs, m, k, n, yh, ldy, partial, slices, st); break;
    case 4: e = a16_launch_mt<4>(t, recs, m, k, n, yh, ldy, partial, slices, st); break;
    case 2: e = a16_launch_mt<2>(t, recs, m, k, n, yh, ldy, partial, slices, st); break;
    default: e = a16_launch_mt<1>(t, recs, m, k, n, yh, ldy, partial, slices, st); break;
  }
  if (e != cudaSuccess || slices == 1) return e;
  const int n_pad = (n + kPanelRows - 1) / kPanelRows * kPanelRows;
  a16_finish_kernel<<<dim3((n + 255) / 256, m), 256, 0, st>>>(partial, t, slices, m, n, n_pad, yh, ldy);
  return cudaGetLastError();
}

cudaError_t launch_w4a16_repack(const void* blob_dev, int n, int k, int has_bias, int row_begin, int row_count,
                                void* tiled_dev, cudaStream_t st) {
  const BlobHeader bh = make_blob_header_a16(n, k, has_bias);
  const TiledHeaderA16 th = make_tiled_header_a16(row_count, k, has_bias);
  cudaError_t e = cudaMemcpyAsync(tiled_dev, &th, sizeof(th), cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) return e;
  const uint8_t* b = static_cast<const uint8_t*>(blob_dev);
  uint8_t* t = static_cast<uint8_t*>(tiled_dev);
  const int cells = (int)(th.num_panels * th.num_groups);
  a16_repack_cells_kernel<<<(cells * 32 + 255) / 256, 256, 0, st>>>(
      b + bh.nibbles_off, reinterpret_cast<const float*>(b + bh.scales_off),
      reinterpret_cast<const float*>(b + a16_zeros_off(bh)), k, row_begin, row_count, (int)th.num_groups,
      (int)th.num_panels, t + th.cells_off,
      reinterpret_cast<unsigned int*>(t + offsetof(TiledHeaderA16, max_weight_bits)));
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int padded = (int)th.num_panels * kPanelRows;
  a16_repack_bias_kernel<<<(padded + 255) / 256, 256, 0, st>>>(
      has_bias ? reinterpret_cast<const float*>(b + bh.bias_off) : nullptr, row_begin, row_count, padded,
      reinterpret_cast<float*>(t + th.bias_off));
  return cudaGetLastError();
}

}  // namespace mllmb200
