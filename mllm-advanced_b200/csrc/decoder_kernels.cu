// The decoder-layer operators around the W4A32 linears, for the Qwen2-1.5B / DeepSeek-Distill-Qwen
// forward (reference project: mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:47-54,106-155,175-215).
// Each op follows the reference's Arm operator named beside it.  Ops that feed a quantized linear
// also emit that linear's quantized activations (the records / blocks of act_quant.cu), so that in
// decode the linears launch without a separate quantization kernel in front of them.
#include "device_common.cuh"

namespace mllmb200 {

// ---------------------------------------------------------------------------------------------
// (residual add +) RMSNorm (+ activation quantization), one CTA per row.
//   h_out = h_in (+ delta);  y = h_out * (w * rsqrt(mean(h_out^2) + eps))
// RMSNorm as in mllm/Backends/Arm/Ops/RMSNormOp.cpp:20-77 (fp32, no unit offset).
// y_out (fp32, may be null), records/hdr (may be null): 48-byte records of y as in act_quant.cu.
// The row lives in registers between the passes (hidden <= 8 * blockDim).
// ---------------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormMaxPerThread = 8;  // hidden <= 2048

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < (blockDim.x >> 5) ? scratch[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__device__ __forceinline__ void block_minmax(float& mn, float& mx, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) {
    scratch[warp] = mn;
    scratch[32 + warp] = mx;
  }
  __syncthreads();
  mn = lane < nw ? scratch[lane] : 3.402823466e+38f;
  mx = lane < nw ? scratch[32 + lane] : -3.402823466e+38f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
}

// Writes the 48-byte records of one row whose values are produced by `value(k)`; every thread of the
// CTA must call it (the quad shuffles need full warps).  k_total a multiple of 8 is not required.
template <class F>
__device__ __forceinline__ void emit_records(F value, int k_total, int num_groups, const ActQuantParams& p,
                                             uint8_t* __restrict__ out) {
  const int num_items = num_groups * 4;
  for (int base = 0; base < num_items; base += blockDim.x) {
    const int item = base + threadIdx.x;
    const bool valid = item < num_items;
    const int k0 = item * 8;
    int q8[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q8[j] = (valid && k0 + j < k_total) ? act_quant_value(value(k0 + j), p) : 0;
    const uint32_t lo = ((uint32_t)q8[0] & 0xFFu) | (((uint32_t)q8[2] & 0xFFu) << 8) | (((uint32_t)q8[4] & 0xFFu) << 16) |
                        (((uint32_t)q8[6] & 0xFFu) << 24);
    const uint32_t hi = ((uint32_t)q8[1] & 0xFFu) | (((uint32_t)q8[3] & 0xFFu) << 8) | (((uint32_t)q8[5] & 0xFFu) << 16) |
                        (((uint32_t)q8[7] & 0xFFu) << 24);
    int s = q8[0] + q8[1] + q8[2] + q8[3] + q8[4] + q8[5] + q8[6] + q8[7];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (valid) {
      const int g = item >> 2, i = item & 3;
      uint32_t* rec = reinterpret_cast<uint32_t*>(out + (size_t)g * kActRecordBytes);
      rec[i] = lo;
      rec[4 + i] = hi;
      if (i == 0) *reinterpret_cast<uint4*>(rec + 8) = make_uint4((uint32_t)(-8 * s), 0u, 0u, 0u);
    }
  }
}

__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_quant_kernel(
    const float* __restrict__ h_in, const float* __restrict__ delta, const float* __restrict__ w, float eps, int hidden,
    float* __restrict__ h_out, float* __restrict__ y_out, uint8_t* __restrict__ records, float2* __restrict__ hdr,
    int use_pdl) {
  __shared__ float scratch[64];
  __shared__ float s_y[kNormThreads * kNormMaxPerThread];
  if (use_pdl) {
    pdl_launch_dependents();
    pdl_wait_prior();
  }
  const int m = blockIdx.x, tid = threadIdx.x;
  const float* hi = h_in + (size_t)m * hidden;
  float v[kNormMaxPerThread], wv[kNormMaxPerThread];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < kNormMaxPerThread; ++i) {
    const int k = tid + i * kNormThreads;
    v[i] = 0.0f;
    wv[i] = k < hidden ? w[k] : 0.0f;  // requested with the row, used after the reduction
    if (k < hidden) {
      v[i] = hi[k] + (delta ? delta[(size_t)m * hidden + k] : 0.0f);
      if (h_out) h_out[(size_t)m * hidden + k] = v[i];
      ss += v[i] * v[i];
    }
  }
  const float rms = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
#pragma unroll
  for (int i = 0; i < kNormMaxPerThread; ++i) {
    const int k = tid + i * kNormThreads;
    if (k < hidden) {
      const float y = v[i] * (wv[i] * rms);
      s_y[k] = y;
      if (y_out) y_out[(size_t)m * hidden + k] = y;
      mn = fminf(mn, y);
      mx = fmaxf(mx, y);
    }
  }
  if (records == nullptr) return;
  block_minmax(mn, mx, scratch);  // contains the __syncthreads that publishes s_y
  const ActQuantParams p = act_quant_params(mn, mx);
  if (tid == 0) hdr[m] = make_float2(p.recip_scale, __int_as_float(-p.nzp));
  const int num_groups = (hidden + kGroup - 1) / kGroup;
  emit_records([&](int k) { return s_y[k]; }, hidden, num_groups, p, records + (size_t)m * num_groups * kActRecordBytes);
}

// ---------------------------------------------------------------------------------------------
// SwiGLU activation: a = silu(gate) * up (mllm/Backends/Arm/Kernels/silu.cpp:19-55 with libm expf;
// the Arm kernel uses a fast sigmoid approximation, so only tolerance parity is meaningful there),
// optionally followed by the activation quantization for the down projection.  One CTA per row.
// ---------------------------------------------------------------------------------------------
constexpr int kSiluThreads = 512;
__global__ void __launch_bounds__(kSiluThreads) silu_mul_quant_kernel(const float* __restrict__ gate,
                                                                      const float* __restrict__ up, int inter,
                                                                      float* __restrict__ a_out,
                                                                      uint8_t* __restrict__ records,
                                                                      float2* __restrict__ hdr, int use_pdl) {
  extern __shared__ float s_a[];  // inter floats
  __shared__ float scratch[64];
  if (use_pdl) {
    pdl_launch_dependents();
    pdl_wait_prior();
  }
  const int m = blockIdx.x, tid = threadIdx.x;
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
  // eight gate/up pairs per thread are requested before the first is used: with one CTA per row the
  // kernel is a chain of memory round trips, not a bandwidth problem
  constexpr int kBatch = 8;
  for (int k0 = 0; k0 < inter; k0 += kSiluThreads * kBatch) {
    float g[kBatch], u[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int k = k0 + j * kSiluThreads + tid;
      g[j] = k < inter ? gate[(size_t)m * inter + k] : 0.0f;
      u[j] = k < inter ? up[(size_t)m * inter + k] : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int k = k0 + j * kSiluThreads + tid;
      if (k < inter) {
        const float a = (g[j] / (1.0f + expf(-g[j]))) * u[j];
        s_a[k] = a;
        if (a_out) a_out[(size_t)m * inter + k] = a;
        mn = fminf(mn, a);
        mx = fmaxf(mx, a);
      }
    }
  }
  if (records == nullptr) return;
  block_minmax(mn, mx, scratch);
  const ActQuantParams p = act_quant_params(mn, mx);
  if (tid == 0) hdr[m] = make_float2(p.recip_scale, __int_as_float(-p.nzp));
  const int num_groups = (inter + kGroup - 1) / kGroup;
  emit_records([&](int k) { return s_a[k]; }, inter, num_groups, p, records + (size_t)m * num_groups * kActRecordBytes);
}

// ---------------------------------------------------------------------------------------------
// Merge of the context splits written by attn_decode_partial_kernel, followed by the activation
// quantization for the o projection.  One CTA, 512 threads, q_heads * D <= 2048.
//   w[h][s] = exp(m[h][s] - max_s m) / sum_s(l[h][s] * exp(m[h][s] - max_s m));  out[h][d] = sum_s w[h][s] * o[h][s][d]
// Dynamic shared memory: q_heads * splits floats.
// ---------------------------------------------------------------------------------------------
constexpr int kCombineThreads = 512;
__global__ void __launch_bounds__(kCombineThreads) attn_combine_quant_kernel(
    const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ pos_ptr, int max_ctx,
    int chunk, int splits, int q_heads, int head_dim, float* __restrict__ attn_out, uint8_t* __restrict__ records,
    float2* __restrict__ hdr, int use_pdl) {
  extern __shared__ float s_w[];  // [q_heads][splits]
  __shared__ float scratch[64];
  __shared__ float s_y[kNormThreads * kNormMaxPerThread];
  if (use_pdl) {
    pdl_launch_dependents();
    pdl_wait_prior();
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos = min(*pos_ptr, max_ctx - 1);
  const int nact = min(splits, pos / chunk + 1);
  for (int h = warp; h < q_heads; h += kCombineThreads / 32) {
    const float* ml = part_ml + (size_t)h * splits * 2;
    float mx = -3.402823466e+38f;
    for (int sidx = lane; sidx < nact; sidx += 32) mx = fmaxf(mx, ml[sidx * 2]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float tot = 0.0f;
    for (int sidx = lane; sidx < nact; sidx += 32) {
      const float e = expf(ml[sidx * 2] - mx);
      s_w[h * splits + sidx] = e;
      tot += ml[sidx * 2 + 1] * e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const float inv = 1.0f / tot;
    for (int sidx = lane; sidx < nact; sidx += 32) s_w[h * splits + sidx] *= inv;  // same lane wrote it
  }
  __syncthreads();
  const int width = q_heads * head_dim;
  float mn = 3.402823466e+38f, mxv = -3.402823466e+38f;
  for (int idx = tid; idx < width; idx += kCombineThreads) {
    const int h = idx / head_dim, d = idx - h * head_dim;
    const float* po = part_o + (size_t)h * splits * head_dim + d;
    float acc = 0.0f;
    for (int s0 = 0; s0 < nact; s0 += 8) {  // eight partial rows requested together (no branch between the loads); summed in split order
      float pv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) pv[j] = po[(size_t)min(s0 + j, nact - 1) * head_dim];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(s0 + j < nact ? s_w[h * splits + s0 + j] : 0.0f, pv[j], acc);
    }
    s_y[idx] = acc;
    if (attn_out) attn_out[idx] = acc;
    mn = fminf(mn, acc);
    mxv = fmaxf(mxv, acc);
  }
  if (records == nullptr) return;
  block_minmax(mn, mxv, scratch);
  const ActQuantParams p = act_quant_params(mn, mxv);
  if (tid == 0) hdr[0] = make_float2(p.recip_scale, __int_as_float(-p.nzp));
  const int num_groups = (width + kGroup - 1) / kGroup;
  emit_records([&](int k) { return s_y[k]; }, width, num_groups, p, records);
}

// Embedding lookup: row gather (mllm/Backends/Arm/Ops/LLMEmbeddingTokenOp.cpp:23-52).
__global__ void embedding_kernel(const int* __restrict__ ids, const float* __restrict__ table, int hidden,
                                 float* __restrict__ out) {
  const int m = blockIdx.x;
  const float* src = table + (size_t)ids[m] * hidden;
  for (int k = threadIdx.x; k < hidden; k += blockDim.x) out[(size_t)m * hidden + k] = src[k];
}

}  // namespace mllmb200
