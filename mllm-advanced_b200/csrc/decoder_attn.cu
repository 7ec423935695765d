// Attention-side operators of the decoder (reference project paths):
//   RoPE, HF half-split form with precomputed tables   mllm/Backends/Arm/Kernels/rope.cpp:20-87
//   KV cache append                                    mllm/Backends/Arm/Ops/KVCacheOp.cpp:15-72
//   scores * 1/sqrt(D), causal mask, softmax, P.V      mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:127-150
//   lm_head product and greedy argmax                  modeling_ds_qwen2.hpp:209-212, mllm/Models/AutoLLM.hpp:70-105
// The reference expands grouped-query K/V heads when it writes the cache (each row stored `rep`
// times); here the cache holds each KV head once and the query heads of a group read the same rows,
// which is the same arithmetic.  fp32 KV cache, fp32 softmax with expf.
#include <cuda_fp16.h>

#include "device_common.cuh"

namespace mllmb200 {

// sin/cos[pos, d] for d < D/2: theta = pos / base^(2d/D)   (rope.cpp:20-36; the upper half duplicates)
__global__ void rope_tables_kernel(float* __restrict__ sin_t, float* __restrict__ cos_t, int max_pos, int half_dim,
                                   float base) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= max_pos * half_dim) return;
  const int pos = idx / half_dim, d = idx % half_dim;
  float theta = 1.0f / powf(base, 2.0f * (float)d / (float)(2 * half_dim));
  theta *= (float)pos;
  sin_t[idx] = sinf(theta);
  cos_t[idx] = cosf(theta);
}

// grid (kv_heads, S), block D: rotate the new keys and append keys/values at positions pos0 + s.
// k_new/v_new: rows of ld floats holding [kv_heads * D]; cache: [kv_heads][max_ctx][D].
__global__ void rope_kv_append_kernel(const float* __restrict__ k_new, const float* __restrict__ v_new, int ld,
                                      const float* __restrict__ sin_t, const float* __restrict__ cos_t,
                                      const int* __restrict__ pos0_ptr, int max_ctx, float* __restrict__ cache_k,
                                      float* __restrict__ cache_v) {
  const int h = blockIdx.x, s = blockIdx.y, d = threadIdx.x, D = blockDim.x, half = D >> 1;
  const int pos = *pos0_ptr + s;  // the position lives in device memory so that one CUDA graph serves every step
  if (pos >= max_ctx) return;
  const float* kr = k_new + (size_t)s * ld + h * D;
  const float* vr = v_new + (size_t)s * ld + h * D;
  const int dd = d < half ? d : d - half;
  const float sn = sin_t[pos * half + dd], cs = cos_t[pos * half + dd];
  const float x0 = kr[dd], x1 = kr[dd + half];
  const float y = d < half ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs);
  cache_k[((size_t)h * max_ctx + pos) * D + d] = y;
  cache_v[((size_t)h * max_ctx + pos) * D + d] = vr[d];
}

// grid (q_heads, S), block D (= 128).  Query row s attends to cache positions [0, pos0 + s].
// q: rows of ldq floats [q_heads * D]; out: rows of ldo floats [q_heads * D].
// Shared memory: (ctx_max + D + 64) floats.
__global__ void attention_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ sin_t,
                                 const float* __restrict__ cos_t, const int* __restrict__ pos0_ptr, int max_ctx, int group,
                                 const float* __restrict__ cache_k, const float* __restrict__ cache_v,
                                 float* __restrict__ out, int ldo, int use_pdl) {
  extern __shared__ float sm[];
  if (use_pdl) {
    pdl_launch_dependents();
    pdl_wait_prior();
  }
  const int h = blockIdx.x, s = blockIdx.y, d = threadIdx.x, D = blockDim.x, half = D >> 1;
  const int pos = min(*pos0_ptr + s, max_ctx - 1), ctx = pos + 1;
  float* s_q = sm;            // D
  float* s_red = sm + D;      // 64
  float* s_p = sm + D + 64;   // ctx scores
  const int kvh = h / group;
  // rotated query
  {
    const float* qr = q + (size_t)s * ldq + h * D;
    const int dd = d < half ? d : d - half;
    const float sn = sin_t[pos * half + dd], cs = cos_t[pos * half + dd];
    const float x0 = qr[dd], x1 = qr[dd + half];
    s_q[d] = d < half ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs);
  }
  __syncthreads();
  const int warp = d >> 5, lane = d & 31, nwarps = D >> 5;
  const float scale = 1.0f / sqrtf((float)D);
  const float* kbase = cache_k + (size_t)kvh * max_ctx * D;
  const float* vbase = cache_v + (size_t)kvh * max_ctx * D;
  float mx = -3.402823466e+38f;
  for (int t = warp; t < ctx; t += nwarps) {
    const float* kr = kbase + (size_t)t * D;
    float acc = 0.0f;
    for (int i = lane; i < D; i += 32) acc += s_q[i] * kr[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    acc *= scale;
    if (lane == 0) s_p[t] = acc;
    mx = fmaxf(mx, acc);
  }
  // block max
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  mx = s_red[0];
  for (int w = 1; w < nwarps; ++w) mx = fmaxf(mx, s_red[w]);
  __syncthreads();
  float sum = 0.0f;
  for (int t = d; t < ctx; t += D) {
    const float e = expf(s_p[t] - mx);
    s_p[t] = e;
    sum += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) s_red[32 + warp] = sum;
  __syncthreads();
  float total = 0.0f;
  for (int w = 0; w < nwarps; ++w) total += s_red[32 + w];
  const float inv = 1.0f / total;
  float o_acc = 0.0f;
  for (int t = 0; t < ctx; ++t) o_acc += (s_p[t] * inv) * vbase[(size_t)t * D + d];
  out[(size_t)s * ldo + h * D + d] = o_acc;
}

// ---------------------------------------------------------------------------------------------
// Decode-step attention (one new token), split over the context so that the whole GPU works on it:
// grid (splits, kv_heads), 256 threads.  CTA (split, kvh) covers cache positions
// [split*chunk, min((split+1)*chunk, pos+1)) for all `group` query heads that share KV head kvh and
// writes, per query head, an unnormalized partial output with its running maximum and sum
// (the usual online-softmax split); attn_combine_quant_kernel merges the splits.  The CTA whose
// range contains the new position rotates the new key, appends key and value to the cache and
// uses them directly, so no separate append launch is needed.
// part_o: [q_heads][splits][D], part_ml: [q_heads][splits][2] = {max, sum}.
// ---------------------------------------------------------------------------------------------
constexpr int kAttnThreads = 256;
constexpr int kAttnMaxGroup = 8;
constexpr int kAttnSub = 32;  // positions per inner block

template <int D>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_partial_kernel(
    const float* __restrict__ q, const float* __restrict__ k_new, const float* __restrict__ v_new,
    const float* __restrict__ sin_t, const float* __restrict__ cos_t, const int* __restrict__ pos_ptr, int max_ctx,
    int chunk, int group, float* __restrict__ cache_k, float* __restrict__ cache_v, float* __restrict__ part_o,
    float* __restrict__ part_ml, int splits, int use_pdl) {
  constexpr int VEC = D / 32, NG = kAttnThreads / D, HALF = D / 2, MAXH = (kAttnMaxGroup + NG - 1) / NG;
  __shared__ float s_q[kAttnMaxGroup * D];
  __shared__ float s_s[kAttnMaxGroup][kAttnSub];
  __shared__ float s_alpha[kAttnMaxGroup], s_mrun[kAttnMaxGroup], s_lrun[kAttnMaxGroup];
  if (use_pdl) {
    pdl_launch_dependents();
    pdl_wait_prior();
  }
  const int pos = min(*pos_ptr, max_ctx - 1), ctx = pos + 1;
  const int split = blockIdx.x, kvh = blockIdx.y;
  const int c0 = split * chunk;
  if (c0 >= ctx) return;
  const int c1 = min(c0 + chunk, ctx);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float scale = 1.0f / sqrtf((float)D);
  // rotated queries of the group
  for (int idx = tid; idx < group * D; idx += kAttnThreads) {
    const int h = idx / D, d = idx - h * D;
    const float* qr = q + (size_t)(kvh * group + h) * D;
    const int dd = d < HALF ? d : d - HALF;
    const float sn = sin_t[pos * HALF + dd], cs = cos_t[pos * HALF + dd];
    const float x0 = qr[dd], x1 = qr[dd + HALF];
    s_q[idx] = d < HALF ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs);
  }
  if (tid < kAttnMaxGroup) {
    s_mrun[tid] = -3.402823466e+38f;
    s_lrun[tid] = 0.0f;
  }
  float* kc = cache_k + (size_t)kvh * max_ctx * D;
  float* vc = cache_v + (size_t)kvh * max_ctx * D;
  const float* kn = k_new + kvh * D;
  const float* vn = v_new + kvh * D;
  const int pd = tid % D, pg = tid / D;  // the output element / head slot this thread accumulates
  float o_acc[MAXH];
#pragma unroll
  for (int i = 0; i < MAXH; ++i) o_acc[i] = 0.0f;
  __syncthreads();

  for (int b0 = c0; b0 < c1; b0 += kAttnSub) {
    // ---- scores: warp w takes positions b0 + w + 8 j
    constexpr int PER_WARP = kAttnSub / (kAttnThreads / 32);
    float kv[PER_WARP][VEC];
#pragma unroll
    for (int j = 0; j < PER_WARP; ++j) {
      const int t = b0 + warp + j * (kAttnThreads / 32);
#pragma unroll
      for (int e = 0; e < VEC; ++e) kv[j][e] = 0.0f;
      if (t < c1) {
        if (t == pos) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const int d = lane * VEC + e, dd = d < HALF ? d : d - HALF;
            const float sn = sin_t[pos * HALF + dd], cs = cos_t[pos * HALF + dd];
            const float x0 = kn[dd], x1 = kn[dd + HALF];
            kv[j][e] = d < HALF ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs);
            kc[(size_t)pos * D + d] = kv[j][e];
          }
        } else if constexpr (VEC == 4) {
          const float4 v4 = *reinterpret_cast<const float4*>(kc + (size_t)t * D + lane * 4);
          kv[j][0] = v4.x, kv[j][1] = v4.y, kv[j][2] = v4.z, kv[j][3] = v4.w;
        } else {
          const float2 v2 = *reinterpret_cast<const float2*>(kc + (size_t)t * D + lane * 2);
          kv[j][0] = v2.x, kv[j][1] = v2.y;
        }
      }
    }
    for (int h = 0; h < group; ++h) {
      float qv[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) qv[e] = s_q[h * D + lane * VEC + e];
#pragma unroll
      for (int j = 0; j < PER_WARP; ++j) {
        float acc = 0.0f;
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc = fmaf(qv[e], kv[j][e], acc);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        const int tl = warp + j * (kAttnThreads / 32);
        if (lane == 0) s_s[h][tl] = (b0 + tl < c1) ? acc * scale : -3.402823466e+38f;
      }
    }
    __syncthreads();
    // ---- online softmax bookkeeping: warp h owns head h
    if (warp < group) {
      const float sc = s_s[warp][lane];
      float mx = sc;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = s_mrun[warp], m_new = fmaxf(m_old, mx);
      const float p = (b0 + lane < c1) ? expf(sc - m_new) : 0.0f;
      float sum = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      s_s[warp][lane] = p;
      if (lane == 0) {
        const float alpha = expf(m_old - m_new);  // 0 on the first block (m_old = -FLT_MAX)
        s_alpha[warp] = alpha;
        s_mrun[warp] = m_new;
        s_lrun[warp] = s_lrun[warp] * alpha + sum;
      }
    }
    __syncthreads();
    // ---- P.V: thread (pd, pg) accumulates element pd of heads pg, pg + NG, ...
    {
      const int nt = min(kAttnSub, c1 - b0);
      float vv[kAttnSub];
#pragma unroll
      for (int t = 0; t < kAttnSub; ++t) {
        vv[t] = 0.0f;
        if (t < nt) {
          if (b0 + t == pos) {
            vv[t] = vn[pd];
            if (pg == 0) vc[(size_t)pos * D + pd] = vv[t];
          } else {
            vv[t] = vc[(size_t)(b0 + t) * D + pd];
          }
        }
      }
#pragma unroll
      for (int i = 0; i < MAXH; ++i) {
        const int h = pg + i * NG;
        if (h < group) {
          float acc = o_acc[i] * s_alpha[h];
#pragma unroll
          for (int t = 0; t < kAttnSub; ++t) acc = fmaf(s_s[h][t], vv[t], acc);
          o_acc[i] = acc;
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < MAXH; ++i) {
    const int h = pg + i * NG;
    if (h < group) part_o[((size_t)(kvh * group + h) * splits + split) * D + pd] = o_acc[i];
  }
  if (tid < group) {
    float* ml = part_ml + ((size_t)(kvh * group + tid) * splits + split) * 2;
    ml[0] = s_mrun[tid];
    ml[1] = s_lrun[tid];
  }
}

template __global__ void attn_decode_partial_kernel<64>(const float*, const float*, const float*, const float*, const float*,
                                                        const int*, int, int, int, float*, float*, float*, float*, int, int);
template __global__ void attn_decode_partial_kernel<128>(const float*, const float*, const float*, const float*,
                                                         const float*, const int*, int, int, int, float*, float*, float*,
                                                         float*, int, int);

// logits[v] = sum_k x[k] * W[v,k], W fp16 [V, hidden] row-major, x fp32 (one row), fp32 accumulation.
// One warp per output row, 16-byte loads; hidden a multiple of 8.
__global__ void __launch_bounds__(256) lm_head_f16_kernel(const float* __restrict__ x, const __half* __restrict__ w,
                                                          int hidden, int vocab, float* __restrict__ logits) {
  extern __shared__ float s_x[];
  for (int k = threadIdx.x; k < hidden; k += blockDim.x) s_x[k] = x[k];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int v = blockIdx.x * wpb + warp; v < vocab; v += gridDim.x * wpb) {
    const uint4* row = reinterpret_cast<const uint4*>(w + (size_t)v * hidden);
    float acc = 0.0f;
    for (int c = lane; c < (hidden >> 3); c += 32) {
      const uint4 pk = row[c];
      const __half2* h2 = reinterpret_cast<const __half2*>(&pk);
      const float* xs = s_x + c * 8;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h2[j]);
        acc = fmaf(f.x, xs[2 * j], acc);
        acc = fmaf(f.y, xs[2 * j + 1], acc);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) logits[v] = acc;
  }
}

// Greedy sampling: index of the largest logit, lowest index on ties (AutoLLM.hpp:70-105 scans in
// order with a strict comparison).  One CTA.
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int n, int* __restrict__ out) {
  __shared__ float s_v[32];
  __shared__ int s_i[32];
  float best = -3.402823466e+38f;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = logits[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_v[warp] = best;
    s_i[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? s_v[lane] : -3.402823466e+38f;
    bi = lane < (blockDim.x >> 5) ? s_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) *out = bi;
  }
}

}  // namespace mllmb200
