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
#include "decoder_attn_body.cuh"

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

// Decode-step attention over context splits: the work of one CTA is attn_partial_body
// (decoder_attn_body.cuh); grid (splits, kv_heads), 256 threads.
template <int D>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_partial_kernel(
    const float* __restrict__ q, const float* __restrict__ k_new, const float* __restrict__ v_new,
    const float* __restrict__ sin_t, const float* __restrict__ cos_t, const int* __restrict__ pos_ptr, int max_ctx,
    int chunk, int group, float* __restrict__ cache_k, float* __restrict__ cache_v, float* __restrict__ part_o,
    float* __restrict__ part_ml, int splits, int use_pdl) {
  __shared__ AttnSmem<D> sm;
  if (use_pdl) {
    pdl_launch_dependents();
    pdl_wait_prior();
  }
  const int pos = min(*pos_ptr, max_ctx - 1);
  const int split = blockIdx.x, kvh = blockIdx.y;
  if (split * chunk > pos) return;
  attn_partial_body<D>(sm, threadIdx.x, [] { __syncthreads(); }, q + (size_t)kvh * group * D, k_new + kvh * D,
                       v_new + kvh * D, sin_t + (size_t)pos * (D / 2), cos_t + (size_t)pos * (D / 2), pos, split * chunk, min((split + 1) * chunk, pos + 1), group,
                       cache_k + (size_t)kvh * max_ctx * D, cache_v + (size_t)kvh * max_ctx * D,
                       part_o + (size_t)kvh * group * splits * D, part_ml + (size_t)kvh * group * splits * 2, splits, split);
}

template __global__ void attn_decode_partial_kernel<64>(const float*, const float*, const float*, const float*, const float*,
                                                        const int*, int, int, int, float*, float*, float*, float*, int, int);
template __global__ void attn_decode_partial_kernel<128>(const float*, const float*, const float*, const float*,
                                                         const float*, const int*, int, int, int, float*, float*, float*,
                                                         float*, int, int);

// logits[v] = sum_k x[k] * W[v,k], W fp16 [V, hidden] row-major, x fp32 (one row), fp32 accumulation.
// One warp per output row, 16-byte loads; hidden a multiple of 8.  Each CTA also leaves the largest
// logit it produced and its index in best[blockIdx] (lowest index on ties), so that greedy sampling
// is a reduction over gridDim.x pairs instead of a pass over the vocabulary.
__global__ void __launch_bounds__(256) lm_head_f16_kernel(const float* __restrict__ x, const __half* __restrict__ w,
                                                          int hidden, int vocab, float* __restrict__ logits,
                                                          float2* __restrict__ best) {
  extern __shared__ float s_x[];
  __shared__ float s_bv[8];
  __shared__ int s_bi[8];
  for (int k = threadIdx.x; k < hidden; k += blockDim.x) s_x[k] = x[k];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  float bv = -3.402823466e+38f;
  int bi = 0x7fffffff;
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
    if (acc > bv) {  // rows come in increasing order within a warp, so a strict test keeps the lowest index
      bv = acc;
      bi = v;
    }
  }
  if (best == nullptr) return;
  if (lane == 0) {
    s_bv[warp] = bv;
    s_bi[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < wpb; ++i)
      if (s_bv[i] > bv || (s_bv[i] == bv && s_bi[i] < bi)) {
        bv = s_bv[i];
        bi = s_bi[i];
      }
    best[blockIdx.x] = make_float2(bv, __int_as_float(bi));
  }
}

// Greedy sampling from the per-CTA candidates of lm_head_f16_kernel, then the bookkeeping of a
// step (greedy = AutoLLM.hpp:70-105 of the reference project: scan in order, strict comparison, so the
// lowest index wins ties): the sampled token becomes the next input and is appended to the history (entry p = the
// token sampled after position p); the position advances.  One warp.
__global__ void sample_advance_kernel(const float2* __restrict__ best, int count, int* __restrict__ pos,
                                      int* __restrict__ token, int* __restrict__ next, int* __restrict__ history,
                                      int max_hist) {
  float bv = -3.402823466e+38f;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < count; i += 32) {
    const float2 c = best[i];
    const int ci = __float_as_int(c.y);
    if (c.x > bv || (c.x == bv && ci < bi)) {
      bv = c.x;
      bi = ci;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if (threadIdx.x == 0) {
    const int p = *pos;
    *next = bi;
    *token = bi;
    if (p < max_hist) history[p] = bi;
    *pos = p + 1;
  }
}

}  // namespace mllmb200
