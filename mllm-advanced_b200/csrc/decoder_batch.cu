// Batched greedy decode on top of the batch-1 decoder: B sequences, each with its own KV cache and position,
// advance one token per step together, so that every quantized linear of the step runs at M = B.
//
// The reference project has no such mode - its KV cache asserts a batch of one
// (mllm/Backends/Arm/Ops/KVCacheOp.cpp:107,156) - so the semantics are those of B independent runs of its
// batch-1 forward (mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:106-155, cache append KVCacheOp.cpp:15-72, greedy
// loop mllm/Models/AutoLLM.hpp:39-105): sequence b of the batch must produce the tokens a batch-1 decoder
// produces on sequence b alone.  The tests check exactly that.
//
// A batch object borrows weights, norms, tables and the stream of a batch-1 decoder (mllmb200_qwen2_create ...)
// and adds per-sequence state: KV caches [layer][sequence][kv head][max_ctx][D] in fp32, positions, current
// tokens, histories.  Sequences are prefilled one at a time through the batch-1 prefill (from token ids, or from
// ready embedding rows for inputs that mix text with vision-patch embeddings) into their own caches; prompts may
// differ in length.  A decode step is then:
//   embedding rows -> per layer { add + RMSNorm (one CTA per row) -> q,k,v = W4A32 linears at M = B (one grouped
//   call) -> attention over (context split, kv head, sequence) CTAs, which also rotate and append the new K/V ->
//   merge of the splits (one CTA per sequence) -> o linear -> add + RMSNorm -> gate,up linears -> silu * up -> down }
//   -> final norm -> lm_head for all rows -> per-sequence argmax and bookkeeping,
// captured once as a CUDA graph and replayed (positions and tokens live in device memory).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <vector>

#include "../../include/mllmb200.h"
#include "decoder_attn_body.cuh"
#include "decoder_state.h"
#include "device_common.cuh"

#ifndef MLLMB200_BATCH_ATTN_CTAS_PER_SM
#define MLLMB200_BATCH_ATTN_CTAS_PER_SM 4
#endif
#ifndef MLLMB200_BATCH_ATTN_V2  // 0: the batch-1 attention body for every sequence (the earlier form)
#define MLLMB200_BATCH_ATTN_V2 1
#endif

namespace mllmb200 {

__global__ void add_rmsnorm_quant_kernel(const float*, const float*, const float*, float, int, float*, float*, uint8_t*,
                                         float2*, int);
__global__ void silu_mul_quant_kernel(const float*, const float*, int, float*, uint8_t*, float2*, int);
__global__ void embedding_kernel(const int*, const float*, int, float*);

// Decode-step attention for a batch: grid (splits, kv_heads, sequences), 256 threads; the work of a CTA is
// attn_partial_body on the sequence's own cache and position.
// q: [B][ldq], k_new / v_new: [B][ldkv]; caches [B][kv_heads][max_ctx][D]; part_o [B][q_heads][splits][D],
// part_ml [B][q_heads][splits][2].
template <int D>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_partial_batched_kernel(
    const float* __restrict__ q, int ldq, const float* __restrict__ k_new, const float* __restrict__ v_new, int ldkv,
    const float* __restrict__ sin_t, const float* __restrict__ cos_t, const int* __restrict__ pos_ptr, int max_ctx, int chunk,
    int group, int q_heads, float* __restrict__ cache_k, float* __restrict__ cache_v, size_t cache_seq_stride,
    float* __restrict__ part_o, float* __restrict__ part_ml, int splits) {
  __shared__ AttnSmem<D> sm;
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int pos = min(pos_ptr[seq], max_ctx - 1);
  if (split * chunk > pos) return;
  const size_t head0 = (size_t)seq * q_heads + (size_t)kvh * group;
  attn_partial_body<D>(sm, threadIdx.x, [] { __syncthreads(); }, q + (size_t)seq * ldq + (size_t)kvh * group * D,
                       k_new + (size_t)seq * ldkv + kvh * D, v_new + (size_t)seq * ldkv + kvh * D,
                       sin_t + (size_t)pos * (D / 2), cos_t + (size_t)pos * (D / 2), pos, split * chunk,
                       min((split + 1) * chunk, pos + 1), group,
                       cache_k + (size_t)seq * cache_seq_stride + (size_t)kvh * max_ctx * D,
                       cache_v + (size_t)seq * cache_seq_stride + (size_t)kvh * max_ctx * D, part_o + head0 * splits * D,
                       part_ml + head0 * splits * 2, splits, split);
}

// The same partial attention laid out for THROUGHPUT (head_dim 128): with 64 sequences x 2 KV heads x splits CTAs
// in flight the GPU does not wait for any one of them, and what bounds the batch-1 body above - one shuffle
// reduction per (position, head) over a full warp and one shared-memory load per multiply-add of P.V - is all
// that is left.  Here, per block of 32 cache positions:
//   scores  warp w takes positions 4w..4w+3, 8 lanes per position, 16 elements of the head dimension per lane:
//           4 16-byte loads of K per lane (128 contiguous bytes per position and instruction), the rotated queries
//           as broadcast 16-byte shared-memory loads, a 3-step shuffle reduction per (position, head);
//   softmax warp h owns head h (running maximum and sum, as in the body above);
//   P.V     warp w takes the same four positions, lane = 4 consecutive elements of the head dimension: 4 16-byte
//           loads of V per lane, the probabilities as two broadcast 16-byte loads per position, 4 x group
//           accumulators per thread; the eight warps' accumulators are added in warp order at the end.
// The next block's K and V are requested before the current block's arithmetic.  The new token's key (rotated)
// and value are appended to the cache by the CTA whose range holds `pos`, before its loop.
constexpr int kBa2Threads = 256, kBa2Block = 32, kBa2D = 128, kBa2G = kAttnMaxGroup;
struct Ba2Smem {
  float q[kBa2G * kBa2D];        // rotated queries
  float sc[kBa2Block][kBa2G];    // scores of the block, position-major
  float pr[kBa2Block][kBa2G];    // probabilities exp(score - running max)
  float alpha[kBa2G], mrun[kBa2G], lrun[kBa2G];
  float red[kBa2Threads / 32][kBa2G * kBa2D / 2];  // final sum over the warps, half of the heads at a time
};
__global__ void __launch_bounds__(kBa2Threads) attn_decode_partial_batched_v2_kernel(
    const float* __restrict__ q, int ldq, const float* __restrict__ k_new, const float* __restrict__ v_new, int ldkv,
    const float* __restrict__ sin_t, const float* __restrict__ cos_t, const int* __restrict__ pos_ptr, int max_ctx, int chunk,
    int group, int q_heads, float* __restrict__ cache_k, float* __restrict__ cache_v, size_t cache_seq_stride,
    float* __restrict__ part_o, float* __restrict__ part_ml, int splits) {
  constexpr int D = kBa2D, HALF = D / 2;
  __shared__ __align__(16) Ba2Smem sm;
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int pos = min(pos_ptr[seq], max_ctx - 1);
  if (split * chunk > pos) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c0 = split * chunk, c1 = min((split + 1) * chunk, pos + 1);
  const size_t head0 = (size_t)seq * q_heads + (size_t)kvh * group;
  const float* qh = q + (size_t)seq * ldq + (size_t)kvh * group * D;
  const float* kn = k_new + (size_t)seq * ldkv + kvh * D;
  const float* vn = v_new + (size_t)seq * ldkv + kvh * D;
  const float* sin_row = sin_t + (size_t)pos * HALF;
  const float* cos_row = cos_t + (size_t)pos * HALF;
  float* kc = cache_k + (size_t)seq * cache_seq_stride + (size_t)kvh * max_ctx * D;
  float* vc = cache_v + (size_t)seq * cache_seq_stride + (size_t)kvh * max_ctx * D;
  part_o += head0 * splits * D;
  part_ml += head0 * splits * 2;
  const float scale = 1.0f / sqrtf((float)D);

  // rotated queries; the new token's key and value into the cache (RoPE as mllm/Backends/Arm/Kernels/rope.cpp:20-87
  // of the reference project: element d pairs with d +- D/2)
  for (int idx = tid; idx < group * D; idx += kBa2Threads) {
    const int h = idx / D, d = idx - h * D, dd = d < HALF ? d : d - HALF;
    const float sn = sin_row[dd], cs = cos_row[dd];
    const float x0 = qh[(size_t)h * D + dd], x1 = qh[(size_t)h * D + dd + HALF];
    sm.q[idx] = d < HALF ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs);
  }
  if (pos >= c0 && pos < c1 && tid < D) {
    const int d = tid, dd = d < HALF ? d : d - HALF;
    const float sn = sin_row[dd], cs = cos_row[dd];
    const float x0 = kn[dd], x1 = kn[dd + HALF];
    kc[(size_t)pos * D + d] = d < HALF ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs);
    vc[(size_t)pos * D + d] = vn[d];
  }
  if (tid < kBa2G) {
    sm.mrun[tid] = -3.402823466e+38f;
    sm.lrun[tid] = 0.0f;
  }
  __threadfence();
  __syncthreads();  // (the appended row is read back below through L2, by this CTA only)

  const int tp = warp * 4 + (lane >> 3), l8 = lane & 7;  // scores: position of the block, slice of the head dimension
  float4 kreg[4], vreg[4];
  auto load_k = [&](int b0) {
    const int t = b0 + tp;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      kreg[i] = t < c1 ? __ldcg(reinterpret_cast<const float4*>(kc + (size_t)t * D + 32 * i + 4 * l8)) : make_float4(0.f, 0.f, 0.f, 0.f);
  };
  auto load_v = [&](int b0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = b0 + warp * 4 + j;
      vreg[j] = t < c1 ? __ldcg(reinterpret_cast<const float4*>(vc + (size_t)t * D + 4 * lane)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  float4 acc[kBa2G];
#pragma unroll
  for (int h = 0; h < kBa2G; ++h) acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
  load_k(c0);
  load_v(c0);

  for (int b0 = c0; b0 < c1; b0 += kBa2Block) {
    // ---- scores
    {
      float part[kBa2G];
#pragma unroll
      for (int h = 0; h < kBa2G; ++h) {
        part[h] = 0.0f;
        if (h < group) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 qv = *reinterpret_cast<const float4*>(&sm.q[h * D + 32 * i + 4 * l8]);
            part[h] = fmaf(qv.x, kreg[i].x, part[h]);
            part[h] = fmaf(qv.y, kreg[i].y, part[h]);
            part[h] = fmaf(qv.z, kreg[i].z, part[h]);
            part[h] = fmaf(qv.w, kreg[i].w, part[h]);
          }
        }
      }
      if (b0 + kBa2Block < c1) load_k(b0 + kBa2Block);  // the next block's keys, on their way during the rest
#pragma unroll
      for (int h = 0; h < kBa2G; ++h) {
        if (h < group) {
          float v = part[h];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          if (l8 == 0) sm.sc[tp][h] = (b0 + tp < c1) ? v * scale : -3.402823466e+38f;
        }
      }
    }
    __syncthreads();
    // ---- online softmax bookkeeping: warp h owns head h, lane = position of the block
    if (warp < group) {
      const float sc = sm.sc[lane][warp];
      float mx = sc;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = sm.mrun[warp], m_new = fmaxf(m_old, mx);
      const float p = (b0 + lane < c1) ? expf(sc - m_new) : 0.0f;
      float sum = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      sm.pr[lane][warp] = p;
      if (lane == 0) {
        const float al = expf(m_old - m_new);  // 0 on the first block (m_old = -FLT_MAX)
        sm.alpha[warp] = al;
        sm.mrun[warp] = m_new;
        sm.lrun[warp] = sm.lrun[warp] * al + sum;
      }
    }
    __syncthreads();
    // ---- P.V: this warp's four positions, lane = elements 4 lane .. 4 lane + 3
    {
      const float4 a0 = *reinterpret_cast<const float4*>(&sm.alpha[0]);
      const float4 a1 = *reinterpret_cast<const float4*>(&sm.alpha[4]);
      const float al[kBa2G] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
      for (int h = 0; h < kBa2G; ++h) {
        if (h < group) {
          acc[h].x *= al[h], acc[h].y *= al[h], acc[h].z *= al[h], acc[h].w *= al[h];
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 p0 = *reinterpret_cast<const float4*>(&sm.pr[warp * 4 + j][0]);
        const float4 p1 = *reinterpret_cast<const float4*>(&sm.pr[warp * 4 + j][4]);
        const float pj[kBa2G] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int h = 0; h < kBa2G; ++h) {
          if (h < group) {
            acc[h].x = fmaf(pj[h], vreg[j].x, acc[h].x);
            acc[h].y = fmaf(pj[h], vreg[j].y, acc[h].y);
            acc[h].z = fmaf(pj[h], vreg[j].z, acc[h].z);
            acc[h].w = fmaf(pj[h], vreg[j].w, acc[h].w);
          }
        }
      }
      if (b0 + kBa2Block < c1) load_v(b0 + kBa2Block);
    }
    // (the next block's scores go to sm.sc, which nobody reads any more; sm.pr and sm.alpha are rewritten only
    // after the next __syncthreads, which every warp reaches after its P.V)
  }
  // ---- the eight warps' accumulators, added in warp order; half of the heads at a time through shared memory
  for (int half = 0; half < 2; ++half) {
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < kBa2G / 2; ++hh) {
      const int h = half * (kBa2G / 2) + hh;
      if (h < group) *reinterpret_cast<float4*>(&sm.red[warp][hh * D + 4 * lane]) = acc[h];
    }
    __syncthreads();
    for (int idx = tid; idx < (kBa2G / 2) * D; idx += kBa2Threads) {
      const int h = half * (kBa2G / 2) + idx / D, d = idx % D;
      if (h < group) {
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < kBa2Threads / 32; ++w) sum += sm.red[w][idx];
        part_o[((size_t)h * splits + split) * D + d] = sum;
      }
    }
  }
  if (tid < group) {
    float* ml = part_ml + ((size_t)tid * splits + split) * 2;
    ml[0] = sm.mrun[tid];
    ml[1] = sm.lrun[tid];
  }
}

// Merge of the context splits of one sequence per CTA (the arithmetic of attn_combine_quant_kernel, fp32 output):
//   w[h][s] = exp(m[h][s] - max_s m) / sum_s(l[h][s] * exp(m[h][s] - max_s m));  out[h][d] = sum_s w[h][s] * o[h][s][d]
// Dynamic shared memory: q_heads * splits floats.
constexpr int kBatchCombineThreads = 512;
__global__ void __launch_bounds__(kBatchCombineThreads) attn_combine_batched_kernel(
    const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ pos_ptr, int max_ctx,
    int chunk, int splits, int q_heads, int head_dim, float* __restrict__ attn_out) {
  extern __shared__ float s_w[];  // [q_heads][splits]
  const int seq = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos = min(pos_ptr[seq], max_ctx - 1);
  const int nact = min(splits, pos / chunk + 1);
  part_o += (size_t)seq * q_heads * splits * head_dim;
  part_ml += (size_t)seq * q_heads * splits * 2;
  for (int h = warp; h < q_heads; h += kBatchCombineThreads / 32) {
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
  for (int idx = tid; idx < width; idx += kBatchCombineThreads) {
    const int h = idx / head_dim, d = idx - h * head_dim;
    const float* po = part_o + (size_t)h * splits * head_dim + d;
    float acc = 0.0f;
    for (int s0 = 0; s0 < nact; s0 += 8) {  // eight partial rows requested together; summed in split order
      float pv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) pv[j] = po[(size_t)min(s0 + j, nact - 1) * head_dim];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(s0 + j < nact ? s_w[h * splits + s0 + j] : 0.0f, pv[j], acc);
    }
    attn_out[(size_t)seq * width + idx] = acc;
  }
}

// logits[b][v] = sum_k x[b][k] * W[v][k] for a tile of kLmRows activation rows (blockIdx.y), W fp16 [V, hidden], on
// the tensor cores without giving up the fp32 activations: x = hi + lo with hi = fp16(x), lo = fp16(x - hi) (error
// 2^-22 |x|), both halves in shared memory, every product w * hi and w * lo exact in the fp32 accumulator of
// mma.sync.m16n8k16.  A warp owns tiles of 16 vocabulary rows; per 32 values of k a lane loads 16 bytes of W rows
// g and g + 8 straight from global memory (k = 8 c .. 8 c + 7 of the step; the contraction index may be permuted
// freely as long as both operands agree, so two instructions use the words {0, 1} and {2, 3} of what was loaded)
// and, per 8 activation rows, 16 bytes of hi and of lo from shared memory for the same k.  Rows of the activation
// tile are padded to 64 bytes past a multiple of 128, which makes those 16-byte loads conflict-free.
// Each CTA also leaves, per activation row, its largest logit and the index (lowest index on ties) in
// best[b][blockIdx.x].  hidden must be a multiple of 32.
constexpr int kLmRows = 32;     // activation rows per CTA tile (4 column tiles of the instruction)
constexpr int kLmWarps = 16;
constexpr int kLmThreads = kLmWarps * 32;
__host__ __device__ inline size_t lm_row_bytes(int hidden) { return (size_t)hidden * 2 + 64; }
__host__ __device__ inline size_t lm_smem_bytes(int hidden) { return 2 * (size_t)kLmRows * lm_row_bytes(hidden); }

__device__ __forceinline__ void lm_mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kLmThreads, 1) lm_head_f16_batched_kernel(const float* __restrict__ x, int batch,
                                                                            const __half* __restrict__ w, int hidden,
                                                                            int vocab, float* __restrict__ logits,
                                                                            float2* __restrict__ best) {
  extern __shared__ __align__(128) uint8_t lm_smem[];
  __shared__ float s_bv[kLmRows][kLmWarps];
  __shared__ int s_bi[kLmRows][kLmWarps];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int b0 = blockIdx.y * kLmRows;
  const int nb = min(kLmRows, batch - b0);
  const size_t row_bytes = lm_row_bytes(hidden);
  uint8_t* s_hi = lm_smem;
  uint8_t* s_lo = lm_smem + (size_t)kLmRows * row_bytes;
  for (int i = tid; i < kLmRows * (hidden >> 1); i += kLmThreads) {  // two values per thread and trip
    const int r = i / (hidden >> 1), k = (i - r * (hidden >> 1)) * 2;
    float2 v = make_float2(0.0f, 0.0f);
    if (r < nb) v = *reinterpret_cast<const float2*>(x + (size_t)(b0 + r) * hidden + k);
    const __half2 hi = __floats2half2_rn(v.x, v.y);
    const float2 hf = __half22float2(hi);
    const __half2 lo = __floats2half2_rn(v.x - hf.x, v.y - hf.y);
    *reinterpret_cast<__half2*>(s_hi + (size_t)r * row_bytes + (size_t)k * 2) = hi;
    *reinterpret_cast<__half2*>(s_lo + (size_t)r * row_bytes + (size_t)k * 2) = lo;
  }
  __syncthreads();
  float bv[8];
  int bi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) bv[i] = -3.402823466e+38f, bi[i] = 0x7fffffff;
  const int steps = hidden >> 5;  // 32 values of k per step
  const uint32_t hi_s = (uint32_t)__cvta_generic_to_shared(s_hi) + (uint32_t)g * (uint32_t)row_bytes + (uint32_t)c * 16;
  const uint32_t lo_s = hi_s + (uint32_t)((size_t)kLmRows * row_bytes);
  for (int v0 = 16 * (blockIdx.x * kLmWarps + warp); v0 < vocab; v0 += 16 * kLmWarps * gridDim.x) {
    float acc[4][4];
#pragma unroll
    for (int t = 0; t < 4; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
    // rows past the end of the vocabulary repeat its last row (their results are dropped)
    const uint4* wa = reinterpret_cast<const uint4*>(w + (size_t)min(v0 + g, vocab - 1) * hidden) + c;
    const uint4* wb = reinterpret_cast<const uint4*>(w + (size_t)min(v0 + g + 8, vocab - 1) * hidden) + c;
#pragma unroll 4
    for (int ss = 0; ss < steps; ++ss) {
      const uint4 ra = wa[ss * 4], rb = wb[ss * 4];  // 16 bytes of either row: k = 32 ss + 8 c ..
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        uint4 xh, xl;
        const uint32_t off = (uint32_t)t * 8 * (uint32_t)row_bytes + (uint32_t)ss * 64;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(xh.x), "=r"(xh.y), "=r"(xh.z), "=r"(xh.w) : "r"(hi_s + off));
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(xl.x), "=r"(xl.y), "=r"(xl.z), "=r"(xl.w) : "r"(lo_s + off));
        lm_mma_f16(acc[t], ra.x, rb.x, ra.y, rb.y, xh.x, xh.y);
        lm_mma_f16(acc[t], ra.x, rb.x, ra.y, rb.y, xl.x, xl.y);
        lm_mma_f16(acc[t], ra.z, rb.z, ra.w, rb.w, xh.z, xh.w);
        lm_mma_f16(acc[t], ra.z, rb.z, ra.w, rb.w, xl.z, xl.w);
      }
    }
    // lane (g, c): rows v0 + g and v0 + g + 8, activation rows 8 t + 2 c and 8 t + 2 c + 1
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int v = v0 + g + (i >> 1) * 8, r = 8 * t + 2 * c + (i & 1);
        if (v < vocab && r < nb) {
          const float a = acc[t][i];
          if (logits) logits[(size_t)(b0 + r) * vocab + v] = a;
          const int slot = 2 * t + (i & 1);
          if (a > bv[slot]) {  // this lane meets the rows of a column in increasing order: a strict test keeps the lowest index
            bv[slot] = a;
            bi[slot] = v;
          }
        }
      }
  }
  // the eight lanes with the same c hold different vocabulary rows of the same activation rows
#pragma unroll
  for (int slot = 0; slot < 8; ++slot) {
    float v = bv[slot];
    int i = bi[slot];
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i, o);
      if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
      }
    }
    if (g == 0) {
      const int r = 8 * (slot >> 1) + 2 * c + (slot & 1);
      s_bv[r][warp] = v;
      s_bi[r][warp] = i;
    }
  }
  __syncthreads();
  if (tid < nb) {
    const int r = tid;
    float v = s_bv[r][0];
    int i = s_bi[r][0];
    for (int k = 1; k < kLmWarps; ++k)
      if (s_bv[r][k] > v || (s_bv[r][k] == v && s_bi[r][k] < i)) {
        v = s_bv[r][k];
        i = s_bi[r][k];
      }
    best[(size_t)(b0 + r) * gridDim.x + blockIdx.x] = make_float2(v, __int_as_float(i));
  }
}

// Greedy sampling and bookkeeping of a step for every sequence (one warp each): sample_advance_kernel per row.
__global__ void sample_advance_batched_kernel(const float2* __restrict__ best, int count, int* __restrict__ pos,
                                              int* __restrict__ token, int* __restrict__ history, int max_hist) {
  const int seq = blockIdx.x;
  best += (size_t)seq * count;
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
    const int p = pos[seq];
    token[seq] = bi;
    if (p < max_hist) history[(size_t)seq * max_hist + p] = bi;
    pos[seq] = p + 1;
  }
}

namespace {

constexpr int kLmCtas = 148;  // vocabulary CTAs of the batched lm_head (x ceil(B / 32) activation tiles)

struct BatchDecoder {
  Decoder* base = nullptr;
  int batch = 0;
  std::vector<float*> cache_k, cache_v;  // per layer: [batch][kv_heads][max_ctx][D]
  size_t cache_seq_stride = 0;
  float *h = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *o = nullptr;
  float *gate = nullptr, *up = nullptr, *act = nullptr, *down = nullptr, *logits = nullptr;
  float *part_o = nullptr, *part_ml = nullptr;
  // context split of the decode attention: with many sequences the grid is full without fine splits, and a CTA's fixed
  // cost (rotating the queries, the first cache round trip) is paid once per chunk - so chunks of about 128 positions
  // for large batches, the batch-1 decoder's fine split for small ones
  int attn_chunk = 32, attn_splits = 1;
  float2* best = nullptr;
  int *pos = nullptr, *token = nullptr, *history = nullptr, *scratch_next = nullptr;
  void* ws = nullptr;
  std::vector<int> host_pos;  // tokens in each sequence's cache (0 = not prefilled)
  cudaGraphExec_t graph = nullptr;
  int policy = 0;
  std::vector<void*> owned;
  int last_error = 0;
};

template <class T>
bool balloc(BatchDecoder* b, T** p, size_t count) {
  void* q = nullptr;
  if (cudaMalloc(&q, count * sizeof(T)) != cudaSuccess) return false;
  b->owned.push_back(q);
  *p = static_cast<T*>(q);
  return true;
}

#define BD_CHECK(expr)                      \
  do {                                      \
    cudaError_t e__ = (expr);               \
    if (e__ != cudaSuccess) {               \
      b->last_error = (int)e__;             \
      return MLLMB200_CUDA_ERROR;           \
    }                                       \
  } while (0)
#define BD_ST(expr)                         \
  do {                                      \
    int s__ = (expr);                       \
    if (s__ != MLLMB200_OK) return s__;     \
  } while (0)

int enqueue_batched_step(BatchDecoder* b) {
  Decoder* d = b->base;
  const auto& c = d->cfg;
  cudaStream_t s = d->stream;
  const int B = b->batch, H = c.hidden, QD = c.q_heads * c.head_dim, KD = c.kv_heads * c.head_dim, I = c.inter;
  const int group = c.q_heads / c.kv_heads;
  embedding_kernel<<<B, 256, 0, s>>>(b->token, d->embedding, H, b->h);
  for (int l = 0; l < c.layers; ++l) {
    const Layer& L = d->layers[l];
    add_rmsnorm_quant_kernel<<<B, 256, 0, s>>>(b->h, l == 0 ? nullptr : b->down, L.ln1, c.eps, H, b->h, b->xn, nullptr,
                                               nullptr, 0);
    {
      const void* tw[3] = {L.w[kQ], L.w[kK], L.w[kV]};
      float* ty[3] = {b->q, b->k, b->v};
      const int tn[3] = {QD, KD, KD};
      BD_ST(mllmb200_w4a32_linear_forward_grouped(b->xn, B, H, H, 3, tw, ty, tn, tn, b->ws, b->policy | 0x100, s));
    }
    {
      const dim3 grid(b->attn_splits, c.kv_heads, B);
      if (c.head_dim == 128 && MLLMB200_BATCH_ATTN_V2)
        attn_decode_partial_batched_v2_kernel<<<grid, kBa2Threads, 0, s>>>(
            b->q, QD, b->k, b->v, KD, d->sin_t, d->cos_t, b->pos, c.max_ctx, b->attn_chunk, group, c.q_heads, b->cache_k[l],
            b->cache_v[l], b->cache_seq_stride, b->part_o, b->part_ml, b->attn_splits);
      else if (c.head_dim == 128)
        attn_decode_partial_batched_kernel<128><<<grid, kAttnThreads, 0, s>>>(
            b->q, QD, b->k, b->v, KD, d->sin_t, d->cos_t, b->pos, c.max_ctx, b->attn_chunk, group, c.q_heads, b->cache_k[l],
            b->cache_v[l], b->cache_seq_stride, b->part_o, b->part_ml, b->attn_splits);
      else
        attn_decode_partial_batched_kernel<64><<<grid, kAttnThreads, 0, s>>>(
            b->q, QD, b->k, b->v, KD, d->sin_t, d->cos_t, b->pos, c.max_ctx, b->attn_chunk, group, c.q_heads, b->cache_k[l],
            b->cache_v[l], b->cache_seq_stride, b->part_o, b->part_ml, b->attn_splits);
      attn_combine_batched_kernel<<<B, kBatchCombineThreads, (size_t)c.q_heads * b->attn_splits * sizeof(float), s>>>(
          b->part_o, b->part_ml, b->pos, c.max_ctx, b->attn_chunk, b->attn_splits, c.q_heads, c.head_dim, b->attn);
    }
    BD_ST(mllmb200_w4a32_linear_forward_ex(b->attn, L.w[kO], b->o, b->ws, B, QD, H, QD, H, b->policy | 0x100, s));
    add_rmsnorm_quant_kernel<<<B, 256, 0, s>>>(b->h, b->o, L.ln2, c.eps, H, b->h, b->xn, nullptr, nullptr, 0);
    {
      const void* tw[2] = {L.w[kGate], L.w[kUp]};
      float* ty[2] = {b->gate, b->up};
      const int tn[2] = {I, I};
      BD_ST(mllmb200_w4a32_linear_forward_grouped(b->xn, B, H, H, 2, tw, ty, tn, tn, b->ws, b->policy | 0x100, s));
    }
    silu_mul_quant_kernel<<<B, 512, (size_t)I * sizeof(float), s>>>(b->gate, b->up, I, b->act, nullptr, nullptr, 0);
    BD_ST(mllmb200_w4a32_linear_forward_ex(b->act, L.w[kDown], b->down, b->ws, B, I, H, I, H, b->policy | 0x100, s));
  }
  add_rmsnorm_quant_kernel<<<B, 256, 0, s>>>(b->h, b->down, d->final_norm, c.eps, H, nullptr, b->xn, nullptr, nullptr, 0);
  {
    const dim3 grid(kLmCtas, (B + kLmRows - 1) / kLmRows);
    lm_head_f16_batched_kernel<<<grid, kLmThreads, lm_smem_bytes(H), s>>>(b->xn, B, d->lm_head, H, c.vocab,
                                                                                      b->logits, b->best);
  }
  sample_advance_batched_kernel<<<B, 32, 0, s>>>(b->best, kLmCtas, b->pos, b->token, b->history, c.max_ctx);
  BD_CHECK(cudaGetLastError());
  return MLLMB200_OK;
}

}  // namespace

// decoder.cu: the batch-1 prefill writing into the given caches and bookkeeping words.
int prefill_into(Decoder* d, const int* tokens_dev, const float* embeds_dev, int n, float* const* cache_k,
                 float* const* cache_v, int* pos, int* token, int* next, int* history);

}  // namespace mllmb200

using namespace mllmb200;

extern "C" {

int mllmb200_qwen2_batch_create(void* decoder, int batch, void** handle) {
  auto* d = static_cast<Decoder*>(decoder);
  if (!d || !handle || batch < 1 || batch > 1024) return MLLMB200_INVALID_ARG;
  const auto& c = d->cfg;
  if (c.hidden % 32 != 0) return MLLMB200_UNSUPPORTED;  // the batched lm_head walks k in steps of 32
  auto* b = new BatchDecoder();
  b->base = d;
  b->batch = batch;
  b->host_pos.assign(batch, 0);
  const size_t B = (size_t)batch;
  const int QD = c.q_heads * c.head_dim, KD = c.kv_heads * c.head_dim;
  b->cache_seq_stride = (size_t)c.kv_heads * c.max_ctx * c.head_dim;
  {
    // aim at about 4 CTAs per SM (two resident at a time; measured against 2, 8 and 16) over the (split, kv head, sequence) grid, chunks a multiple of 32 and at least the batch-1 chunk
    const long long want_splits = std::max<long long>(1, ((long long)MLLMB200_BATCH_ATTN_CTAS_PER_SM * 148) / ((long long)batch * c.kv_heads));
    int chunk = (int)((c.max_ctx + want_splits - 1) / want_splits);
    chunk = std::max(d->attn_chunk, (chunk + 31) / 32 * 32);
    b->attn_chunk = chunk;
    b->attn_splits = (c.max_ctx + chunk - 1) / chunk;
  }
  bool ok = balloc(b, &b->h, B * c.hidden) && balloc(b, &b->xn, B * c.hidden) && balloc(b, &b->q, B * QD) &&
            balloc(b, &b->k, B * KD) && balloc(b, &b->v, B * KD) && balloc(b, &b->attn, B * QD) && balloc(b, &b->o, B * c.hidden) &&
            balloc(b, &b->gate, B * c.inter) && balloc(b, &b->up, B * c.inter) && balloc(b, &b->act, B * c.inter) &&
            balloc(b, &b->down, B * c.hidden) && balloc(b, &b->logits, B * c.vocab) &&
            balloc(b, &b->part_o, B * c.q_heads * b->attn_splits * c.head_dim) &&
            balloc(b, &b->part_ml, B * c.q_heads * b->attn_splits * 2) && balloc(b, &b->best, B * kLmCtas) &&
            balloc(b, &b->pos, B) && balloc(b, &b->token, B) && balloc(b, &b->scratch_next, 1) &&
            balloc(b, &b->history, B * c.max_ctx);
  size_t wsb = 0;
  const int max_k = std::max(std::max(c.inter, c.hidden), QD);
  ok = ok && mllmb200_w4a32_workspace_size(batch, max_k, &wsb) == MLLMB200_OK;
  if (ok) {
    uint8_t* w = nullptr;
    ok = balloc(b, &w, wsb);
    b->ws = w;
  }
  b->cache_k.resize(c.layers);
  b->cache_v.resize(c.layers);
  for (int l = 0; ok && l < c.layers; ++l)
    ok = balloc(b, &b->cache_k[l], B * b->cache_seq_stride) && balloc(b, &b->cache_v[l], B * b->cache_seq_stride);
  if (ok)
    ok = cudaFuncSetAttribute(lm_head_f16_batched_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)lm_smem_bytes(c.hidden)) == cudaSuccess &&
         cudaMemsetAsync(b->pos, 0, B * sizeof(int), d->stream) == cudaSuccess &&
         cudaMemsetAsync(b->token, 0, B * sizeof(int), d->stream) == cudaSuccess &&
         cudaStreamSynchronize(d->stream) == cudaSuccess;
  if (!ok) {
    for (void* p : b->owned) cudaFree(p);
    delete b;
    return MLLMB200_CUDA_ERROR;
  }
  *handle = b;
  return MLLMB200_OK;
}

void mllmb200_qwen2_batch_destroy(void* handle) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b) return;
  cudaStreamSynchronize(b->base->stream);
  if (b->graph) cudaGraphExecDestroy(b->graph);
  for (void* p : b->owned) cudaFree(p);
  delete b;
}

// Kernel policy of the M = batch linears (0 auto: exact int32 group sums; 4 / 5: fp16 tensor cores where they apply).
int mllmb200_qwen2_batch_set_policy(void* handle, int policy) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b || (policy != 0 && policy != 4 && policy != 5)) return MLLMB200_INVALID_ARG;
  if (policy != b->policy && b->graph) {
    cudaGraphExecDestroy(b->graph);
    b->graph = nullptr;
  }
  b->policy = policy;
  return MLLMB200_OK;
}

// Prefills sequence `seq` from an empty cache and samples its first token.  Exactly one of tokens_dev (int32 [n])
// and embeds_dev (fp32 [n, hidden]: rows that are already embeddings, e.g. vision-patch embeddings mixed with
// looked-up text tokens) is given.  Asynchronous on the decoder's stream.
int mllmb200_qwen2_batch_prefill(void* handle, int seq, const int* tokens_dev, const float* embeds_dev, int n) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b || seq < 0 || seq >= b->batch || (tokens_dev == nullptr) == (embeds_dev == nullptr) || n <= 0 ||
      n >= b->base->cfg.max_ctx)
    return MLLMB200_INVALID_ARG;
  Decoder* d = b->base;
  const int layers = d->cfg.layers;
  std::vector<float*> ck(layers), cv(layers);
  for (int l = 0; l < layers; ++l) {
    ck[l] = b->cache_k[l] + (size_t)seq * b->cache_seq_stride;
    cv[l] = b->cache_v[l] + (size_t)seq * b->cache_seq_stride;
  }
  BD_ST(prefill_into(d, tokens_dev, embeds_dev, n, ck.data(), cv.data(), b->pos + seq, b->token + seq, b->scratch_next,
                     b->history + (size_t)seq * d->cfg.max_ctx));
  b->host_pos[seq] = n;
  return MLLMB200_OK;
}

// `steps` greedy steps for all sequences together (every sequence needs a prefill first and room in its cache).
int mllmb200_qwen2_batch_decode(void* handle, int steps) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b || steps < 0) return MLLMB200_INVALID_ARG;
  Decoder* d = b->base;
  for (int p : b->host_pos)
    if (p < 1 || p + steps > d->cfg.max_ctx) return MLLMB200_INVALID_ARG;
  if (steps == 0) return MLLMB200_OK;
  auto advance = [&] {
    for (int& p : b->host_pos) ++p;
  };
  if (!b->graph) {
    BD_ST(enqueue_batched_step(b));  // plain run first: kernel attributes get configured outside capture
    advance();
    BD_CHECK(cudaStreamSynchronize(d->stream));
    --steps;
    if (steps == 0) return MLLMB200_OK;
    cudaGraph_t g = nullptr;
    BD_CHECK(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
    const int st = enqueue_batched_step(b);
    cudaError_t e = cudaStreamEndCapture(d->stream, &g);
    if (st != MLLMB200_OK || e != cudaSuccess) {
      if (g) cudaGraphDestroy(g);
      if (st != MLLMB200_OK) return st;
      BD_CHECK(e);
    }
    e = cudaGraphInstantiate(&b->graph, g, 0);
    cudaGraphDestroy(g);
    BD_CHECK(e);
  }
  for (int i = 0; i < steps; ++i) {
    BD_CHECK(cudaGraphLaunch(b->graph, d->stream));
    advance();
  }
  return MLLMB200_OK;
}

// Synchronizes; copies to HOST memory history[first, first + count) of sequence `seq` (entry p = the token sampled
// after position p), its number of cached tokens, and the last logits [vocab] of that sequence; NULLs are skipped.
int mllmb200_qwen2_batch_read(void* handle, int seq, int first, int count, int* tokens_out, int* pos_out, float* logits_out) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b || seq < 0 || seq >= b->batch || first < 0 || count < 0 || first + count > b->base->cfg.max_ctx)
    return MLLMB200_INVALID_ARG;
  Decoder* d = b->base;
  BD_CHECK(cudaStreamSynchronize(d->stream));
  if (tokens_out && count)
    BD_CHECK(cudaMemcpy(tokens_out, b->history + (size_t)seq * d->cfg.max_ctx + first, (size_t)count * 4, cudaMemcpyDeviceToHost));
  if (pos_out) BD_CHECK(cudaMemcpy(pos_out, b->pos + seq, 4, cudaMemcpyDeviceToHost));
  if (logits_out)
    BD_CHECK(cudaMemcpy(logits_out, b->logits + (size_t)seq * d->cfg.vocab, (size_t)d->cfg.vocab * 4, cudaMemcpyDeviceToHost));
  return MLLMB200_OK;
}

}  // extern "C"
