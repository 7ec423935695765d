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

// ---------------------------------------------------------------------------------------------
// Prefill attention, tiled: grid (ceil(S / R), kv_heads), R * W warps (R = kPfRows = 4 query rows, W = kPfHeadWarps = 4
// warps per row).  A CTA owns R consecutive query rows of all `group` query heads that share one KV head (R * group
// <= 32 query vectors, rotated into shared memory once) and walks the cache in blocks of 32 positions up to the causal
// limit: a key/value block is read from L2 once per CTA (not once per head and row), scores are formed with lane = key
// position (key rows padded to D + 1 floats: no bank conflicts), and the running softmax (max, sum, rescale) is the
// usual online form.  A block is a chain of dependent steps (stage, barrier, scores, softmax, barrier, P.V, barrier)
// whose length - not the SM's throughput - set the run time: with 8 rows and one warp per row the launch took as long as
// the tile with the longest causal range (16 blocks of ~8 us on a 512-token prompt: 134 us per layer, SMs busy half of
// the time).  Now each warp takes the heads w / R, w / R + W, .. of its row (a shorter chain per block), a tile has 4
// rows (more CTAs than SMs), and the tiles are dispatched longest first: 512-token prefill of the 1.5B model 8.3 -> 7.1 ms.
// Arithmetic: scores * 1/sqrt(D), causal mask, softmax, P.V (modeling_ds_qwen2.hpp:127-150 of the reference project).
// q: rows of ldq floats, row s at position pos0 + s; out: rows of ldo floats.
// ---------------------------------------------------------------------------------------------
#ifndef MLLMB200_PF_ROWS
#define MLLMB200_PF_ROWS 4
#endif
#ifndef MLLMB200_PF_LONGEST_FIRST
#define MLLMB200_PF_LONGEST_FIRST 1
#endif
#ifndef MLLMB200_PF_HEAD_WARPS
#define MLLMB200_PF_HEAD_WARPS 4
#endif
constexpr int kPfRows = MLLMB200_PF_ROWS;  // query rows per CTA
constexpr int kPfHeadWarps = MLLMB200_PF_HEAD_WARPS;  // warps per query row: warp w owns row w % rows and the heads w / rows, w / rows + kPfHeadWarps, ..
constexpr int kPfKeys = 32;     // cache positions per block
constexpr int kPfThreads = kPfRows * kPfHeadWarps * 32;
constexpr int kPfHeadsPerWarp = (kAttnMaxGroup + kPfHeadWarps - 1) / kPfHeadWarps;

template <int D>
struct PrefillAttnSmem {
  float q[kPfRows * kAttnMaxGroup][D];
  float k[kPfKeys][D + 1];
  float v[kPfKeys][D];
  float p[kPfRows * kAttnMaxGroup][kPfKeys];
  float alpha[kPfRows * kAttnMaxGroup], lsum[kPfRows * kAttnMaxGroup];
};

template <int D>
__global__ void __launch_bounds__(kPfThreads) attention_prefill_kernel(
    const float* __restrict__ q, int ldq, int S, const float* __restrict__ sin_t, const float* __restrict__ cos_t,
    const int* __restrict__ pos0_ptr, int max_ctx, int group, const float* __restrict__ cache_k,
    const float* __restrict__ cache_v, float* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) uint8_t pf_smem[];
  PrefillAttnSmem<D>& sm = *reinterpret_cast<PrefillAttnSmem<D>*>(pf_smem);
  constexpr int HALF = D / 2, NG = kPfThreads / (D / 4), QPT = (kPfRows * kAttnMaxGroup + NG - 1) / NG;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // CTAs are dispatched in order of blockIdx.x and a tile's work grows with its position (causal range): the last
  // tile goes first, so that the long ones start together and the short ones fill the SMs that free up
  const int tile = MLLMB200_PF_LONGEST_FIRST ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int s0 = tile * kPfRows, kvh = blockIdx.y;
  const int pos0 = *pos0_ptr;
  const int nrows = min(kPfRows, S - s0);
  const int nq = group * kPfRows;  // query vectors of this CTA: index = h * kPfRows + r
  // rotated queries (rows past S stay zero)
  for (int idx = tid; idx < nq * D; idx += kPfThreads) {
    const int qi = idx / D, d = idx - qi * D;
    const int h = qi / kPfRows, r = qi - h * kPfRows;
    float val = 0.0f;
    if (r < nrows) {
      const int pos = min(pos0 + s0 + r, max_ctx - 1);
      const float* qr = q + (size_t)(s0 + r) * ldq + (kvh * group + h) * D;
      const int dd = d < HALF ? d : d - HALF;
      const float sn = sin_t[pos * HALF + dd], cs = cos_t[pos * HALF + dd];
      const float x0 = qr[dd], x1 = qr[dd + HALF];
      val = d < HALF ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs);
    }
    sm.q[qi][d] = val;
  }
  const float scale = 1.0f / sqrtf((float)D);
  const float* kbase = cache_k + (size_t)kvh * max_ctx * D;
  const float* vbase = cache_v + (size_t)kvh * max_ctx * D;
  const int last_pos = min(pos0 + s0 + nrows - 1, max_ctx - 1);  // causal limit of the tile
  // running state: warp w owns query vectors w, w + 8, ... (lane-uniform copies of max and sum)
  float m_run[kPfHeadsPerWarp], l_run[kPfHeadsPerWarp];
#pragma unroll
  for (int i = 0; i < kPfHeadsPerWarp; ++i) m_run[i] = -3.402823466e+38f, l_run[i] = 0.0f;
  const int wr = warp % kPfRows, wh = warp / kPfRows;  // this warp's query row and first head
  // output accumulators: thread (pc, pg) holds elements 4 pc .. 4 pc + 3 of query vectors pg, pg + NG, ...
  // (a 4-wide register tile: one 16-byte value load and one 16-byte probability load feed 16 FMAs -
  // the kernel is bound by shared-memory wavefronts, not by FMAs)
  const int pc = tid % (D / 4), pg = tid / (D / 4);
  float o_acc[QPT][4];
#pragma unroll
  for (int i = 0; i < QPT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;

  // A block's key/value rows are requested into registers one block ahead (L2 round trips of ~1k
  // cycles each otherwise sit between the blocks): thread t moves chunks t, t + 256, ... of the block.
  constexpr int kLd = kPfKeys * (D / 4) / kPfThreads;  // 16-byte chunks per thread and matrix
  float4 kreg[kLd], vreg[kLd];
  auto fetch = [&](int b0) {
    const int nk = min(kPfKeys, last_pos + 1 - b0);
#pragma unroll
    for (int u = 0; u < kLd; ++u) {
      const int idx = tid + u * kPfThreads;
      const int j = idx / (D / 4), c = idx - j * (D / 4);
      kreg[u] = vreg[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < nk) {
        kreg[u] = *reinterpret_cast<const float4*>(kbase + (size_t)(b0 + j) * D + c * 4);
        vreg[u] = *reinterpret_cast<const float4*>(vbase + (size_t)(b0 + j) * D + c * 4);
      }
    }
  };
  fetch(0);
  for (int b0 = 0; b0 <= last_pos; b0 += kPfKeys) {
    const int nk = min(kPfKeys, last_pos + 1 - b0);
    __syncthreads();  // the previous block's k, v, p are no longer read
#pragma unroll
    for (int u = 0; u < kLd; ++u) {
      const int idx = tid + u * kPfThreads;
      const int j = idx / (D / 4), c = idx - j * (D / 4);
      sm.k[j][c * 4 + 0] = kreg[u].x, sm.k[j][c * 4 + 1] = kreg[u].y, sm.k[j][c * 4 + 2] = kreg[u].z, sm.k[j][c * 4 + 3] = kreg[u].w;
      *reinterpret_cast<float4*>(&sm.v[j][c * 4]) = vreg[u];
    }
    if (b0 + kPfKeys <= last_pos) fetch(b0 + kPfKeys);
    __syncthreads();
    // ---- scores: lane = key position, warp w takes query vectors w + 8 i
    {
      float sc[kPfHeadsPerWarp];
#pragma unroll
      for (int i = 0; i < kPfHeadsPerWarp; ++i) sc[i] = 0.0f;
#pragma unroll 4
      for (int d = 0; d < D; d += 4) {  // query elements as 16-byte broadcast loads, key elements scalar (padded rows)
        const float k0 = sm.k[lane][d], k1 = sm.k[lane][d + 1], k2 = sm.k[lane][d + 2], k3 = sm.k[lane][d + 3];
#pragma unroll
        for (int i = 0; i < kPfHeadsPerWarp; ++i) {
          if (wh + kPfHeadWarps * i < group) {
            const float4 q4 = *reinterpret_cast<const float4*>(&sm.q[wr + kPfRows * (wh + kPfHeadWarps * i)][d]);
            sc[i] = fmaf(q4.x, k0, sc[i]);
            sc[i] = fmaf(q4.y, k1, sc[i]);
            sc[i] = fmaf(q4.z, k2, sc[i]);
            sc[i] = fmaf(q4.w, k3, sc[i]);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < kPfHeadsPerWarp; ++i) {
        if (wh + kPfHeadWarps * i >= group) break;
        const int qi = wr + kPfRows * (wh + kPfHeadWarps * i);  // = h * kPfRows + r
        const int pos = pos0 + s0 + wr;        // position of this query row
        const bool valid = lane < nk && b0 + lane <= pos && wr < nrows;
        const float sv = valid ? sc[i] * scale : -3.402823466e+38f;
        float mx = sv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m_run[i], mx);
        const float pv = valid ? expf(sv - m_new) : 0.0f;
        float sum = pv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float alpha = expf(m_run[i] - m_new);
        m_run[i] = m_new;
        l_run[i] = l_run[i] * alpha + sum;
        sm.p[qi][lane] = pv;
        if (lane == 0) {
          sm.alpha[qi] = alpha;
          sm.lsum[qi] = l_run[i];
        }
      }
    }
    __syncthreads();
    // ---- P.V: keys outermost, so that a value row is loaded once for all query vectors of the thread
#pragma unroll
    for (int i = 0; i < QPT; ++i) {
      const int qi = pg + i * NG;
      const float al = qi < nq ? sm.alpha[qi] : 1.0f;
      o_acc[i][0] *= al, o_acc[i][1] *= al, o_acc[i][2] *= al, o_acc[i][3] *= al;
    }
#pragma unroll 2
    for (int j = 0; j < kPfKeys; j += 4) {
      float4 v4[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) v4[jj] = *reinterpret_cast<const float4*>(&sm.v[j + jj][pc * 4]);
#pragma unroll
      for (int i = 0; i < QPT; ++i) {
        const int qi = pg + i * NG;
        if (qi < nq) {
          const float4 p4 = *reinterpret_cast<const float4*>(&sm.p[qi][j]);
          const float pj[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            o_acc[i][0] = fmaf(pj[jj], v4[jj].x, o_acc[i][0]);
            o_acc[i][1] = fmaf(pj[jj], v4[jj].y, o_acc[i][1]);
            o_acc[i][2] = fmaf(pj[jj], v4[jj].z, o_acc[i][2]);
            o_acc[i][3] = fmaf(pj[jj], v4[jj].w, o_acc[i][3]);
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < QPT; ++i) {
    const int qi = pg + i * NG;
    if (qi < nq) {
      const int h = qi / kPfRows, r = qi - h * kPfRows;
      if (r < nrows) {
        const float inv = 1.0f / sm.lsum[qi];
        *reinterpret_cast<float4*>(out + (size_t)(s0 + r) * ldo + (kvh * group + h) * D + pc * 4) =
            make_float4(o_acc[i][0] * inv, o_acc[i][1] * inv, o_acc[i][2] * inv, o_acc[i][3] * inv);
      }
    }
  }
}

template __global__ void attention_prefill_kernel<64>(const float*, int, int, const float*, const float*, const int*, int, int,
                                                      const float*, const float*, float*, int);
template __global__ void attention_prefill_kernel<128>(const float*, int, int, const float*, const float*, const int*, int, int,
                                                       const float*, const float*, float*, int);
int attention_prefill_rows() { return kPfRows; }
int attention_prefill_threads() { return kPfThreads; }
size_t attention_prefill_smem_bytes(int head_dim) {
  return head_dim == 128 ? sizeof(PrefillAttnSmem<128>) : sizeof(PrefillAttnSmem<64>);
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
