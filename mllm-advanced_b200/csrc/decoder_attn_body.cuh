// One CTA's share of the decode-step attention (one new token), used by the stand-alone kernel
// (decoder_attn.cu) and by the persistent decode kernel (decoder_persistent.cu).
//
// The context is split over CTAs so that the whole GPU works on it.  The caller covers cache
// positions [c0, c1) of one KV head for all `group` query heads that share it and gets, per query
// head, an unnormalized partial output with its running maximum and sum (the usual online-softmax
// split); a merge step combines the splits.  The CTA whose range contains the new position `pos`
// rotates the new key, appends key and value to the cache and uses them directly, so no separate
// append pass is needed.  Follows the reference project's attention
// (mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:127-150; RoPE mllm/Backends/Arm/Kernels/rope.cpp:20-87).
//
// sin_row / cos_row: the D/2 rotation sines and cosines of position `pos`.
// Threads tid < 256 work; the caller may run more threads, all of which must call the body (they
// only take part in `sync`, which must synchronize every calling thread).
// part_o: [group][splits][D], part_ml: [group][splits][2] = {max, sum}, both for this KV head.
#pragma once
#include "device_common.cuh"

namespace mllmb200 {

constexpr int kAttnThreads = 256;
constexpr int kAttnMaxGroup = 8;
constexpr int kAttnSub = 32;  // positions per inner block

template <int D>
struct AttnSmem {
  float q[kAttnMaxGroup * D];
  float s[kAttnMaxGroup][kAttnSub];
  float alpha[kAttnMaxGroup], mrun[kAttnMaxGroup], lrun[kAttnMaxGroup];
};

template <int D, class Sync>
__device__ __forceinline__ void attn_partial_body(AttnSmem<D>& sm, int tid, Sync sync, const float* q, const float* kn,
                                                  const float* vn, const float* __restrict__ sin_row,
                                                  const float* __restrict__ cos_row, int pos, int c0, int c1, int group,
                                                  float* kc, float* vc, float* part_o, float* part_ml, int splits,
                                                  int split) {
  constexpr int VEC = D / 32, NG = kAttnThreads / D, HALF = D / 2, MAXH = (kAttnMaxGroup + NG - 1) / NG;
  const bool active = tid < kAttnThreads;
  const int warp = tid >> 5, lane = tid & 31;
  const float scale = 1.0f / sqrtf((float)D);
  constexpr int PER_WARP = kAttnSub / (kAttnThreads / 32);
  const int pd = tid % D, pg = tid / D;  // the output element / head slot this thread accumulates
  float kv[PER_WARP][VEC];  // this warp's key rows of the block (lane = VEC consecutive elements)
  float vv[kAttnSub];       // element pd of the block's value rows
  // All cache loads of a block are issued together, before anything that depends on them: they
  // are L2 round trips (the rows may have been written by another SM earlier in the same launch).
  auto load_block = [&](int b0) {
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
            const float sn = sin_row[dd], cs = cos_row[dd];
            const float x0 = kn[dd], x1 = kn[dd + HALF];
            kv[j][e] = d < HALF ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs);
            kc[(size_t)pos * D + d] = kv[j][e];
          }
        } else if constexpr (VEC == 4) {
          const float4 v4 = __ldcg(reinterpret_cast<const float4*>(kc + (size_t)t * D + lane * 4));
          kv[j][0] = v4.x, kv[j][1] = v4.y, kv[j][2] = v4.z, kv[j][3] = v4.w;
        } else {
          const float2 v2 = __ldcg(reinterpret_cast<const float2*>(kc + (size_t)t * D + lane * 2));
          kv[j][0] = v2.x, kv[j][1] = v2.y;
        }
      }
    }
    const int nt = min(kAttnSub, c1 - b0);
#pragma unroll
    for (int t = 0; t < kAttnSub; ++t) {
      vv[t] = 0.0f;
      if (t < nt) {
        if (b0 + t == pos) {
          vv[t] = vn[pd];
          if (pg == 0) vc[(size_t)pos * D + pd] = vv[t];
        } else {
          vv[t] = __ldcg(vc + (size_t)(b0 + t) * D + pd);
        }
      }
    }
  };
  if (active) load_block(c0);
  // rotated queries of the group
  if (active) {
    for (int idx = tid; idx < group * D; idx += kAttnThreads) {
      const int h = idx / D, d = idx - h * D;
      const float* qr = q + (size_t)h * D;
      const int dd = d < HALF ? d : d - HALF;
      const float sn = sin_row[dd], cs = cos_row[dd];
      const float x0 = qr[dd], x1 = qr[dd + HALF];
      sm.q[idx] = d < HALF ? (x0 * cs - x1 * sn) : (x0 * sn + x1 * cs);
    }
    if (tid < kAttnMaxGroup) {
      sm.mrun[tid] = -3.402823466e+38f;
      sm.lrun[tid] = 0.0f;
    }
  }
  float o_acc[MAXH];
#pragma unroll
  for (int i = 0; i < MAXH; ++i) o_acc[i] = 0.0f;
  sync();

  for (int b0 = c0; b0 < c1; b0 += kAttnSub) {
    // ---- scores: warp w holds positions b0 + w + 8 j
    if (active) {
      for (int h = 0; h < group; ++h) {
        float qv[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) qv[e] = sm.q[h * D + lane * VEC + e];
#pragma unroll
        for (int j = 0; j < PER_WARP; ++j) {
          float acc = 0.0f;
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc = fmaf(qv[e], kv[j][e], acc);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
          const int tl = warp + j * (kAttnThreads / 32);
          if (lane == 0) sm.s[h][tl] = (b0 + tl < c1) ? acc * scale : -3.402823466e+38f;
        }
      }
    }
    sync();
    // ---- online softmax bookkeeping: warp h owns head h
    if (active && warp < group) {
      const float sc = sm.s[warp][lane];
      float mx = sc;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = sm.mrun[warp], m_new = fmaxf(m_old, mx);
      const float p = (b0 + lane < c1) ? expf(sc - m_new) : 0.0f;
      float sum = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      sm.s[warp][lane] = p;
      if (lane == 0) {
        const float alpha = expf(m_old - m_new);  // 0 on the first block (m_old = -FLT_MAX)
        sm.alpha[warp] = alpha;
        sm.mrun[warp] = m_new;
        sm.lrun[warp] = sm.lrun[warp] * alpha + sum;
      }
    }
    sync();
    // ---- P.V: thread (pd, pg) accumulates element pd of heads pg, pg + NG, ...
    if (active) {
#pragma unroll
      for (int i = 0; i < MAXH; ++i) {
        const int h = pg + i * NG;
        if (h < group) {
          float acc = o_acc[i] * sm.alpha[h];
#pragma unroll
          for (int t = 0; t < kAttnSub; ++t) acc = fmaf(sm.s[h][t], vv[t], acc);
          o_acc[i] = acc;
        }
      }
    }
    sync();
    if (active && b0 + kAttnSub < c1) load_block(b0 + kAttnSub);
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < MAXH; ++i) {
      const int h = pg + i * NG;
      if (h < group) part_o[((size_t)h * splits + split) * D + pd] = o_acc[i];
    }
    if (tid < group) {
      float* ml = part_ml + ((size_t)tid * splits + split) * 2;
      ml[0] = sm.mrun[tid];
      ml[1] = sm.lrun[tid];
    }
  }
}

}  // namespace mllmb200
