// Persistent decode kernel: a whole greedy decode step (all layers, lm_head, sampling) - and any
// number of steps - in ONE cooperative launch of one CTA per SM.
//
// Why: at batch 1 a decoder layer is 26 MB of packed weights (4 us of HBM time on this GPU) but
// nine dependent kernel launches of 4-8 us each when every operator is its own launch.  Here the
// CTAs stay resident; each one owns a fixed share of every weight matrix (decoder_plan.h) and a
// producer warp streams that share through a 184 KB shared-memory ring with bulk copies
// (cp.async.bulk + mbarrier), running ahead of the compute warps across phase boundaries, so HBM
// is busy while the compute warps synchronize.  Phases are separated by a grid-wide barrier (one
// atomic counter in global memory; the cooperative launch guarantees that all CTAs are resident;
// every wait is bounded and raises the device status word instead of hanging).
//
// Per layer (reference project: mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:47-54,106-155,175-183):
//   P1  every CTA: residual add + RMSNorm + int8 activation quantization (redundantly, into its
//       own shared memory), then its share of the q,k,v GEMV           -> partial sums   | barrier
//   P2  attention over context splits (decoder_attn_body.cuh)         -> split partials | barrier
//   P2b merge of the splits, one CTA per query head                   -> attention row  | barrier
//   P3  quantize the attention row, share of the o GEMV               -> partial sums   | barrier
//   P4  residual add + RMSNorm + quantization, gate/up panel pairs, silu(g)*u -> activation row | barrier
//   P5  quantize the needed part of that row, share of the down GEMV  -> partial sums   | barrier
// then the final norm, the fp16 lm_head rows of this CTA and greedy sampling (every CTA reduces the
// per-CTA candidates itself, so the next step starts without another barrier).
// The residual stream lives replicated in every CTA's shared memory; nothing but partial sums,
// attention partials, the activation row and the KV cache goes through global memory (L2).
// GEMV arithmetic per cell is that of gemv.cu (exact int32 group sums by dp4a, one FMA per group
// scale); partial sums of a row are added in a fixed order, so results are deterministic.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <vector>

#include "decoder_attn_body.cuh"
#include "decoder_plan.h"
#include "decoder_state.h"
#include "device_common.cuh"

namespace mllmb200 {

constexpr int kPComputeWarps = 16;
constexpr int kPComputeThreads = kPComputeWarps * 32;
constexpr int kPThreads = kPComputeThreads + 32;  // + the producer warp
constexpr int kPSlots = 20;
constexpr int kPSlotBytes = kPlanChunkCells * kCellBytes;  // 9216
constexpr int kPMaxGroups = 320;                           // K <= 10240
constexpr int kPMaxHidden = 2048;

struct PersistLin {  // one weight matrix of one layer
  const uint8_t* base;
  uint32_t zsum_off, bias_off;
  int scale_mode, pad;
};
struct PersistLayer {
  const float *ln1, *ln2;
  float *cache_k, *cache_v;
};

struct PersistParams {
  int layers, hidden, q_heads, kv_heads, inter, vocab, max_ctx, steps;
  float eps;
  // plan
  const PlanChunk* chunks;
  const int* phase_begin;
  int max_chunks;
  const uint8_t *slots_qkv, *slots_o, *slots_down;
  const PersistLin* lins;      // [layers][7]
  const PersistLayer* layer;   // [layers]
  const float *final_norm, *embedding, *sin_t, *cos_t;
  const __half* lm_head;
  // scratch in global memory (L2)
  float *part_qkv, *part_o, *part_down;  // [kPlanMaxSlots][stride]
  int qkv_stride, h_stride;
  float *attn_po, *attn_ml, *attn_out;
  float2* head_minmax;  // [q_heads]
  int attn_chunk, attn_splits;
  float* act;           // [inter]
  float2* cta_minmax;   // [gridDim.x]
  float* logits;
  float2* best;         // [gridDim.x]
  int *pos, *token, *next, *history;
  unsigned* bar_counter;
  int* abort_flag;
};

__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, %0;" ::"n"(kPComputeThreads) : "memory"); }

// Sum / min-max over the compute threads; every thread gets the result.  red: 64 floats.
__device__ __forceinline__ float cblock_sum(float v, float* red, int warp, int lane) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  cbar();
  if (lane == 0) red[warp] = v;
  cbar();
  float t = lane < kPComputeWarps ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
__device__ __forceinline__ void cblock_minmax(float& mn, float& mx, float* red, int warp, int lane) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  cbar();
  if (lane == 0) {
    red[warp] = mn;
    red[32 + warp] = mx;
  }
  cbar();
  mn = lane < kPComputeWarps ? red[lane] : 3.402823466e+38f;
  mx = lane < kPComputeWarps ? red[32 + lane] : -3.402823466e+38f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
}

// Bounded wait on an mbarrier phase that also gives up when the CTA has been told to stop.
__device__ __forceinline__ bool pwait(uint64_t* bar, uint32_t parity, volatile int* s_abort, int* g_abort) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*s_abort) return false;
    if (clock64() - t0 > (1ll << 31)) {
      atomicOr(&g_device_status, kDevStatusTimeout);
      atomicExch(g_abort, 1);
      *s_abort = 1;
      return false;
    }
  }
  return true;
}

// Grid-wide barrier of the compute threads.  `epoch` counts barriers (same in every thread).
// Returns false - in every thread of the CTA alike - when the kernel is being abandoned: thread 0
// alone decides, between the two CTA barriers, and publishes the decision in *s_go.
__device__ __forceinline__ bool grid_barrier(const PersistParams& p, unsigned& epoch, volatile int* s_abort,
                                             volatile int* s_go, int tid) {
  ++epoch;
  cbar();
  if (tid == 0) {
    bool go = !*s_abort;
    if (go) {
      __threadfence();
      atomicAdd(p.bar_counter, 1u);
      const unsigned target = epoch * gridDim.x;
      const long long t0 = clock64();
      for (;;) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.bar_counter) : "memory");
        if (v >= target) break;
        if (*reinterpret_cast<volatile int*>(p.abort_flag)) {
          go = false;
          break;
        }
        if (clock64() - t0 > (1ll << 31)) {
          atomicOr(&g_device_status, kDevStatusTimeout);
          go = false;
          break;
        }
      }
      __threadfence();
    }
    if (!go) {
      atomicExch(p.abort_flag, 1);
      *s_abort = 1;
    }
    *s_go = go ? 1 : 0;
  }
  cbar();
  return *s_go != 0;
}

// int8 records (layout.h, kActRecordBytes) of groups [g_begin, g_end) of a row into shared memory.
// value(k) yields element k; every compute thread calls this (uniform trip count).
template <class F>
__device__ __forceinline__ void quantize_groups(F value, int g_begin, int g_end, const ActQuantParams& qp, uint8_t* arec,
                                                int tid) {
  const int first = g_begin * 4, last = g_end * 4;
  for (int base = first; base < last; base += kPComputeThreads) {
    const int item = base + tid;
    const bool valid = item < last;
    int q8[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q8[j] = valid ? act_quant_value(value(item * 8 + j), qp) : 0;
    const uint32_t lo = ((uint32_t)q8[0] & 0xFFu) | (((uint32_t)q8[2] & 0xFFu) << 8) | (((uint32_t)q8[4] & 0xFFu) << 16) |
                        (((uint32_t)q8[6] & 0xFFu) << 24);
    const uint32_t hi = ((uint32_t)q8[1] & 0xFFu) | (((uint32_t)q8[3] & 0xFFu) << 8) | (((uint32_t)q8[5] & 0xFFu) << 16) |
                        (((uint32_t)q8[7] & 0xFFu) << 24);
    int s = q8[0] + q8[1] + q8[2] + q8[3] + q8[4] + q8[5] + q8[6] + q8[7];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (valid) {
      const int g = item >> 2, i = item & 3;
      uint32_t* rec = reinterpret_cast<uint32_t*>(arec + (size_t)g * kActRecordBytes);
      rec[i] = lo;
      rec[4 + i] = hi;
      if (i == 0) rec[8] = (uint32_t)(-8 * s);
    }
  }
}

// Shared-memory carve-up (dynamic, 128-byte aligned base):
//   [0, 512)   full[kPSlots], empty[kPSlots] mbarriers, then small scalars
//   ring       kPSlots * 9216           weight chunks (bulk copy destinations)
//   arec       kPMaxGroups * 48         int8 activation records; raw q/k/v staging during attention
//   hrow       kPMaxHidden floats       the residual stream (persists across phases and layers)
//   work       kPMaxHidden floats       normalized row / attention scratch (AttnSmem) / merge scratch
//   red        16 * 32 floats           cross-warp partial sums, block reductions
constexpr size_t kPOffRing = 512;
constexpr size_t kPOffArec = kPOffRing + (size_t)kPSlots * kPSlotBytes;
constexpr size_t kPOffHrow = kPOffArec + (size_t)kPMaxGroups * kActRecordBytes;
constexpr size_t kPOffWork = kPOffHrow + (size_t)kPMaxHidden * 4;
constexpr size_t kPOffRed = kPOffWork + (size_t)kPMaxHidden * 4;
constexpr size_t kPSmemBytes = kPOffRed + (size_t)kPComputeWarps * 32 * 4 + 128;
static_assert(sizeof(AttnSmem<128>) <= (size_t)kPMaxHidden * 4, "attention scratch fits the work row");
static_assert(kPSmemBytes <= 227 * 1024, "persistent kernel shared memory");

template <int D>
__global__ void __launch_bounds__(kPThreads, 1) decode_persistent_kernel(const PersistParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kPSlots;
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + 2 * kPSlots * 8);
  volatile unsigned* s_issued = reinterpret_cast<volatile unsigned*>(smem + 2 * kPSlots * 8 + 4);
  volatile unsigned* s_consumed = reinterpret_cast<volatile unsigned*>(smem + 2 * kPSlots * 8 + 8);
  volatile int* s_token = reinterpret_cast<volatile int*>(smem + 2 * kPSlots * 8 + 12);
  volatile int* s_go = reinterpret_cast<volatile int*>(smem + 2 * kPSlots * 8 + 16);
  float* s_gate = reinterpret_cast<float*>(smem + 2 * kPSlots * 8 + 64);  // 32 floats
  uint8_t* ring = smem + kPOffRing;
  uint8_t* arec = smem + kPOffArec;
  float* hrow = reinterpret_cast<float*>(smem + kPOffHrow);
  float* work = reinterpret_cast<float*>(smem + kPOffWork);
  float* red = reinterpret_cast<float*>(smem + kPOffRed);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.hidden, QD = p.q_heads * D, KD = p.kv_heads * D, group = p.q_heads / p.kv_heads;
  const PlanChunk* my_chunks = p.chunks + (size_t)blockIdx.x * p.max_chunks;
  const int* pb = p.phase_begin + (size_t)blockIdx.x * (kPlanPhases + 1);

  if (tid == 0) {
    for (int i = 0; i < kPSlots; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kPComputeWarps);
    }
    *s_abort = 0;
    *s_issued = 0;
    *s_consumed = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kPComputeWarps) {
    // ------------------------------------------------------------------ producer warp
    if (lane == 0) {
      unsigned seq = 0;
      const int nch = pb[kPlanPhases];
      bool go = true;
      for (int step = 0; step < p.steps && go; ++step) {
        for (int l = 0; l < p.layers && go; ++l) {
          for (int i = 0; i < nch; ++i) {
            const PlanChunk ch = my_chunks[i];
            const unsigned slot = seq % kPSlots;
            if (seq >= (unsigned)kPSlots && !pwait(&empty[slot], ((seq / kPSlots) - 1u) & 1u, s_abort, p.abort_flag)) {
              go = false;
              break;
            }
            if (*s_abort) {
              go = false;
              break;
            }
            const PersistLin& L = p.lins[l * 7 + ch.lin];
            const uint32_t bytes = (uint32_t)ch.ncells * kCellBytes;
            mbar_arrive_expect_tx(&full[slot], bytes);
            bulk_g2s(ring + (size_t)slot * kPSlotBytes, L.base + ch.byte_off, bytes, &full[slot]);
            ++seq;
            *s_issued = seq;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    unsigned seq = 0, epoch = 0;
    bool ok = true;
    int pos = *p.pos, token = *p.token;
    float lhs_scale = 0.0f, a_off = 0.0f;  // of the row quantized last

    // residual add of a finished GEMV (partial slots in order), into hrow
    auto add_parts = [&](const float* parts, int stride, const uint8_t* slots) {
      for (int i = tid; i < H; i += kPComputeThreads) {
        float v = hrow[i];
        const int ns = slots[i >> 5];
        for (int s = 0; s < ns; ++s) v += __ldcg(parts + (size_t)s * stride + i);
        hrow[i] = v;
      }
    };
    // RMSNorm of hrow into work (mllm/Backends/Arm/Ops/RMSNormOp.cpp:20-77), optionally followed by
    // the quantization of the whole row into arec
    auto norm_row = [&](const float* w, bool quantize) {
      float ss = 0.0f;
      for (int i = tid; i < H; i += kPComputeThreads) ss += hrow[i] * hrow[i];
      const float rms = 1.0f / sqrtf(cblock_sum(ss, red, warp, lane) / (float)H + p.eps);
      float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
      for (int i = tid; i < H; i += kPComputeThreads) {
        const float y = hrow[i] * (w[i] * rms);
        work[i] = y;
        mn = fminf(mn, y);
        mx = fmaxf(mx, y);
      }
      if (!quantize) {
        cbar();
        return;
      }
      cblock_minmax(mn, mx, red, warp, lane);  // its barriers also publish `work`
      const ActQuantParams qp = act_quant_params(mn, mx);
      lhs_scale = qp.recip_scale;
      a_off = (float)(-qp.nzp);
      quantize_groups([&](int k) { return work[k]; }, 0, H / kGroup, qp, arec, tid);
      cbar();
    };
    // One cell: the lane's row of 32 nibbles against the group's record (same arithmetic as gemv.cu).
    auto do_cell = [&](const uint8_t* cell, int g, uint32_t scale_mode, float& acc) {
      const uint4 wq = *reinterpret_cast<const uint4*>(cell + lane * 16);
      const uint32_t sraw = *reinterpret_cast<const uint16_t*>(cell + kCellNibbleBytes + lane * 2);
      const float s = decode_scale(sraw, scale_mode);
      const uint8_t* rec = arec + (size_t)g * kActRecordBytes;
      const int4 alo = *reinterpret_cast<const int4*>(rec);
      const int4 ahi = *reinterpret_cast<const int4*>(rec + 16);
      int ia = *reinterpret_cast<const int*>(rec + 32), ib = 0;
      ia = __dp4a(alo.x, (int)(wq.x & 0x0F0F0F0Fu), ia);
      ib = __dp4a(ahi.x, (int)((wq.x >> 4) & 0x0F0F0F0Fu), ib);
      ia = __dp4a(alo.y, (int)(wq.y & 0x0F0F0F0Fu), ia);
      ib = __dp4a(ahi.y, (int)((wq.y >> 4) & 0x0F0F0F0Fu), ib);
      ia = __dp4a(alo.z, (int)(wq.z & 0x0F0F0F0Fu), ia);
      ib = __dp4a(ahi.z, (int)((wq.z >> 4) & 0x0F0F0F0Fu), ib);
      ia = __dp4a(alo.w, (int)(wq.w & 0x0F0F0F0Fu), ia);
      ib = __dp4a(ahi.w, (int)((wq.w >> 4) & 0x0F0F0F0Fu), ib);
      acc = fmaf((float)(ia + ib), s, acc);
    };
    // The CTA's share of one GEMV phase.  finish(ch, lin, part, zs, bs) runs in warp 0 (lane = row
    // of the panel) at the end of every panel run with the run's sum over the CTA's K-groups.
    auto gemv_phase = [&](int ph, int l, auto&& finish) {
      float acc = 0.0f, zs = 0.0f, bs = 0.0f;
      for (int i = pb[ph]; i < pb[ph + 1]; ++i) {  // trip count and barriers are uniform even after a failed wait
        const PlanChunk ch = my_chunks[i];
        const PersistLin& L = p.lins[l * 7 + ch.lin];
        if (warp == 0 && (ch.flags & kChunkFirstOfRun)) {  // per-row constants, requested early
          zs = reinterpret_cast<const float*>(L.base + L.zsum_off)[ch.panel * kPanelRows + lane];
          bs = reinterpret_cast<const float*>(L.base + L.bias_off)[ch.panel * kPanelRows + lane];
        }
        const unsigned slot = seq % kPSlots;
        ok = ok && pwait(&full[slot], (seq / kPSlots) & 1u, s_abort, p.abort_flag);
        ++seq;
        if (ok && warp < ch.ncells) do_cell(ring + (size_t)slot * kPSlotBytes + (size_t)warp * kCellBytes, ch.group0 + warp,
                                      (uint32_t)L.scale_mode, acc);
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(&empty[slot]);
        if (ch.flags & kChunkLastOfRun) {
          red[warp * 32 + lane] = acc;
          acc = 0.0f;
          cbar();
          if (warp == 0) {
            float part = 0.0f;
#pragma unroll
            for (int w = 0; w < kPComputeWarps; ++w) part += red[w * 32 + lane];
            finish(ch, part, zs, bs);
          }
          cbar();
        }
      }
    };
    // partial-sum epilogue: slot 0 carries the zero-point term and the bias
    auto store_partial = [&](float* parts, int stride, int n, const PlanChunk& ch, float part, float zs, float bs) {
      const float v = ch.slot == 0 ? fmaf(fmaf(a_off, zs, part), lhs_scale, bs) : part * lhs_scale;
      parts[(size_t)ch.slot * stride + n] = v;
    };

    bool alive = true;  // uniform over the compute threads: false once a grid barrier was abandoned
    for (int step = 0; step < p.steps && alive; ++step) {
      pos = min(pos, p.max_ctx - 1);
      for (int i = tid; i < H; i += kPComputeThreads) hrow[i] = p.embedding[(size_t)token * H + i];
      cbar();
      alive = false;
      int l = 0;
      for (; l < p.layers; ++l) {
        const PersistLayer& LY = p.layer[l];
        // ---------------- P1: norm + q,k,v
        if (l > 0) {
          add_parts(p.part_down, p.h_stride, p.slots_down);
          cbar();
        }
        norm_row(LY.ln1, true);
        gemv_phase(0, l, [&](const PlanChunk& ch, float part, float zs, float bs) {
          const int cat = (ch.lin == 0 ? 0 : (ch.lin == 1 ? QD : QD + KD)) + ch.panel * kPanelRows + lane;
          store_partial(p.part_qkv, p.qkv_stride, cat, ch, part, zs, bs);
        });
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        // ---------------- P2: attention over context splits
        for (int item = blockIdx.x; item < p.kv_heads * p.attn_splits; item += gridDim.x) {
          const int kvh = item / p.attn_splits, split = item - kvh * p.attn_splits;
          const int c0 = split * p.attn_chunk;
          if (c0 > pos) continue;
          float* raw = reinterpret_cast<float*>(arec);  // [group*D q | D k | D v], summed over the slots
          for (int idx = tid; idx < (group + 2) * D; idx += kPComputeThreads) {
            const int cat = idx < group * D ? kvh * group * D + idx
                                            : (idx < (group + 1) * D ? QD + kvh * D + (idx - group * D)
                                                                     : QD + KD + kvh * D + (idx - (group + 1) * D));
            const int ns = p.slots_qkv[cat >> 5];
            float v = 0.0f;
            for (int s = 0; s < ns; ++s) v += __ldcg(p.part_qkv + (size_t)s * p.qkv_stride + cat);
            raw[idx] = v;
          }
          cbar();
          attn_partial_body<D>(*reinterpret_cast<AttnSmem<D>*>(work), tid, [] { cbar(); }, raw, raw + group * D,
                               raw + (group + 1) * D, p.sin_t, p.cos_t, pos, c0, min(c0 + p.attn_chunk, pos + 1), group,
                               LY.cache_k + (size_t)kvh * p.max_ctx * D, LY.cache_v + (size_t)kvh * p.max_ctx * D,
                               p.attn_po + (size_t)kvh * group * p.attn_splits * D,
                               p.attn_ml + (size_t)kvh * group * p.attn_splits * 2, p.attn_splits, split);
          cbar();
        }
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        // ---------------- P2b: merge of the splits, one CTA per query head
        for (int h = blockIdx.x; h < p.q_heads; h += gridDim.x) {
          const int nact = min(p.attn_splits, pos / p.attn_chunk + 1);
          const float* ml = p.attn_ml + (size_t)h * p.attn_splits * 2;
          float* wsp = red;  // merge weights of the splits (attn_splits <= 64)
          if (warp == 0) {
            float mx = -3.402823466e+38f;
            for (int s = lane; s < nact; s += 32) mx = fmaxf(mx, __ldcg(ml + s * 2));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float tot = 0.0f;
            for (int s = lane; s < nact; s += 32) {
              const float e = expf(__ldcg(ml + s * 2) - mx);
              wsp[s] = e;
              tot += __ldcg(ml + s * 2 + 1) * e;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
            const float inv = 1.0f / tot;
            for (int s = lane; s < nact; s += 32) wsp[s] *= inv;
          }
          cbar();
          constexpr int NSG = kPComputeThreads / D;
          const int d = tid % D, sg = tid / D;
          const float* po = p.attn_po + (size_t)h * p.attn_splits * D + d;
          float acc = 0.0f;
          for (int s = sg; s < nact; s += NSG) acc = fmaf(wsp[s], __ldcg(po + (size_t)s * D), acc);
          work[sg * D + d] = acc;
          cbar();
          if (tid < D) {
            float v = 0.0f;
#pragma unroll
            for (int g = 0; g < NSG; ++g) v += work[g * D + tid];
            p.attn_out[h * D + tid] = v;
            float mn = v, mx = v;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
              mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
              mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            }
            if (lane == 0) {
              red[64 + warp] = mn;
              red[96 + warp] = mx;
            }
          }
          cbar();
          if (tid == 0) {
            float mn = red[64], mx = red[96];
            for (int w = 1; w < D / 32; ++w) {
              mn = fminf(mn, red[64 + w]);
              mx = fmaxf(mx, red[96 + w]);
            }
            p.head_minmax[h] = make_float2(mn, mx);
          }
          cbar();
        }
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        // ---------------- P3: quantize the attention row, o projection
        {
          float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
          for (int h = 0; h < p.q_heads; ++h) {
            const float2 mm = __ldcg(p.head_minmax + h);
            mn = fminf(mn, mm.x);
            mx = fmaxf(mx, mm.y);
          }
          const ActQuantParams qp = act_quant_params(mn, mx);
          lhs_scale = qp.recip_scale;
          a_off = (float)(-qp.nzp);
          quantize_groups([&](int k) { return __ldcg(p.attn_out + k); }, 0, QD / kGroup, qp, arec, tid);
          cbar();
        }
        gemv_phase(1, l, [&](const PlanChunk& ch, float part, float zs, float bs) {
          store_partial(p.part_o, p.h_stride, ch.panel * kPanelRows + lane, ch, part, zs, bs);
        });
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        // ---------------- P4: residual + norm, gate/up panel pairs, silu(g) * u
        add_parts(p.part_o, p.h_stride, p.slots_o);
        cbar();
        norm_row(LY.ln2, true);
        {
          float amn = 3.402823466e+38f, amx = -3.402823466e+38f;  // warp 0: over this CTA's activation rows
          gemv_phase(2, l, [&](const PlanChunk& ch, float part, float zs, float bs) {
            const float v = clamp_flt_max(fmaf(fmaf(a_off, zs, part), lhs_scale, bs));
            if (ch.lin == 4) {
              s_gate[lane] = v;
            } else {
              const float g = s_gate[lane];
              const float a = (g / (1.0f + expf(-g))) * v;
              p.act[ch.panel * kPanelRows + lane] = a;
              amn = fminf(amn, a);
              amx = fmaxf(amx, a);
            }
          });
          if (warp == 0) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
              amn = fminf(amn, __shfl_xor_sync(0xffffffffu, amn, o));
              amx = fmaxf(amx, __shfl_xor_sync(0xffffffffu, amx, o));
            }
            if (lane == 0) p.cta_minmax[blockIdx.x] = make_float2(amn, amx);
          }
        }
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        // ---------------- P5: quantize the needed part of the activation row, down projection
        {
          float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
          for (int c = tid; c < (int)gridDim.x; c += kPComputeThreads) {
            const float2 mm = __ldcg(p.cta_minmax + c);
            mn = fminf(mn, mm.x);
            mx = fmaxf(mx, mm.y);
          }
          cblock_minmax(mn, mx, red, warp, lane);
          const ActQuantParams qp = act_quant_params(mn, mx);
          lhs_scale = qp.recip_scale;
          a_off = (float)(-qp.nzp);
          for (int i = pb[3]; i < pb[4]; ++i) {
            const PlanChunk ch = my_chunks[i];
            if (ch.flags & kChunkFirstOfRun)
              quantize_groups([&](int k) { return __ldcg(p.act + k); }, ch.group0, ch.group0 + ch.run_groups, qp, arec, tid);
          }
          cbar();
        }
        gemv_phase(3, l, [&](const PlanChunk& ch, float part, float zs, float bs) {
          store_partial(p.part_down, p.h_stride, ch.panel * kPanelRows + lane, ch, part, zs, bs);
        });
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
      }
      if (l < p.layers) break;  // left the layer loop through an abandoned barrier
      // ---------------- final norm, lm_head rows of this CTA, greedy sampling
      add_parts(p.part_down, p.h_stride, p.slots_down);
      cbar();
      norm_row(p.final_norm, false);
      {
        const int v0 = (int)((long long)p.vocab * blockIdx.x / gridDim.x);
        const int v1 = (int)((long long)p.vocab * (blockIdx.x + 1) / gridDim.x);
        float bv = -3.402823466e+38f;
        int bi = 0x7fffffff;
        for (int v = v0 + warp; v < v1; v += kPComputeWarps) {
          const uint4* row = reinterpret_cast<const uint4*>(p.lm_head + (size_t)v * H);
          float acc = 0.0f;
          for (int c = lane; c < (H >> 3); c += 32) {
            const uint4 pk = row[c];
            const __half2* h2 = reinterpret_cast<const __half2*>(&pk);
            const float* xs = work + c * 8;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __half22float2(h2[j]);
              acc = fmaf(f.x, xs[2 * j], acc);
              acc = fmaf(f.y, xs[2 * j + 1], acc);
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
          if (lane == 0) p.logits[v] = acc;
          if (acc > bv) {
            bv = acc;
            bi = v;
          }
        }
        cbar();
        if (lane == 0) {
          red[warp] = bv;
          red[32 + warp] = __int_as_float(bi);
        }
        cbar();
        if (tid == 0) {
          for (int w = 1; w < kPComputeWarps; ++w) {
            const float ov = red[w];
            const int oi = __float_as_int(red[32 + w]);
            if (ov > bv || (ov == bv && oi < bi)) {
              bv = ov;
              bi = oi;
            }
          }
          p.best[blockIdx.x] = make_float2(bv, __int_as_float(bi));
        }
      }
      if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
      if (warp == 0) {  // every CTA reduces the candidates itself: lowest index wins ties (AutoLLM.hpp:70-105)
        float bv = -3.402823466e+38f;
        int bi = 0x7fffffff;
        for (int c = lane; c < (int)gridDim.x; c += 32) {
          const float2 cand = __ldcg(p.best + c);
          const int ci = __float_as_int(cand.y);
          if (cand.x > bv || (cand.x == bv && ci < bi)) {
            bv = cand.x;
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
        if (lane == 0) *s_token = bi;
      }
      cbar();
      token = *s_token;
      if (blockIdx.x == 0 && tid == 0) {
        if (pos < p.max_ctx) p.history[pos] = token;
        *p.next = token;
        *p.token = token;
        *p.pos = pos + 1;
      }
      pos += 1;
      alive = true;
    }
    if (tid == 0) *s_consumed = seq;
  }

  // ------------------------------------------------------------------ exit
  __syncthreads();
  if (tid == 0 && *s_abort) {
    // a wait gave up: let the copies that were issued but never consumed land before the CTA leaves
    for (unsigned q = *s_consumed; q < *s_issued; ++q) mbar_wait_bounded(&full[q % kPSlots], (q / kPSlots) & 1u);
  }
}

// ---- host side ---------------------------------------------------------------------------------
struct PersistentState {
  bool ready = false, usable = false;
  int nctas = 0;
  DecodePlan plan;
  PersistParams prm{};
  std::vector<void*> owned;
  int last_cuda_error = 0;
};

namespace {
template <class T>
bool pdev_copy(PersistentState* st, T** dst, const void* src, size_t bytes) {
  void* q = nullptr;
  if (cudaMalloc(&q, bytes ? bytes : 16) != cudaSuccess) return false;
  st->owned.push_back(q);
  if (src && bytes && cudaMemcpy(q, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return false;
  if (!src && bytes && cudaMemset(q, 0, bytes) != cudaSuccess) return false;
  *dst = static_cast<T*>(q);
  return true;
}
}  // namespace

PlanShape plan_shape_of(const mllmb200_qwen2_config& c) {
  return PlanShape{c.hidden, c.q_heads * c.head_dim, c.kv_heads * c.head_dim, c.inter};
}

// Builds the plan and the device tables once all weights are set.  Leaves usable = false (the
// decoder then keeps to its one-launch-per-operator path) when the device or the shape does not
// allow the persistent kernel.
void persistent_prepare(Decoder* d) {
  if (d->persist && d->persist->ready) return;
  if (!d->persist) d->persist = new PersistentState();
  PersistentState* st = d->persist;
  st->ready = true;
  const auto& c = d->cfg;
  int dev = 0, coop = 0, sms = 0, smem_optin = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (!coop || sms < 1 || (size_t)smem_optin < kPSmemBytes) return;
  if (c.hidden > kPMaxHidden || c.inter > kPMaxGroups * kGroup || c.q_heads * c.head_dim > kPMaxGroups * kGroup ||
      c.q_heads * c.head_dim > kPMaxHidden || d->attn_splits > 64 || (c.hidden % 32) || (c.inter % 32))
    return;
  const void* fn = c.head_dim == 128 ? (const void*)decode_persistent_kernel<128> : (const void*)decode_persistent_kernel<64>;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPSmemBytes) != cudaSuccess) return;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kPThreads, kPSmemBytes) != cudaSuccess || per_sm < 1) return;
  st->nctas = sms;
  const PlanShape shape = plan_shape_of(c);
  if (!build_decode_plan(shape, st->nctas, &st->plan) || check_decode_plan(shape, st->plan) != 0) return;

  PersistParams& p = st->prm;
  p.layers = c.layers, p.hidden = c.hidden, p.q_heads = c.q_heads, p.kv_heads = c.kv_heads, p.inter = c.inter;
  p.vocab = c.vocab, p.max_ctx = c.max_ctx, p.eps = c.eps;
  p.max_chunks = st->plan.max_chunks;
  const int QD = c.q_heads * c.head_dim, KD = c.kv_heads * c.head_dim;
  const int lin_n[7] = {QD, KD, KD, c.hidden, c.inter, c.inter, c.hidden};
  const int lin_k[7] = {c.hidden, c.hidden, c.hidden, QD, c.hidden, c.hidden, c.inter};
  std::vector<PersistLin> lins((size_t)c.layers * 7);
  std::vector<PersistLayer> lay(c.layers);
  for (int l = 0; l < c.layers; ++l) {
    for (int i = 0; i < 7; ++i) {
      const TiledHeader th = make_tiled_header(lin_n[i], lin_k[i], 0, 0);
      TiledHeader on_dev{};
      if (cudaMemcpy(&on_dev, d->layers[l].w[i], sizeof(TiledHeader), cudaMemcpyDeviceToHost) != cudaSuccess) return;
      if (on_dev.magic != kTiledMagic || on_dev.n != (uint32_t)lin_n[i] || on_dev.k != (uint32_t)lin_k[i]) return;
      lins[(size_t)l * 7 + i] = PersistLin{static_cast<const uint8_t*>(d->layers[l].w[i]), (uint32_t)th.zsum_off,
                                           (uint32_t)th.bias_off, (int)on_dev.scale_mode, 0};
    }
    lay[l] = PersistLayer{d->layers[l].ln1, d->layers[l].ln2, d->layers[l].cache_k, d->layers[l].cache_v};
  }
  p.qkv_stride = QD + 2 * KD;
  p.h_stride = c.hidden;
  bool ok = pdev_copy(st, const_cast<PlanChunk**>(&p.chunks), st->plan.chunks.data(), st->plan.chunks.size() * sizeof(PlanChunk)) &&
            pdev_copy(st, const_cast<int**>(&p.phase_begin), st->plan.phase_begin.data(), st->plan.phase_begin.size() * 4) &&
            pdev_copy(st, const_cast<uint8_t**>(&p.slots_qkv), st->plan.slots_qkv.data(), st->plan.slots_qkv.size()) &&
            pdev_copy(st, const_cast<uint8_t**>(&p.slots_o), st->plan.slots_o.data(), st->plan.slots_o.size()) &&
            pdev_copy(st, const_cast<uint8_t**>(&p.slots_down), st->plan.slots_down.data(), st->plan.slots_down.size()) &&
            pdev_copy(st, const_cast<PersistLin**>(&p.lins), lins.data(), lins.size() * sizeof(PersistLin)) &&
            pdev_copy(st, const_cast<PersistLayer**>(&p.layer), lay.data(), lay.size() * sizeof(PersistLayer)) &&
            pdev_copy(st, &p.part_qkv, nullptr, (size_t)kPlanMaxSlots * p.qkv_stride * 4) &&
            pdev_copy(st, &p.part_o, nullptr, (size_t)kPlanMaxSlots * p.h_stride * 4) &&
            pdev_copy(st, &p.part_down, nullptr, (size_t)kPlanMaxSlots * p.h_stride * 4) &&
            pdev_copy(st, &p.attn_out, nullptr, (size_t)QD * 4) && pdev_copy(st, &p.head_minmax, nullptr, (size_t)c.q_heads * 8) &&
            pdev_copy(st, &p.act, nullptr, (size_t)c.inter * 4) && pdev_copy(st, &p.cta_minmax, nullptr, (size_t)st->nctas * 8) &&
            pdev_copy(st, &p.best, nullptr, (size_t)st->nctas * 8) && pdev_copy(st, &p.bar_counter, nullptr, 4) &&
            pdev_copy(st, &p.abort_flag, nullptr, 4);
  if (!ok) return;
  p.final_norm = d->final_norm, p.embedding = d->embedding, p.sin_t = d->sin_t, p.cos_t = d->cos_t, p.lm_head = d->lm_head;
  p.attn_po = d->part_o, p.attn_ml = d->part_ml, p.attn_chunk = d->attn_chunk, p.attn_splits = d->attn_splits;
  p.logits = d->logits;
  p.pos = d->pos, p.token = d->token, p.next = d->next, p.history = d->history;
  st->usable = true;
}

bool persistent_usable(Decoder* d) { return d->persist && d->persist->ready && d->persist->usable; }

// `steps` decode steps in one cooperative launch on the decoder's stream.
cudaError_t persistent_decode(Decoder* d, int steps) {
  PersistentState* st = d->persist;
  PersistParams prm = st->prm;
  prm.steps = steps;
  prm.embedding = d->embedding, prm.lm_head = d->lm_head;
  cudaError_t e = cudaMemsetAsync(prm.bar_counter, 0, 4, d->stream);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(prm.abort_flag, 0, 4, d->stream);
  if (e != cudaSuccess) return e;
  void* args[] = {&prm};
  const void* fn = d->cfg.head_dim == 128 ? (const void*)decode_persistent_kernel<128> : (const void*)decode_persistent_kernel<64>;
  return cudaLaunchCooperativeKernel(fn, dim3(st->nctas), dim3(kPThreads), args, kPSmemBytes, d->stream);
}

void persistent_destroy(Decoder* d) {
  if (!d->persist) return;
  for (void* q : d->persist->owned) cudaFree(q);
  delete d->persist;
  d->persist = nullptr;
}

}  // namespace mllmb200

// Host-only check of the persistent kernel's work plan for a model shape and CTA count (no GPU
// needed): builds the plan and verifies that every weight cell is streamed exactly once.
extern "C" int mllmb200_qwen2_plan_check(const mllmb200_qwen2_config* cfg, int nctas, int* max_chunks, int* max_slots,
                                         int* total_chunks) {
  using namespace mllmb200;
  if (!cfg || nctas < 1) return MLLMB200_INVALID_ARG;
  DecodePlan plan;
  const PlanShape shape = plan_shape_of(*cfg);
  if (!build_decode_plan(shape, nctas, &plan)) return MLLMB200_UNSUPPORTED;
  if (check_decode_plan(shape, plan) != 0) return MLLMB200_INVALID_ARG;
  if (max_chunks) *max_chunks = plan.max_chunks;
  if (max_slots) *max_slots = plan.max_slots;
  if (total_chunks) {
    int t = 0;
    for (int c = 0; c < nctas; ++c) t += plan.phase_begin[(size_t)c * (kPlanPhases + 1) + kPlanPhases];
    *total_chunks = t;
  }
  return MLLMB200_OK;
}
