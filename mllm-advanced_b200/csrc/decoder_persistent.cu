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

constexpr int kPComputeWarps = 8;  // few, fat warps: up to 224 registers each, two cells of a chunk per warp
constexpr int kPComputeThreads = kPComputeWarps * 32;
constexpr int kPThreads = kPComputeThreads + 32;  // + the producer warp
constexpr int kPSlots = 20;
constexpr int kPSlotBytes = kPlanChunkCells * kCellBytes;  // 9216
constexpr int kPMaxGroups = 296;                           // K <= 9472
constexpr int kPMaxHidden = 2048;
constexpr int kPMaxLayers = 48;   // per-layer tables are kept in shared memory
constexpr int kPMaxChunks = 64;   // chunks per CTA and layer
constexpr int kPMaxPanels = 256;  // slot-table entries (q,k,v panels + o panels + down panels)
constexpr int kPStamps = 26;  // profiling slots per CTA (see decode_persistent_kernel)

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
  long long* phase_cycles;  // [gridDim.x][kPStamps] clock cycles per phase, summed over layers and steps (may be null)
};

__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, %0;" ::"n"(kPComputeThreads) : "memory"); }

// Sum / min-max over the compute threads; every thread gets the result.  scratch: 64 floats that no
// thread still reads (the callers rotate over four such buffers, so one barrier per reduction is enough).
__device__ __forceinline__ float cblock_sum(float v, float* scratch, int warp, int lane) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) scratch[warp] = v;
  cbar();
  float t = lane < kPComputeWarps ? scratch[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
__device__ __forceinline__ void cblock_minmax(float& mn, float& mx, float* scratch, int warp, int lane) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0) {
    scratch[warp] = mn;
    scratch[32 + warp] = mx;
  }
  cbar();
  mn = lane < kPComputeWarps ? scratch[lane] : 3.402823466e+38f;
  mx = lane < kPComputeWarps ? scratch[32 + lane] : -3.402823466e+38f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
}

// Bounded wait on an mbarrier phase that also gives up when the CTA has been told to stop.
// kSleep: back off between polls (the producer's wait for a free slot is never urgent, and a
// spinning warp takes issue slots from the compute warps of its scheduler).
template <bool kSleep = false>
__device__ __forceinline__ bool pwait(uint64_t* bar, uint32_t parity, volatile int* s_abort, int* g_abort) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (kSleep) __nanosleep(256);
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
      const unsigned target = epoch * gridDim.x;
      unsigned v;
      // release: the CTA barrier above ordered every compute thread's writes before this;
      // acquire: for the last arriver, whose own increment completes the count
      asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(v) : "l"(p.bar_counter) : "memory");
      ++v;
      const long long t0 = clock64();
      while (v < target) {  // the last arriver sees its own increment complete the count and never polls
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

// One pass of quantize_groups on values that are already in registers: thread tid holds the 8
// elements of item item0 + pass * kPComputeThreads + tid (zeros when that is past nitems).
__device__ __forceinline__ void quantize_item(const float (&v)[8], int item0, int nitems, int pass,
                                              const ActQuantParams& qp, uint8_t* arec, int tid) {
  const int rel = pass * kPComputeThreads + tid;
  const bool valid = rel < nitems;
  const int item = item0 + rel;
  int q8[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) q8[j] = valid ? act_quant_value(v[j], qp) : 0;
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
// The loads for quantize_item: two 16-byte L2 loads per thread (src 32-byte aligned per item).
__device__ __forceinline__ void preload_item(const float* src, int item0, int nitems, int pass, float (&v)[8], int tid) {
  const int rel = pass * kPComputeThreads + tid;
  if (rel < nitems) {
    const float4* q = reinterpret_cast<const float4*>(src + (size_t)(item0 + rel) * 8);
    const float4 a = __ldcg(q), b = __ldcg(q + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.0f;
  }
}

// Shared-memory carve-up (dynamic, 128-byte aligned base):
//   [0, 512)   full[kPSlots], empty[kPSlots] mbarriers, then small scalars
//   ring       kPSlots * 9216           weight chunks (bulk copy destinations)
//   arec       kPMaxGroups * 48         int8 activation records; raw q/k/v staging during attention
//   hrow       kPMaxHidden floats       the residual stream (persists across phases and layers)
//   work       kPMaxHidden floats       normalized row / attention scratch (AttnSmem) / merge scratch
//   red        2 * 16 * 32 floats       cross-warp partial sums of the panel runs (two buffers, alternating)
//   redx       4 * 64 floats            block-reduction scratch (four buffers, rotating)
constexpr size_t kPOffRing = 512;
constexpr size_t kPOffArec = kPOffRing + (size_t)kPSlots * kPSlotBytes;
constexpr size_t kPOffHrow = kPOffArec + (size_t)kPMaxGroups * kActRecordBytes;
constexpr size_t kPOffWork = kPOffHrow + (size_t)kPMaxHidden * 4;
constexpr size_t kPOffRed = kPOffWork + (size_t)kPMaxHidden * 4;
constexpr size_t kPOffRedx = kPOffRed + (size_t)2 * kPComputeWarps * 32 * 4;
constexpr size_t kPOffTime = kPOffRedx + (size_t)4 * 64 * 4;
//   tables     this CTA's chunk list, the slot tables, the per-layer weight and pointer tables: read
//              on every chunk and phase, so they must not cost an L2 round trip each time
constexpr size_t kPOffChunks = kPOffTime + (size_t)kPStamps * 8;
constexpr size_t kPOffSlots = kPOffChunks + (size_t)kPMaxChunks * sizeof(PlanChunk);
constexpr size_t kPOffLins = kPOffSlots + (size_t)kPMaxPanels;
constexpr size_t kPOffLayers = kPOffLins + (size_t)kPMaxLayers * 7 * sizeof(PersistLin);
constexpr size_t kPOffRope = kPOffLayers + (size_t)kPMaxLayers * sizeof(PersistLayer);  // sin | cos of this step's position
constexpr size_t kPSmemBytes = kPOffRope + 128 * 4 + 128;
static_assert(sizeof(PersistLin) == 24 && sizeof(PersistLayer) == 32, "table entry sizes");
static_assert(kPOffLins % 8 == 0 && kPOffLayers % 8 == 0 && kPOffChunks % 16 == 0, "table alignment");
static_assert(kPlanChunkCells == 2 * kPComputeWarps && kPComputeThreads == kAttnThreads, "warp / cell / attention thread mapping");
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
  float* redx = reinterpret_cast<float*>(smem + kPOffRedx);
  long long* s_time = reinterpret_cast<long long*>(smem + kPOffTime);
  float* s_rope = reinterpret_cast<float*>(smem + kPOffRope);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = p.hidden, QD = p.q_heads * D, KD = p.kv_heads * D, group = p.q_heads / p.kv_heads;
  int pb[kPlanPhases + 1];
#pragma unroll
  for (int k = 0; k <= kPlanPhases; ++k) pb[k] = p.phase_begin[(size_t)blockIdx.x * (kPlanPhases + 1) + k];
  const PlanChunk* my_chunks = reinterpret_cast<const PlanChunk*>(smem + kPOffChunks);
  const uint8_t* slots_qkv = smem + kPOffSlots;
  const uint8_t* slots_o = slots_qkv + (QD + 2 * KD) / kPanelRows;
  const uint8_t* slots_down = slots_o + H / kPanelRows;
  const PersistLin* lins = reinterpret_cast<const PersistLin*>(smem + kPOffLins);
  const PersistLayer* layer_tab = reinterpret_cast<const PersistLayer*>(smem + kPOffLayers);
  {  // fill the tables (all threads)
    const uint32_t* src = reinterpret_cast<const uint32_t*>(p.chunks + (size_t)blockIdx.x * p.max_chunks);
    uint32_t* dst = reinterpret_cast<uint32_t*>(smem + kPOffChunks);
    for (int i = tid; i < p.max_chunks * 4; i += kPThreads) dst[i] = src[i];
    uint8_t* sl = smem + kPOffSlots;
    const int nq = (QD + 2 * KD) / kPanelRows, nh = H / kPanelRows;
    for (int i = tid; i < nq; i += kPThreads) sl[i] = p.slots_qkv[i];
    for (int i = tid; i < nh; i += kPThreads) {
      sl[nq + i] = p.slots_o[i];
      sl[nq + nh + i] = p.slots_down[i];
    }
    const uint32_t* ls = reinterpret_cast<const uint32_t*>(p.lins);
    uint32_t* ld = reinterpret_cast<uint32_t*>(smem + kPOffLins);
    for (int i = tid; i < p.layers * 7 * (int)(sizeof(PersistLin) / 4); i += kPThreads) ld[i] = ls[i];
    const uint32_t* ys = reinterpret_cast<const uint32_t*>(p.layer);
    uint32_t* yd = reinterpret_cast<uint32_t*>(smem + kPOffLayers);
    for (int i = tid; i < p.layers * (int)(sizeof(PersistLayer) / 4); i += kPThreads) yd[i] = ys[i];
  }

  if (tid == 0) {
    for (int i = 0; i < kPSlots; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kPComputeWarps);
    }
    *s_abort = 0;
    *s_issued = 0;
    *s_consumed = 0;
    for (int i = 0; i < kPStamps; ++i) s_time[i] = 0;
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
            if (seq >= (unsigned)kPSlots && !pwait<true>(&empty[slot], ((seq / kPSlots) - 1u) & 1u, s_abort, p.abort_flag)) {
              go = false;
              break;
            }
            if (*s_abort) {
              go = false;
              break;
            }
            const PersistLin& L = lins[l * 7 + ch.lin];
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
    unsigned rot = 0, flush_no = 0;        // rotation of the reduction scratch / of the run-flush buffers
    auto scratch = [&]() { return redx + 64 * (rot++ & 3u); };
    // profiling: thread 0 adds the cycles since its previous stamp to slot k
    long long t_last = clock64();
    auto stamp = [&](int k) {
      if (tid == 0 && p.phase_cycles) {
        const long long now = clock64();
        s_time[k] += now - t_last;
        t_last = now;
      }
    };

    // residual add of a finished GEMV (partial slots in order), into hrow
    auto add_parts = [&](const float* parts, int stride, const uint8_t* slots) {
      // all loads first (each is an L2 round trip), then the sums in slot order
      constexpr int PER = kPMaxHidden / kPComputeThreads;
      float t[PER][kPlanMaxSlots];
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = tid + j * kPComputeThreads;
        const int ns = i < H ? slots[i >> 5] : 0;
#pragma unroll
        for (int s = 0; s < kPlanMaxSlots; ++s) t[j][s] = s < ns ? __ldcg(parts + (size_t)s * stride + i) : 0.0f;
      }
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = tid + j * kPComputeThreads;
        if (i < H) {
          float v = hrow[i];
#pragma unroll
          for (int s = 0; s < kPlanMaxSlots; ++s) v += t[j][s];
          hrow[i] = v;
        }
      }
    };
    // RMSNorm of hrow into work (mllm/Backends/Arm/Ops/RMSNormOp.cpp:20-77), optionally followed by
    // the quantization of the whole row into arec
    constexpr int kPer = kPMaxHidden / kPComputeThreads;  // row elements per thread
    // norm weights are first touched once per layer and token (an HBM round trip): they are
    // requested a phase ahead into registers
    auto load_w = [&](const float* w, float (&wv)[kPer]) {
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const int i = tid + j * kPComputeThreads;
        wv[j] = i < H ? w[i] : 0.0f;
      }
    };
    auto norm_row = [&](const float (&wv)[kPer], bool quantize) {
      constexpr int PER = kPer;
      float ss = 0.0f;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = tid + j * kPComputeThreads;
        if (i < H) ss += hrow[i] * hrow[i];
      }
      const float rms = 1.0f / sqrtf(cblock_sum(ss, scratch(), warp, lane) / (float)H + p.eps);
      float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = tid + j * kPComputeThreads;
        if (i < H) {
          const float y = hrow[i] * (wv[j] * rms);
          work[i] = y;
          mn = fminf(mn, y);
          mx = fmaxf(mx, y);
        }
      }
      if (!quantize) {
        cbar();
        return;
      }
      cblock_minmax(mn, mx, scratch(), warp, lane);  // its barrier also publishes `work`
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
    // Per-row constants (zsum, bias) of a phase's panel runs and the norm weights are first touched
    // once per layer and token - an HBM round trip when loaded on demand.  They are pulled into L2
    // a phase ahead with prefetch hints (no registers, nothing waits on them); the loads at the
    // point of use are then L2 hits.
    auto l2_prefetch = [&](const void* ptr) { asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr)); };
    auto prefetch_consts = [&](int ph, int l) {
      if (warp != 0 || lane >= 8) return;  // 8 lanes x 32 bytes cover one run's 128-byte zsum row; same for bias
      for (int i = pb[ph]; i < pb[ph + 1]; ++i) {
        const PlanChunk ch = my_chunks[i];
        if (!(ch.flags & kChunkFirstOfRun)) continue;
        const PersistLin& L = lins[l * 7 + ch.lin];
        const float* z = reinterpret_cast<const float*>(L.base + L.zsum_off) + ch.panel * kPanelRows;
        const float* b = reinterpret_cast<const float*>(L.base + L.bias_off) + ch.panel * kPanelRows;
        l2_prefetch(lane < 4 ? z + lane * 8 : b + (lane - 4) * 8);
      }
    };
    auto prefetch_row = [&](const float* w) {  // H floats
      if (warp == 1 && lane * 8 < H)
        for (int i = lane * 8; i < H; i += 256) l2_prefetch(w + i);
    };
    // The CTA's share of one GEMV phase.  finish(ch, part, zs, bs) runs in warp 0 (lane = row of the
    // panel) at the end of every panel run with the run's sum over the CTA's K-groups.
    auto gemv_phase = [&](int ph, int l, auto&& finish) {
      float acc = 0.0f, zs = 0.0f, bs = 0.0f;
      // end of a panel run: warps -> one of two shared buffers (alternating, so one barrier is
      // enough: a buffer is rewritten two flushes later, after warp 0 passed the barrier in between)
      auto flush = [&](const PlanChunk& ch) {
        float* rb = red + (flush_no++ & 1u) * (kPComputeWarps * 32);
        rb[warp * 32 + lane] = acc;
        acc = 0.0f;
        cbar();
        if (warp == 0) {
          float part = 0.0f;
#pragma unroll
          for (int w = 0; w < kPComputeWarps; ++w) part += rb[w * 32 + lane];
          finish(ch, part, zs, bs);
        }
        stamp(22);
      };
      auto open_run = [&](const PlanChunk& ch, const PersistLin& L, float& z, float& b) {  // the run's constants (L2 hits)
        if (warp == 0 && (ch.flags & kChunkFirstOfRun)) {
          z = reinterpret_cast<const float*>(L.base + L.zsum_off)[ch.panel * kPanelRows + lane];
          b = reinterpret_cast<const float*>(L.base + L.bias_off)[ch.panel * kPanelRows + lane];
        }
      };
      // Two chunks (<= 16 cells each) per trip: both waits first, then warp w takes cells w and w + 8
      // of each as four independent instruction chains.  Trip count and barriers are uniform over
      // the compute threads even after a failed wait.
      for (int i = pb[ph]; i < pb[ph + 1]; i += 2) {
        const bool two = i + 1 < pb[ph + 1];
        const PlanChunk ca = my_chunks[i];
        const PlanChunk cb = my_chunks[two ? i + 1 : i];
        const PersistLin& La = lins[l * 7 + ca.lin];
        const PersistLin& Lb = lins[l * 7 + cb.lin];
        const unsigned sa = seq % kPSlots, sb = (seq + 1) % kPSlots;
        float zs2 = zs, bs2 = bs;  // the second chunk may open a new run while the first closes the old one
        open_run(ca, La, zs, bs);
        if (two) open_run(cb, Lb, zs2, bs2);
        stamp(21);
        ok = ok && pwait(&full[sa], (seq / kPSlots) & 1u, s_abort, p.abort_flag);
        if (two) ok = ok && pwait(&full[sb], ((seq + 1) / kPSlots) & 1u, s_abort, p.abort_flag);
        stamp(20);
        seq += two ? 2 : 1;
        float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
        const uint8_t* cells_a = ring + (size_t)sa * kPSlotBytes;
        const uint8_t* cells_b = ring + (size_t)sb * kPSlotBytes;
        const int w2 = warp + kPComputeWarps;
        if (ok && warp < ca.ncells) do_cell(cells_a + (size_t)warp * kCellBytes, ca.group0 + warp, (uint32_t)La.scale_mode, a0);
        if (ok && two && warp < cb.ncells) do_cell(cells_b + (size_t)warp * kCellBytes, cb.group0 + warp, (uint32_t)Lb.scale_mode, b0);
        if (ok && w2 < ca.ncells) do_cell(cells_a + (size_t)w2 * kCellBytes, ca.group0 + w2, (uint32_t)La.scale_mode, a1);
        if (ok && two && w2 < cb.ncells) do_cell(cells_b + (size_t)w2 * kCellBytes, cb.group0 + w2, (uint32_t)Lb.scale_mode, b1);
        __syncwarp();
        if (lane == 0 && ok) {
          mbar_arrive(&empty[sa]);
          if (two) mbar_arrive(&empty[sb]);
        }
        acc += a0 + a1;
        if (ca.flags & kChunkLastOfRun) flush(ca);
        if (two) {
          if (cb.flags & kChunkFirstOfRun) {
            zs = zs2;
            bs = bs2;
          }
          acc += b0 + b1;
          if (cb.flags & kChunkLastOfRun) flush(cb);
        }
      }
    };
    // partial-sum epilogue: slot 0 carries the zero-point term and the bias
    auto store_partial = [&](float* parts, int stride, int n, const PlanChunk& ch, float part, float zs, float bs) {
      const float v = ch.slot == 0 ? fmaf(fmaf(a_off, zs, part), lhs_scale, bs) : part * lhs_scale;
      parts[(size_t)ch.slot * stride + n] = v;
    };

    if (p.phase_cycles) {  // profiling probes: 8 dependent L2 loads, then 4 empty grid barriers
      stamp(25);
      if (tid == 0) {
        int off = 0;
        for (int r = 0; r < 8; ++r) off = (int)(__ldcg(p.part_down + 32 * r + off) * 0.0f);
        if (off == 12345) p.part_down[0] = 0.0f;
      }
      stamp(23);
      bool g = true;
      for (int r = 0; r < 4 && g; ++r) g = grid_barrier(p, epoch, s_abort, s_go, tid);
      stamp(24);
    }
    float wv1[kPer];  // norm weights of the row being normalized
    bool alive = true;  // uniform over the compute threads: false once a grid barrier was abandoned
    for (int step = 0; step < p.steps && alive; ++step) {
      pos = min(pos, p.max_ctx - 1);
      for (int i = tid; i < H; i += kPComputeThreads) hrow[i] = p.embedding[(size_t)token * H + i];
      if (tid < D) s_rope[tid] = tid < D / 2 ? p.sin_t[(size_t)pos * (D / 2) + tid] : p.cos_t[(size_t)pos * (D / 2) + tid - D / 2];
      prefetch_consts(0, 0);
      cbar();
      alive = false;
      int l = 0;
      for (; l < p.layers; ++l) {
        const PersistLayer& LY = layer_tab[l];
        // ---------------- P1: norm + q,k,v
        prefetch_consts(1, l);  // for P3; P1's own were requested during the previous layer's P5
        prefetch_row(LY.ln2);
        load_w(LY.ln1, wv1);
        if (l > 0) add_parts(p.part_down, p.h_stride, slots_down);
        norm_row(wv1, true);
        stamp(0);
        gemv_phase(0, l, [&](const PlanChunk& ch, float part, float zs, float bs) {
          const int cat = (ch.lin == 0 ? 0 : (ch.lin == 1 ? QD : QD + KD)) + ch.panel * kPanelRows + lane;
          store_partial(p.part_qkv, p.qkv_stride, cat, ch, part, zs, bs);
        });
        stamp(1);
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        stamp(2);
        // ---------------- P2: attention over context splits
        for (int item = blockIdx.x; item < p.kv_heads * p.attn_splits; item += gridDim.x) {
          const int kvh = item / p.attn_splits, split = item - kvh * p.attn_splits;
          const int c0 = split * p.attn_chunk;
          if (c0 > pos) continue;
          float* raw = reinterpret_cast<float*>(arec);  // [group*D q | D k | D v], summed over the slots
          {
            constexpr int PER = ((kAttnMaxGroup + 2) * D + kPComputeThreads - 1) / kPComputeThreads;
            float t[PER][kPlanMaxSlots];
#pragma unroll
            for (int j = 0; j < PER; ++j) {
              const int idx = tid + j * kPComputeThreads;
              const int cat = idx < group * D ? kvh * group * D + idx
                                              : (idx < (group + 1) * D ? QD + kvh * D + (idx - group * D)
                                                                       : QD + KD + kvh * D + (idx - (group + 1) * D));
              const int ns = idx < (group + 2) * D ? slots_qkv[cat >> 5] : 0;
#pragma unroll
              for (int s = 0; s < kPlanMaxSlots; ++s)
                t[j][s] = s < ns ? __ldcg(p.part_qkv + (size_t)s * p.qkv_stride + cat) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < PER; ++j) {
              const int idx = tid + j * kPComputeThreads;
              if (idx < (group + 2) * D) {
                float v = 0.0f;
#pragma unroll
                for (int s = 0; s < kPlanMaxSlots; ++s) v += t[j][s];
                raw[idx] = v;
              }
            }
          }
          cbar();
          attn_partial_body<D>(*reinterpret_cast<AttnSmem<D>*>(work), tid, [] { cbar(); }, raw, raw + group * D,
                               raw + (group + 1) * D, s_rope, s_rope + D / 2, pos, c0, min(c0 + p.attn_chunk, pos + 1), group,
                               LY.cache_k + (size_t)kvh * p.max_ctx * D, LY.cache_v + (size_t)kvh * p.max_ctx * D,
                               p.attn_po + (size_t)kvh * group * p.attn_splits * D,
                               p.attn_ml + (size_t)kvh * group * p.attn_splits * 2, p.attn_splits, split);
          cbar();
        }
        stamp(3);
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        stamp(4);
        // ---------------- P2b: merge of the splits, one CTA per query head
        for (int h = blockIdx.x; h < p.q_heads; h += gridDim.x) {
          const int nact = min(p.attn_splits, pos / p.attn_chunk + 1);
          const float* ml = p.attn_ml + (size_t)h * p.attn_splits * 2;
          float* wsp = red;  // merge weights of the splits (attn_splits <= 64)
          if (warp == 0) {
            const float2 ml0 = lane < nact ? __ldcg(reinterpret_cast<const float2*>(ml) + lane) : make_float2(-3.402823466e+38f, 0.0f);
            const float2 ml1 = lane + 32 < nact ? __ldcg(reinterpret_cast<const float2*>(ml) + lane + 32)
                                                : make_float2(-3.402823466e+38f, 0.0f);
            float mx = fmaxf(ml0.x, ml1.x);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float e0 = lane < nact ? expf(ml0.x - mx) : 0.0f, e1 = lane + 32 < nact ? expf(ml1.x - mx) : 0.0f;
            float tot = ml0.y * e0 + ml1.y * e1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
            const float inv = 1.0f / tot;
            wsp[lane] = e0 * inv;
            wsp[lane + 32] = e1 * inv;
          }
          cbar();
          constexpr int NSG = kPComputeThreads / D;
          const int d = tid % D, sg = tid / D;
          const float* po = p.attn_po + (size_t)h * p.attn_splits * D + d;
          float acc = 0.0f;
          {
            constexpr int PER = 64 / NSG;  // attn_splits <= 64
            float pv[PER];
#pragma unroll
            for (int j = 0; j < PER; ++j) {
              const int sp = sg + j * NSG;
              pv[j] = sp < nact ? __ldcg(po + (size_t)sp * D) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < PER; ++j) {
              const int sp = sg + j * NSG;
              if (sp < nact) acc = fmaf(wsp[sp], pv[j], acc);
            }
          }
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
        stamp(5);
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        stamp(6);
        // ---------------- P3: quantize the attention row, o projection
        {
          prefetch_consts(2, l);  // for P4
          float v8[8];  // QD <= 2048: one item of 8 elements per thread, requested together with the bounds
          preload_item(p.attn_out, 0, QD / 8, 0, v8, tid);
          float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
          if (lane < p.q_heads) {  // q_heads <= 32: one load per lane, every warp on its own
            const float2 mm = __ldcg(p.head_minmax + lane);
            mn = mm.x;
            mx = mm.y;
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          }
          const ActQuantParams qp = act_quant_params(mn, mx);
          lhs_scale = qp.recip_scale;
          a_off = (float)(-qp.nzp);
          quantize_item(v8, 0, QD / 8, 0, qp, arec, tid);
          cbar();
        }
        stamp(7);
        gemv_phase(1, l, [&](const PlanChunk& ch, float part, float zs, float bs) {
          store_partial(p.part_o, p.h_stride, ch.panel * kPanelRows + lane, ch, part, zs, bs);
        });
        stamp(8);
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        stamp(9);
        // ---------------- P4: residual + norm, gate/up panel pairs, silu(g) * u
        prefetch_consts(3, l);  // for P5
        prefetch_row(l + 1 < p.layers ? layer_tab[l + 1].ln1 : p.final_norm);
        load_w(LY.ln2, wv1);
        add_parts(p.part_o, p.h_stride, slots_o);
        norm_row(wv1, true);
        stamp(10);
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
        stamp(11);
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        stamp(12);
        // ---------------- P5: quantize the needed part of the activation row, down projection
        {
          if (l + 1 < p.layers) prefetch_consts(0, l + 1);  // for the next layer's P1
          // the K-group ranges of this CTA's first two panel runs: their first two passes of items
          // are requested together with the bounds; anything beyond that is loaded afterwards
          int rg0[2] = {0, 0}, rn[2] = {0, 0}, nr = 0;
          for (int i = pb[3]; i < pb[4]; ++i) {
            const PlanChunk ch = my_chunks[i];
            if (ch.flags & kChunkFirstOfRun) {
              if (nr == 0) rg0[0] = ch.group0, rn[0] = ch.run_groups;
              if (nr == 1) rg0[1] = ch.group0, rn[1] = ch.run_groups;
              ++nr;
            }
          }
          float v8[2][2][8];
#pragma unroll
          for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int ps = 0; ps < 2; ++ps) preload_item(p.act, rg0[r] * 4, rn[r] * 4, ps, v8[r][ps], tid);
          float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
          {  // every warp on its own: up to 8 loads per lane in flight, then a shuffle reduction
            float2 mm[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int c = lane + 32 * j;
              mm[j] = c < (int)gridDim.x ? __ldcg(p.cta_minmax + c) : make_float2(3.402823466e+38f, -3.402823466e+38f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              mn = fminf(mn, mm[j].x);
              mx = fmaxf(mx, mm[j].y);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
              mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
              mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            }
          }
          const ActQuantParams qp = act_quant_params(mn, mx);
          lhs_scale = qp.recip_scale;
          a_off = (float)(-qp.nzp);
#pragma unroll
          for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int ps = 0; ps < 2; ++ps) quantize_item(v8[r][ps], rg0[r] * 4, rn[r] * 4, ps, qp, arec, tid);
            constexpr int kPre = 2 * kPComputeThreads / 4;  // groups covered by the two preloaded passes
            if (rn[r] > kPre)
              quantize_groups([&](int k) { return __ldcg(p.act + k); }, rg0[r] + kPre, rg0[r] + rn[r], qp, arec, tid);
          }
          if (nr > 2) {
            int seen = 0;
            for (int i = pb[3]; i < pb[4]; ++i) {
              const PlanChunk ch = my_chunks[i];
              if ((ch.flags & kChunkFirstOfRun) && seen++ >= 2)
                quantize_groups([&](int k) { return __ldcg(p.act + k); }, ch.group0, ch.group0 + ch.run_groups, qp, arec, tid);
            }
          }
          cbar();
        }
        stamp(13);
        gemv_phase(3, l, [&](const PlanChunk& ch, float part, float zs, float bs) {
          store_partial(p.part_down, p.h_stride, ch.panel * kPanelRows + lane, ch, part, zs, bs);
        });
        stamp(14);
        if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
        stamp(15);
      }
      if (l < p.layers) break;  // left the layer loop through an abandoned barrier
      // ---------------- final norm, lm_head rows of this CTA, greedy sampling
      add_parts(p.part_down, p.h_stride, slots_down);
      load_w(p.final_norm, wv1);
      norm_row(wv1, false);
      stamp(16);
      {
        const int v0 = (int)((long long)p.vocab * blockIdx.x / gridDim.x);
        const int v1 = (int)((long long)p.vocab * (blockIdx.x + 1) / gridDim.x);
        float bv = -3.402823466e+38f;
        int bi = 0x7fffffff;
        // Two rows per warp and trip, all 16-byte loads of both rows issued before the first use
        // (H <= 2048: at most 8 per lane and row), so that each warp keeps ~8 KB in flight.
        const int nvec = H >> 3;
        for (int v = v0 + warp; v < v1; v += 2 * kPComputeWarps) {
          const int vb = v + kPComputeWarps;
          const bool has_b = vb < v1;
          const uint4* row_a = reinterpret_cast<const uint4*>(p.lm_head + (size_t)v * H);
          const uint4* row_b = reinterpret_cast<const uint4*>(p.lm_head + (size_t)(has_b ? vb : v) * H);
          uint4 pa[8], pb2[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int c = u * 32 + lane;
            pa[u] = c < nvec ? row_a[c] : make_uint4(0, 0, 0, 0);
            pb2[u] = c < nvec ? row_b[c] : make_uint4(0, 0, 0, 0);
          }
          float acc_a = 0.0f, acc_b = 0.0f;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int c = u * 32 + lane;
            if (c < nvec) {
              const __half2* ha = reinterpret_cast<const __half2*>(&pa[u]);
              const __half2* hb = reinterpret_cast<const __half2*>(&pb2[u]);
              const float* xs = work + c * 8;
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) {
                const float2 fa = __half22float2(ha[jj]), fb = __half22float2(hb[jj]);
                acc_a = fmaf(fa.x, xs[2 * jj], acc_a);
                acc_a = fmaf(fa.y, xs[2 * jj + 1], acc_a);
                acc_b = fmaf(fb.x, xs[2 * jj], acc_b);
                acc_b = fmaf(fb.y, xs[2 * jj + 1], acc_b);
              }
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            acc_a += __shfl_xor_sync(0xffffffffu, acc_a, o);
            acc_b += __shfl_xor_sync(0xffffffffu, acc_b, o);
          }
          if (lane == 0) {
            p.logits[v] = acc_a;
            if (has_b) p.logits[vb] = acc_b;
          }
          if (acc_a > bv) {
            bv = acc_a;
            bi = v;
          }
          if (has_b && acc_b > bv) {
            bv = acc_b;
            bi = vb;
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
      stamp(17);
      if (!grid_barrier(p, epoch, s_abort, s_go, tid)) break;
      stamp(18);
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
      stamp(19);
    }
    if (tid == 0) {
      *s_consumed = seq;
      if (p.phase_cycles)
        for (int k = 0; k < kPStamps; ++k) p.phase_cycles[(size_t)blockIdx.x * kPStamps + k] = s_time[k];
    }
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
      c.q_heads * c.head_dim > kPMaxHidden || d->attn_splits > 64 || (c.hidden % 32) || (c.inter % 32) ||
      c.layers > kPMaxLayers || c.q_heads > 32 || sms > 256 ||
      (c.q_heads * c.head_dim + 2 * c.kv_heads * c.head_dim + 2 * c.hidden) / kPanelRows > kPMaxPanels)
    return;
  const void* fn = c.head_dim == 128 ? (const void*)decode_persistent_kernel<128> : (const void*)decode_persistent_kernel<64>;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPSmemBytes) != cudaSuccess) return;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kPThreads, kPSmemBytes) != cudaSuccess || per_sm < 1) return;
  st->nctas = sms;
  const PlanShape shape = plan_shape_of(c);
  if (!build_decode_plan(shape, st->nctas, &st->plan) || check_decode_plan(shape, st->plan) != 0 ||
      st->plan.max_chunks > kPMaxChunks)
    return;

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
            pdev_copy(st, &p.abort_flag, nullptr, 4) &&
            pdev_copy(st, &p.phase_cycles, nullptr, (size_t)st->nctas * kPStamps * 8);
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
  if (!d->profile) prm.phase_cycles = nullptr;
  cudaError_t e = cudaMemsetAsync(prm.bar_counter, 0, 4, d->stream);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(prm.abort_flag, 0, 4, d->stream);
  if (e != cudaSuccess) return e;
  void* args[] = {&prm};
  const void* fn = d->cfg.head_dim == 128 ? (const void*)decode_persistent_kernel<128> : (const void*)decode_persistent_kernel<64>;
  return cudaLaunchCooperativeKernel(fn, dim3(st->nctas), dim3(kPThreads), args, kPSmemBytes, d->stream);
}

// Copies the per-CTA phase cycle counts of the last persistent launch (after synchronizing).
int persistent_phase_cycles(Decoder* d, long long* out, int capacity, int* nctas, int* stamps) {
  if (!persistent_usable(d)) return MLLMB200_UNSUPPORTED;
  PersistentState* st = d->persist;
  if (nctas) *nctas = st->nctas;
  if (stamps) *stamps = kPStamps;
  if (!out) return MLLMB200_OK;
  if (capacity < st->nctas * kPStamps) return MLLMB200_INVALID_ARG;
  if (cudaStreamSynchronize(d->stream) != cudaSuccess) return MLLMB200_CUDA_ERROR;
  if (cudaMemcpy(out, st->prm.phase_cycles, (size_t)st->nctas * kPStamps * 8, cudaMemcpyDeviceToHost) != cudaSuccess)
    return MLLMB200_CUDA_ERROR;
  return MLLMB200_OK;
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
