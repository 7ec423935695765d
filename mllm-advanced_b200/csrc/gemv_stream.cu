// Streaming W4A32 GEMV for decode (M <= 4 activation rows), sm_100a: ONE launch per call.
//
// y[m,n] = lhs_scale[m] * ( sum_b float(sum_{k in b} a_q[m,k] * w[n,k]) * s[n,b]  +  a_off[m] * zsum[n] ) + bias[n]
//
// which equals the reference expression (reference project, tests/Arm/KaiLinearTest.hpp:338-377;
// production call mllm/Backends/Arm/Kernels/kai_linear.cpp:350-398) with the zero-point term
// a_off * sum_k w[n,k] s[n,b] taken out of the integer sum (zsum is precomputed per row at repack).
//
// Shape of the kernel.  At most about one CTA per SM, whatever the matrix size: 8 compute warps and
// one producer warp.  A call holds up to eight matrices, each with its own activations (or several
// sharing theirs: q/k/v, gate/up); every matrix gets a share of the grid's clusters in proportion to
// its size.  Its weight cells (layout.h: [panel of 32 rows][K-group] x 576 bytes) form one sequence; a
// cluster of S CTAs takes a contiguous range of whole panels and cuts its cells into S equal
// contiguous runs, one per CTA (S > 1 only where a matrix has too few panels, or too uneven a
// number of them, to fill the SMs with whole panels; the size is chosen from what the device can
// co-schedule).  A CTA walks its run in bands of two panels (one where the run begins or ends
// inside a panel), each band in blocks of 48 K-groups; one block is one stage of a shared-memory
// ring: one bulk copy of up to 27 KB per panel (cp.async.bulk, a full/empty mbarrier pair per stage,
// the weights marked evict-first in L2 so that they do not displace activations and outputs).
// Compute warp w takes K-groups w, w + 8, ... of the block: it reads the group's activation record
// once and uses it for the cell of either panel (lane = weight row, one 16-byte shared load = the
// row's 32 nibbles, two masks, eight dp4a, one FMA with the group scale).  A small matrix fits
// entirely in the ring, so all of its bytes are requested by the first instructions of the kernel
// (one stage per lane of the producer warp); a large one streams through the ring without
// draining - the producer only ever reads constant weights, so it never waits for the previous
// kernel.
//
// Under programmatic dependent launch the first copies are issued before griddepcontrol.wait, i.e.
// while the previous kernel of the stream still runs; with 288 threads, <= 96 registers and, for runs of
// a few hundred KB, a ring of at most 90 KB, two consecutive launches are resident on an SM together,
// so a call's first stages are in shared memory before its activations exist (long runs get a 180 KB
// ring instead: the head start is worth less there than depth for the stream).  Only what depends on
// x comes after the wait:
//   * the dynamic per-row int8 quantization of x (reference: tests/Arm/KaiLinearTest.hpp:163-230;
//     production call kai_linear.cpp:358-362), done by every CTA for itself into shared memory in
//     the byte order the nibble masks produce (48-byte records, layout.h) - only the K-groups the
//     CTA's run needs, though the row's min/max take the whole row - or, when the caller already
//     holds such records (the decoder's producers write them), a plain copy of those;
//   * the main loop over cells that are long since in shared memory;
//   * the reduction: every warp leaves one partial sum per panel of the CTA's run in shared memory,
//     added in warp order; a panel cut between CTAs of a cluster is finished by the CTA that holds
//     its first cell, the others send their part into its shared memory (DSMEM) and are added in
//     rank order - deterministic.
//
// Measured on B200 (CUDA events, graph replay): the seven linears of a Qwen2-1.5B layer in one launch
// ~8.5 us per layer (26.5 MB), of which ~4 us are the chain's serial part (release of the dependent
// launch ~1.3 us, quantization of x 1.3-2.4 us, epilogue 0.5 us); the 28672 x 8192 matrix ~27 us
// (132 MB).  With its cells resident in shared memory the main loop takes ~16 SM cycles per cell for
// single panels and ~12 for panel pairs (8 warps; shared-memory wavefronts + integer pipe); HBM
// delivers a cell per ~25 cycles per SM.
#include <algorithm>
#include <vector>

#include "device_common.cuh"

namespace mllmb200 {

constexpr int kGsCWarps = 8;                  // compute warps
constexpr int kGsCThreads = kGsCWarps * 32;   // 256
constexpr int kGsThreads = kGsCThreads + 32;  // + the producer warp
constexpr int kGsMaxProblems = 8;
constexpr int kGsMaxPeers = 7;
constexpr int kGsMaxM = 4;
constexpr int kGsMaxSlots = 16;       // (panels of a CTA's run) x (activation rows, padded) kept per warp
constexpr int kGsMaxStages = 16;      // ring stages
constexpr int kGsMaxCluster = 8;
#ifndef MLLMB200_GS_ITEMS
#define MLLMB200_GS_ITEMS 5
#endif
constexpr int kGsItemsPerThread = MLLMB200_GS_ITEMS;  // 8-value items of x a thread keeps in registers between the two passes
constexpr size_t kGsSmemBudget = 200 * 1024;
#ifndef MLLMB200_GS_BLOCK_GROUPS
#define MLLMB200_GS_BLOCK_GROUPS 48
#endif
constexpr int kGsBlockGroups = MLLMB200_GS_BLOCK_GROUPS;      // K-groups of a panel per ring stage (a multiple of 16)
#ifndef MLLMB200_GS_MIN_CTAS
#define MLLMB200_GS_MIN_CTAS 2
#endif
#ifndef MLLMB200_GS_RING_KB
#define MLLMB200_GS_RING_KB 90
#endif
#ifndef MLLMB200_GS_RING_LONG_KB
#define MLLMB200_GS_RING_LONG_KB 180
#endif
// Ring of a run too long to be in flight all at once.  Runs of a few hundred KB get the small ring: two CTAs
// then fit on an SM, so the next launch of a chain moves in beside the running one and has its first stages
// in shared memory by the time its activations are ready.  For long runs that head start is worth less than
// a deep ring for the stream itself.
constexpr long long kGsRingBytes = MLLMB200_GS_RING_KB * 1024LL;
constexpr long long kGsRingBytesLong = MLLMB200_GS_RING_LONG_KB * 1024LL;
constexpr long long kGsLongRunBytes = 400 * 1024LL;
constexpr int kGsBandBytes = kGsBlockGroups * kCellBytes;     // 27648: one panel's share of a stage

// How a CTA walks its run of cells [cb, ce) (cells of the cluster, [panel][K-group] order): in bands of one
// or two whole-or-partial panels, each band in blocks of kGsBlockGroups K-groups.  One block of a band is one ring stage
// (one bulk copy per panel of the band); two panels in a band let a warp use the activation record of a
// K-group for two cells.  The producer, the compute warps and the host-side plan check all run this code.
struct GsWalk {
  int G, ce, rmax;
  int c;      // first cell of the run not yet assigned to a band
  int panel;  // first panel of the current band (relative to the cluster's first panel)
  int R;      // panels of the current band (0 before the first)
  int g_end, g_next;
  int g0, cnt;  // current stage: first K-group and number of K-groups (<= kGsBlockGroups)
  bool band_end;
  __host__ __device__ void init(int cb, int ce_, int G_, int rmax_) {
    G = G_;
    ce = ce_;
    rmax = rmax_;
    c = cb;
    panel = cb / G_;
    R = 0;
    g_end = g_next = g0 = cnt = 0;
    band_end = false;
  }
  __host__ __device__ bool next() {
    if (g_next >= g_end) {  // open the next band
      if (c >= ce) return false;
      panel += R;
      const int g_begin = c - panel * G;
      const int remaining = ce - c;
      if (g_begin == 0 && rmax >= 2 && remaining >= 2 * G) {
        R = 2;
        g_end = G;
        c += 2 * G;
      } else {
        R = 1;
        g_end = g_begin + remaining < G ? g_begin + remaining : G;
        c += g_end - g_begin;
      }
      g_next = g_begin;
    }
    g0 = g_next;
    cnt = g_end - g0 < kGsBlockGroups ? g_end - g0 : kGsBlockGroups;
    g_next += cnt;
    band_end = g_next >= g_end;
    return true;
  }
};
constexpr int kGsTraceStamps = 10;

// Optional trace (see w4a32_gemv_stream_set_trace): per launch kGsTraceStamps %globaltimer values of
// thread 0 of CTA 0 and as many of thread 0 of the last CTA.
__device__ unsigned long long* g_gs_trace = nullptr;
__device__ int g_gs_trace_capacity = 0;

struct GsProblem {
  const float* x;        // fp32 [m, ldx], or nullptr when records are given
  const uint8_t* a_rec;  // [m][num_groups] 48-byte records (x == nullptr)
  const float2* a_hdr;   // [m] {lhs_scale, a_off bits}    (x == nullptr)
  const uint8_t* tiled;  // TiledHeader at offset 0
  float* y;
  int ldx, ldy, n, k;
  int num_groups, num_panels;
  int cl_begin, clusters;     // clusters [cl_begin, cl_begin + clusters) of the grid work on this matrix
  size_t zsum_off, bias_off;  // byte offsets of the per-row arrays inside the tiled buffer
  // tensor parallelism: the same element is also stored at y_peer[i][m * ldy + n] for i < num_peers - the output
  // buffers of the other GPUs, mapped into this process (plain stores over NVLink)
  int num_peers;
  float* y_peer[kGsMaxPeers];
};

struct GsParams {
  int m, cluster_size;
  int rmax, stages;  // panels per band (1 or 2: a ring stage is rmax * kGsBandBytes bytes), ring stages
  int np_max;       // panels a CTA's run may touch (np_max * M_MAX <= kGsMaxSlots)
  int g_max;        // largest num_groups of the call (sizes the record buffer)
  int use_pdl, num_problems, trace;
  GsProblem prob[kGsMaxProblems];
};

// shared memory carve-up (dynamic, 128-byte aligned base)
struct GsSmem {
  size_t full, empty, rowc, scratch, flags, abuf, red, cred, ring, total;
};
__host__ __device__ inline GsSmem gs_smem_layout(int m_max, int g_max, int cluster_size, int rmax, int stages, int np_max) {
  GsSmem s;
  size_t off = 0;
  s.full = off;  // one mbarrier per stage: bytes landed
  off += (size_t)kGsMaxStages * 8;
  s.empty = off;  // one mbarrier per stage: the compute warps are done with it
  off += (size_t)kGsMaxStages * 8;
  s.rowc = off;  // per activation row {lhs_scale, a_off}
  off += (size_t)kGsMaxM * 8;
  s.scratch = off;  // min/max exchange: 2 * 8 floats per activation row
  off += (size_t)kGsMaxM * 2 * kGsCWarps * 4;
  s.flags = off;  // [0] = a bounded wait ran out somewhere in this CTA
  off += 16;
  off = (off + 15) & ~size_t(15);
  s.abuf = off;  // quantized activation records [m][group] x 48 bytes
  off += (size_t)m_max * g_max * kActRecordBytes;
  s.red = off;  // [warp][panel of the run][m][32] floats
  off += (size_t)kGsCWarps * np_max * m_max * 32 * 4;
  s.cred = off;  // [cluster rank][m][32] floats (parts of a panel received from other CTAs)
  off += cluster_size > 1 ? (size_t)cluster_size * m_max * 32 * 4 : 0;
  off = (off + 127) & ~size_t(127);
  s.ring = off;  // [stage][panel of the band][16 cells]
  off += (size_t)stages * rmax * kGsBandBytes;
  s.total = off + 128;  // slack for the base alignment
  return s;
}

__device__ __forceinline__ int dp4a_s8_u8(int a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// bytes {sat8(v0), sat8(v1), sat8(v2), sat8(v3)} from low to high: two packing conversions with signed saturation
__device__ __forceinline__ uint32_t pack_sat_s8x4(int v0, int v1, int v2, int v3) {
  uint32_t t, d;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(t) : "r"(v3), "r"(v2));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(v1), "r"(v0), "r"(t));
  return d;
}
__device__ __forceinline__ float warp_min_f32(float v) {
  float r;
  asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float warp_max_f32(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Shared-memory accesses by 32-bit shared-space address (the ring is carved out of dynamic shared memory
// through integer arithmetic, which hides the address space from the compiler).
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
  uint32_t v;
  asm volatile("{\n\t.reg .u16 t;\n\tld.shared.u16 t, [%1];\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }
// barrier 1: the compute warps only (the producer warp is busy streaming)
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kGsCThreads) : "memory"); }

template <int M_MAX>
__global__ void __launch_bounds__(kGsThreads, MLLMB200_GS_MIN_CTAS) w4a32_gemv_stream_kernel(const __grid_constant__ GsParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  // the next kernels of the stream may become resident and start fetching their own (constant) weights
  if (p.use_pdl) pdl_launch_dependents();

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // trace: thread 0 of the first and of the last CTA stamp the global timer at the phase boundaries
  unsigned long long* trace = nullptr;
  if (p.trace > 0 && tid == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1) && g_gs_trace != nullptr &&
      p.trace <= g_gs_trace_capacity)
    trace = g_gs_trace + 1 + (size_t)(p.trace - 1) * (2 * kGsTraceStamps) + (blockIdx.x == 0 ? 0 : kGsTraceStamps);
  auto stamp = [&](int i) {
    if (trace != nullptr) trace[i] = global_timer_ns();
  };
  stamp(0);

  const int S = p.cluster_size;
  const GsSmem Lo = gs_smem_layout(M_MAX, p.g_max, S, p.rmax, p.stages, p.np_max);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Lo.full);
  uint64_t* empty = reinterpret_cast<uint64_t*>(smem + Lo.empty);
  float2* rowc = reinterpret_cast<float2*>(smem + Lo.rowc);
  float* scratch = reinterpret_cast<float*>(smem + Lo.scratch);
  volatile int* flags = reinterpret_cast<volatile int*>(smem + Lo.flags);
  uint8_t* abuf = smem + Lo.abuf;
  float* red = reinterpret_cast<float*>(smem + Lo.red);
  float* cred = reinterpret_cast<float*>(smem + Lo.cred);
  uint8_t* ring = smem + Lo.ring;

  const uint32_t rank = S > 1 ? cluster_ctarank() : 0u;
  const int cluster = (int)blockIdx.x / S;
  // Peers write into each other's shared memory at the end; they may only do so once the target
  // runs.  Arrive now, wait just before the remote stores: the barrier latency hides behind the work.
  if (S > 1) cluster_arrive_relaxed();

  // ---- which matrix, and which of its cells, are ours:
  // cluster -> matrix pi and whole panels [p0, p1) of it = T cells; CTA of rank r -> cells [r T / S, (r+1) T / S)
  int pi = 0;
#pragma unroll
  for (int i = 1; i < kGsMaxProblems; ++i)
    if (i < p.num_problems && cluster >= p.prob[i].cl_begin) pi = i;
  const GsProblem& pr = p.prob[pi];
  const int G = pr.num_groups;
  const uint32_t q = (uint32_t)(cluster - pr.cl_begin);
  const int p0 = (int)((q * (uint32_t)pr.num_panels) / (uint32_t)pr.clusters);  // < 2^31 by the plan
  const int p1 = (int)(((q + 1) * (uint32_t)pr.num_panels) / (uint32_t)pr.clusters);
  const uint32_t T = (uint32_t)(p1 - p0) * (uint32_t)G;
  auto cta_begin = [&](uint32_t r) { return S > 1 ? (int)((r * T) / (uint32_t)S) : (int)(r * T); };  // first cell of rank r's run
  const int cb = cta_begin(rank), ce = cta_begin(rank + 1);
  const int Lc = ce - cb;
  const int pa = cb / G;                                  // first panel the run touches (relative to p0)
  const int np_run = Lc > 0 ? (ce - 1) / G - pa + 1 : 0;  // panels the run touches (<= np_max by the plan)
  const int np_cta = np_run <= p.np_max ? np_run : 0;
  // A run of a single panel never pairs panels: it cuts the ring into twice as many stages of half the size.
  const int rmax_cta = (p.rmax == 2 && np_run >= 2) ? 2 : 1;
  const int NS = min(kGsMaxStages, p.stages * p.rmax / rmax_cta);
  const int stage_bytes = rmax_cta * kGsBandBytes;

  // ---- tile header: checked before a single byte of the matrix is requested
  bool hdr_ok, f16;
  {
    uint32_t okbits = 0;
    if (lane == 0) {
      const uint4 h = *reinterpret_cast<const uint4*>(pr.tiled);  // magic, version, n, k
      const bool good = h.x == kTiledMagic && h.z == (uint32_t)pr.n && h.w == (uint32_t)pr.k;
      okbits = (good ? 1u : 0u) | (reinterpret_cast<const TiledHeader*>(pr.tiled)->scale_mode == 2u ? 2u : 0u);
    }
    okbits = __shfl_sync(0xffffffffu, okbits, 0);
    hdr_ok = (okbits & 1u) != 0u;
    f16 = (okbits & 2u) != 0u;
    if (!hdr_ok && tid == 0) atomicOr(&g_device_status, kDevStatusBadHeader);
  }
  hdr_ok = hdr_ok && np_run <= p.np_max && G <= p.g_max;  // cannot fail with a plan from gs_make_plan
  if (tid == 0) flags[0] = 0;

  if (warp == kGsCWarps) {
    // =============================== producer warp ===============================
    // a stage = one block of <= kGsBlockGroups K-groups of a band: one contiguous copy per panel of the band
    const uint8_t* cells_src = pr.tiled + sizeof(TiledHeader) + (size_t)p0 * G * kCellBytes;  // first cell of the cluster
    const uint64_t stream_once = l2_policy_evict_first();
    auto issue_stage = [&](const GsWalk& w, int st) {  // one thread
      const uint32_t bytes = (uint32_t)(w.cnt * kCellBytes);
      mbar_arrive_expect_tx(&full[st], bytes * (uint32_t)w.R);
      for (int r = 0; r < w.R; ++r)
#ifdef MLLMB200_GS_NO_HINT
        bulk_g2s(ring + (size_t)st * stage_bytes + (size_t)r * kGsBandBytes,
                      cells_src + ((size_t)(w.panel + r) * G + w.g0) * kCellBytes, bytes, &full[st]);
#else
        bulk_g2s_hint(ring + (size_t)st * stage_bytes + (size_t)r * kGsBandBytes,
                      cells_src + ((size_t)(w.panel + r) * G + w.g0) * kCellBytes, bytes, &full[st], stream_once);
#endif
    };
    if (lane < NS) {
      mbar_init(&full[lane], 1);
      mbar_init(&empty[lane], kGsCWarps);
    }
    mbar_fence_init();
    __syncwarp();
    GsWalk walk;
    walk.init(cb, hdr_ok ? ce : cb, G, rmax_cta);
    {
      // the first lap: lane i walks to stage i and requests it
      bool have = false;
      for (int i = 0; i <= lane && lane < NS; ++i) {
        have = walk.next();
        if (!have) break;
      }
      if (have && lane < NS) issue_stage(walk, lane);
    }
    __syncthreads();  // (A) barriers initialised; pairs with the compute warps' sync after the quantization
    if (lane == 0) {
      // lane 0 has walked one stage; catch up to the end of the first lap, then refill stages as they are released
      bool have = true;
      for (int i = 1; i < NS && have; ++i) have = walk.next();
      int st = 0;
      uint32_t ph = 0;
      while (have && walk.next()) {
        if (!mbar_wait_bounded(&empty[st], ph)) {  // the compute warps have left the stage
          flags[0] = 1;
          break;
        }
        issue_stage(walk, st);
        if (++st == NS) {
          st = 0;
          ph ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // =============================== compute warps ===============================
    // epilogue constants (zsum, bias) requested now, used at the very end.
    // Pair t = (panel pa + t / m, activation row t % m); warp w finishes t = w, w + 8, ...
    const int npairs = np_cta * p.m;
    const float* zsum = reinterpret_cast<const float*>(pr.tiled + pr.zsum_off);
    const float* bias = reinterpret_cast<const float*>(pr.tiled + pr.bias_off);
    float zs0 = 0.0f, bs0 = 0.0f;
    if (warp < npairs && hdr_ok) {
      const int n_pad = (p0 + pa + warp / p.m) * kPanelRows + lane;  // always inside the padded per-row arrays
      zs0 = zsum[n_pad];
      bs0 = bias[n_pad];
    }
    // K-groups whose records this CTA will read: all of them, unless the run stays inside one panel
    const int g_lo = np_run == 1 ? cb - pa * G : 0;
    const int g_hi = np_run == 1 ? ce - 1 - pa * G : G - 1;
    stamp(1);
    // the weights are constant; the activations may come from the kernel before us
    if (p.use_pdl) pdl_wait_prior();
    stamp(2);

    // ---- activations -> 48-byte records in shared memory
    if (pr.x != nullptr) {
      const int num_items = G * 4;                    // item = 8 consecutive k
      const int first_item = g_lo * 4;                // items are walked from here, wrapping around
      const int needed = (g_hi - g_lo + 1) * 4;       // ... and only this many of them are quantized
      const int k = pr.k;
      for (int m = 0; m < p.m; ++m) {
        const float* row = pr.x + (size_t)m * pr.ldx;
        const bool vec = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
        float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
        // Item j (counted from first_item) -> v8 and the running min/max.  The common case (a whole item of
        // an aligned row) is split in two steps so that a thread has all its loads in flight before it uses
        // the first of them: one round trip to memory per row instead of one per item.
        auto item_k0 = [&](int j) {
          int item = first_item + j;
          if (item >= num_items) item -= num_items;
          return item * 8;
        };
        auto fold = [&](const float (&v8)[8]) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            mn = fminf(mn, v8[e]);
            mx = fmaxf(mx, v8[e]);
          }
        };
        auto load_ragged = [&](int k0, float (&v8)[8]) {  // an item cut by the end of the row, or an unaligned row
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const bool in = k0 + e < k;
            v8[e] = in ? row[k0 + e] : 0.0f;
            if (in) {
              mn = fminf(mn, v8[e]);
              mx = fmaxf(mx, v8[e]);
            }
          }
        };
        auto load_whole = [&](int j, bool& is_whole, float (&v8)[8]) {
          const int k0 = item_k0(j);
          is_whole = vec && j < num_items && k0 + 8 <= k;
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
          if (is_whole) {
            a = *reinterpret_cast<const float4*>(row + k0);
            b = *reinterpret_cast<const float4*>(row + k0 + 4);
          }
          v8[0] = a.x; v8[1] = a.y; v8[2] = a.z; v8[3] = a.w;
          v8[4] = b.x; v8[5] = b.y; v8[6] = b.z; v8[7] = b.w;
        };
        float v[kGsItemsPerThread][8];
        bool whole[kGsItemsPerThread];
#pragma unroll
        for (int it = 0; it < kGsItemsPerThread; ++it) load_whole(tid + it * kGsCThreads, whole[it], v[it]);
#pragma unroll
        for (int it = 0; it < kGsItemsPerThread; ++it) {
          const int j = tid + it * kGsCThreads;
          if (whole[it]) fold(v[it]);
          else if (j < num_items && item_k0(j) < k) load_ragged(item_k0(j), v[it]);
        }
        // the rest of a very long row only feeds the min/max here, and is read again when it is packed
        for (int j = kGsItemsPerThread * kGsCThreads + tid; j < num_items; j += kGsCThreads) {
          float t0[8];
          if (item_k0(j) < k) load_ragged(item_k0(j), t0);
        }
        mn = warp_min_f32(mn);
        mx = warp_max_f32(mx);
        if (lane == 0) {
          scratch[(m * 2 + 0) * kGsCWarps + warp] = mn;
          scratch[(m * 2 + 1) * kGsCWarps + warp] = mx;
        }
        compute_sync();
        mn = warp_min_f32(scratch[(m * 2 + 0) * kGsCWarps + (lane & (kGsCWarps - 1))]);
        mx = warp_max_f32(scratch[(m * 2 + 1) * kGsCWarps + (lane & (kGsCWarps - 1))]);
        const ActQuantParams qp = act_quant_params(mn, mx);
        if (tid == 0) rowc[m] = make_float2(qp.recip_scale, (float)(-qp.nzp));
        uint32_t* out = reinterpret_cast<uint32_t*>(abuf + (size_t)m * G * kActRecordBytes);
        // Packs item j into its record.  Called by every thread of a warp together (the shuffles need full
        // warps); the four items of a K-group sit in four neighbouring lanes.
        auto emit = [&](int j, bool from_regs, const float (&v8)[8]) {
          int item = first_item + j;
          if (item >= num_items) item -= num_items;
          const bool valid = j < needed;
          const int k0 = item * 8;
          int q8[8];  // round_half_away(x * scale0) + nzp, not yet clamped (0 outside the row)
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const bool in = valid && k0 + e < k;
            const float xv = from_regs ? v8[e] : (in ? row[k0 + e] : 0.0f);
            q8[e] = in ? (int)roundf(__fmul_rn(xv, qp.scale0)) + qp.nzp : 0;
          }
          // clamp to int8 and pack in one step: even k into the low word, odd k into the high word
          const uint32_t lo = pack_sat_s8x4(q8[0], q8[2], q8[4], q8[6]);
          const uint32_t hi = pack_sat_s8x4(q8[1], q8[3], q8[5], q8[7]);
          int s = __dp4a((int)lo, 0x01010101, __dp4a((int)hi, 0x01010101, 0));  // sum of the eight clamped values
          s += __shfl_xor_sync(0xffffffffu, s, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          if (valid) {
            uint32_t* rec = out + (size_t)(item >> 2) * (kActRecordBytes / 4);
            rec[item & 3] = lo;
            rec[4 + (item & 3)] = hi;
            if ((item & 3) == 0) rec[8] = (uint32_t)(-8 * s);  // nibbles are q+8
          }
        };
#pragma unroll
        for (int it = 0; it < kGsItemsPerThread; ++it) {
          if (it * kGsCThreads >= needed) break;  // uniform over the compute warps
          emit(tid + it * kGsCThreads, true, v[it]);
        }
        for (int base = kGsItemsPerThread * kGsCThreads; base < needed; base += kGsCThreads) {  // uniform trip count
          float none[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          emit(base + tid, false, none);
        }
      }
    } else {
      const int words = p.m * G * (kActRecordBytes / 16);
      const uint4* src = reinterpret_cast<const uint4*>(pr.a_rec);
      uint4* dst = reinterpret_cast<uint4*>(abuf);
      for (int i = tid; i < words; i += kGsCThreads) dst[i] = src[i];
      if (tid < p.m) {
        const float2 h = pr.a_hdr[tid];
        rowc[tid] = make_float2(h.x, (float)__float_as_int(h.y));
      }
    }
    __syncthreads();  // (A) records and row constants visible to every warp; mbarriers initialised
    stamp(3);

    // ---- main loop.  Of the K-groups of a stage warp w takes groups w, w + 8, w + 16, ..., each for every panel
    // of the band.  The weights of the next stage are requested before the arithmetic of the current one.
    constexpr int RM = 2;  // panels per band the registers are laid out for
    float acc[RM][M_MAX];
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
      for (int m = 0; m < M_MAX; ++m) acc[r][m] = 0.0f;
    bool ok = true;
    const uint32_t abuf_s = smem_u32(abuf);
    const uint32_t row_stride = (uint32_t)G * kActRecordBytes;  // records of the next activation row
    const uint32_t red_s = smem_u32(red) + ((uint32_t)warp * p.np_max * M_MAX * 32 + lane) * 4;  // slot 0, row 0 of this lane
    long long wait_cycles = 0;  // trace only: time thread 0 spent waiting for stages to land
    // one cell: the lane's 32 nibbles and its group scale against the group's activation record(s)
    auto compute = [&](const uint4 wq, const uint32_t sraw, uint32_t rec, float (&a)[M_MAX]) {
      const float s = f16 ? __half2float(__ushort_as_half((unsigned short)sraw)) : __uint_as_float(sraw << 16);
      // low half-bytes as they are (0..15), high half-bytes left in place (16 * (0..15), exact >> 4 at the end)
      const uint32_t lo0 = wq.x & 0x0F0F0F0Fu, hi0 = wq.x & 0xF0F0F0F0u;
      const uint32_t lo1 = wq.y & 0x0F0F0F0Fu, hi1 = wq.y & 0xF0F0F0F0u;
      const uint32_t lo2 = wq.z & 0x0F0F0F0Fu, hi2 = wq.z & 0xF0F0F0F0u;
      const uint32_t lo3 = wq.w & 0x0F0F0F0Fu, hi3 = wq.w & 0xF0F0F0F0u;
#pragma unroll
      for (int m = 0; m < M_MAX; ++m) {
        if (M_MAX == 1 || m < p.m) {
          const uint4 alo = lds128(rec);
          const uint4 ahi = lds128(rec + 16);
          int ia = (int)lds32(rec + 32);  // -8 * sum(a_q)
          int ib = 0;
          ia = dp4a_s8_u8((int)alo.x, lo0, ia);
          ib = dp4a_s8_u8((int)ahi.x, hi0, ib);
          ia = dp4a_s8_u8((int)alo.y, lo1, ia);
          ib = dp4a_s8_u8((int)ahi.y, hi1, ib);
          ia = dp4a_s8_u8((int)alo.z, lo2, ia);
          ib = dp4a_s8_u8((int)ahi.z, hi2, ib);
          ia = dp4a_s8_u8((int)alo.w, lo3, ia);
          ib = dp4a_s8_u8((int)ahi.w, hi3, ib);
          a[m] = fmaf((float)(ia + (ib >> 4)), s, a[m]);
        }
        rec += row_stride;
      }
    };
    // the same cell pair with ONE pass over the activation record (M = 1: the record is read into registers once)
    auto compute2 = [&](const uint4 w0, const uint32_t s0raw, const uint4 w1, const uint32_t s1raw, uint32_t rec) {
      const float s0 = f16 ? __half2float(__ushort_as_half((unsigned short)s0raw)) : __uint_as_float(s0raw << 16);
      const float s1 = f16 ? __half2float(__ushort_as_half((unsigned short)s1raw)) : __uint_as_float(s1raw << 16);
#pragma unroll
      for (int m = 0; m < M_MAX; ++m) {
        if (M_MAX == 1 || m < p.m) {
          const uint4 alo = lds128(rec);
          const uint4 ahi = lds128(rec + 16);
          const int a8 = (int)lds32(rec + 32);  // -8 * sum(a_q)
          int ia = a8, ib = 0, ja = a8, jb = 0;
          ia = dp4a_s8_u8((int)alo.x, w0.x & 0x0F0F0F0Fu, ia);
          ib = dp4a_s8_u8((int)ahi.x, w0.x & 0xF0F0F0F0u, ib);
          ja = dp4a_s8_u8((int)alo.x, w1.x & 0x0F0F0F0Fu, ja);
          jb = dp4a_s8_u8((int)ahi.x, w1.x & 0xF0F0F0F0u, jb);
          ia = dp4a_s8_u8((int)alo.y, w0.y & 0x0F0F0F0Fu, ia);
          ib = dp4a_s8_u8((int)ahi.y, w0.y & 0xF0F0F0F0u, ib);
          ja = dp4a_s8_u8((int)alo.y, w1.y & 0x0F0F0F0Fu, ja);
          jb = dp4a_s8_u8((int)ahi.y, w1.y & 0xF0F0F0F0u, jb);
          ia = dp4a_s8_u8((int)alo.z, w0.z & 0x0F0F0F0Fu, ia);
          ib = dp4a_s8_u8((int)ahi.z, w0.z & 0xF0F0F0F0u, ib);
          ja = dp4a_s8_u8((int)alo.z, w1.z & 0x0F0F0F0Fu, ja);
          jb = dp4a_s8_u8((int)ahi.z, w1.z & 0xF0F0F0F0u, jb);
          ia = dp4a_s8_u8((int)alo.w, w0.w & 0x0F0F0F0Fu, ia);
          ib = dp4a_s8_u8((int)ahi.w, w0.w & 0xF0F0F0F0u, ib);
          ja = dp4a_s8_u8((int)alo.w, w1.w & 0x0F0F0F0Fu, ja);
          jb = dp4a_s8_u8((int)ahi.w, w1.w & 0xF0F0F0F0u, jb);
          acc[0][m] = fmaf((float)(ia + (ib >> 4)), s0, acc[0][m]);
          acc[1][m] = fmaf((float)(ja + (jb >> 4)), s1, acc[1][m]);
        }
        rec += row_stride;
      }
    };
    const uint32_t lane_off = (uint32_t)warp * kCellBytes + lane * 16;  // this lane's row in cell `warp` of a band block
    const uint32_t scale_off = kCellNibbleBytes - lane * 14;            // from the lane's nibble row to its scale
    const uint32_t ring_s = smem_u32(ring);
    int st = 0;
    uint32_t ph = 0;
    GsWalk cur;
    cur.init(cb, hdr_ok ? ce : cb, G, rmax_cta);
    while (cur.next()) {
      const long long tw0 = trace != nullptr ? clock64() : 0;
      if (!mbar_wait_bounded(&full[st], ph)) {
        ok = false;
        break;
      }
      if (trace != nullptr) wait_cycles += clock64() - tw0;
      for (int h = 0; h < kGsBlockGroups; h += 2 * kGsCWarps) {  // 16 K-groups at a time: two per warp
        if (h >= cur.cnt) break;
        const uint32_t base = ring_s + (uint32_t)st * stage_bytes + lane_off + (uint32_t)h * kCellBytes;
        const uint32_t rec = abuf_s + (uint32_t)(cur.g0 + h + warp) * kActRecordBytes;
        const bool has_a = h + warp < cur.cnt, has_b = h + warp + kGsCWarps < cur.cnt;
        if (cur.R == 2) {
          // requests for all four cells first, then the arithmetic
          uint4 wa0 = make_uint4(0, 0, 0, 0), wa1 = wa0, wb0 = wa0, wb1 = wa0;
          uint32_t sa0 = 0, sa1 = 0, sb0 = 0, sb1 = 0;
          if (has_a) {
            wa0 = lds128(base);
            sa0 = lds16(base + scale_off);
            wa1 = lds128(base + kGsBandBytes);
            sa1 = lds16(base + kGsBandBytes + scale_off);
          }
          if (has_b) {
            wb0 = lds128(base + kGsCWarps * kCellBytes);
            sb0 = lds16(base + kGsCWarps * kCellBytes + scale_off);
            wb1 = lds128(base + kGsCWarps * kCellBytes + kGsBandBytes);
            sb1 = lds16(base + kGsCWarps * kCellBytes + kGsBandBytes + scale_off);
          }
          if (has_a) compute2(wa0, sa0, wa1, sa1, rec);
          if (has_b) compute2(wb0, sb0, wb1, sb1, rec + kGsCWarps * kActRecordBytes);
        } else {
          uint4 wa0 = make_uint4(0, 0, 0, 0), wb0 = wa0;
          uint32_t sa0 = 0, sb0 = 0;
          if (has_a) {
            wa0 = lds128(base);
            sa0 = lds16(base + scale_off);
          }
          if (has_b) {
            wb0 = lds128(base + kGsCWarps * kCellBytes);
            sb0 = lds16(base + kGsCWarps * kCellBytes + scale_off);
          }
          if (has_a) compute(wa0, sa0, rec, acc[0]);
          if (has_b) compute(wb0, sb0, rec + kGsCWarps * kActRecordBytes, acc[0]);
        }
      }
      __syncwarp();  // every lane is done reading the stage
      if (lane == 0) mbar_arrive(&empty[st]);
      if (++st == NS) {
        st = 0;
        ph ^= 1u;
      }
      if (cur.band_end) {  // the band's panels are finished for this warp: park the accumulators
        const int slot0 = cur.panel - pa;
#pragma unroll
        for (int r = 0; r < RM; ++r) {
          if (r < cur.R) {
#pragma unroll
            for (int m = 0; m < M_MAX; ++m) {
              sts_f32(red_s + (uint32_t)(((slot0 + r) * M_MAX + m) * 128), acc[r][m]);
              acc[r][m] = 0.0f;
            }
          }
        }
      }
    }
    if (!__all_sync(0xffffffffu, ok) && lane == 0) flags[0] = 1;
    stamp(4);
    if (trace != nullptr) trace[8] = (unsigned long long)wait_cycles;
    compute_sync();  // partial sums visible; one verdict per CTA
    const bool all_ok = hdr_ok && flags[0] == 0;
    stamp(5);

    // ---- reduction + epilogue
    if (S > 1) cluster_wait();  // every CTA of the cluster has started (pairs with the arrive at the top)
    stamp(6);
    const bool own_first = cb == pa * G;  // our first panel starts with us; all later ones always do
    float keep = 0.0f;                    // our part of a last panel that continues in the next CTAs
    int keep_t = -1;
    auto finish = [&](int t, int jp, int m, float part) {
      const int n_pad = (p0 + pa + jp) * kPanelRows + lane;
      const float zs = t == warp ? zs0 : zsum[n_pad];
      const float bs = t == warp ? bs0 : bias[n_pad];
      if (n_pad < pr.n) {
        const float2 rc = rowc[m];
        float v = fmaf(rc.y, zs, part);
        v = fmaf(v, rc.x, bs);
        v = clamp_flt_max(v);
        const size_t at = (size_t)m * pr.ldy + n_pad;
        pr.y[at] = v;
        for (int i = 0; i < pr.num_peers; ++i) pr.y_peer[i][at] = v;
      }
    };
    for (int t = warp; t < npairs; t += kGsCWarps) {
      const int jp = t / p.m, m = t - jp * p.m;  // panel pa + jp of the cluster, activation row m
      const int c_lo = (pa + jp) * G, c_hi = c_lo + G;
      float part = 0.0f;
#pragma unroll
      for (int w = 0; w < kGsCWarps; ++w) part += red[((w * p.np_max + jp) * M_MAX + m) * 32 + lane];
      const bool complete = cb <= c_lo && ce >= c_hi;
      if (jp == 0 && !own_first) {
        // the panel began in an earlier CTA: the one that holds its first cell finishes it
        uint32_t owner = 0;
        for (uint32_t r = 1; r < rank; ++r)
          if (cta_begin(r) <= c_lo && cta_begin(r + 1) > c_lo) owner = r;
        st_cluster_f32(map_to_cta(&cred[((int)rank * M_MAX + m) * 32 + lane], owner), part);
      } else if (!complete) {
        keep = part;
        keep_t = t;
      } else if (all_ok) {
        finish(t, jp, m, part);
      }
    }
    if (S > 1) {
      cluster_sync_all();  // remote parts have landed (release/acquire)
      if (keep_t >= 0 && all_ok) {
        const int t = keep_t;
        const int jp = t / p.m, m = t - jp * p.m;
        const int c_hi = (pa + jp + 1) * G;
        float part = keep;
        for (uint32_t r = rank + 1; r < (uint32_t)S; ++r)  // the following CTAs that hold cells of this panel, in rank order
          if (cta_begin(r) < c_hi && cta_begin(r + 1) > cta_begin(r)) part += cred[((int)r * M_MAX + m) * 32 + lane];
        finish(t, jp, m, part);
      }
    }
    stamp(7);
    return;
  }
  // producer warp: the cluster-wide barriers count every thread of every CTA
  if (S > 1) {
    cluster_wait();
    cluster_sync_all();
  }
}

// ---- host side ---------------------------------------------------------------------------------
struct GsPlan {
  int cluster_size, rmax, stages, np_max, g_max, total_clusters;
  int cl_begin[kGsMaxProblems], clusters[kGsMaxProblems];
  size_t smem;
};

// Sets the kernel's shared-memory attributes once per device (per M_MAX instantiation).
template <int M_MAX>
static cudaError_t gs_configure() {
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && configured[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(w4a32_gemv_stream_kernel<M_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGsSmemBudget);
  if (e != cudaSuccess) return e;
  // always the largest shared-memory configuration: consecutive launches with different ring sizes then
  // never make an SM drain to change its L1 / shared-memory split, which would undo the overlap
  e = cudaFuncSetAttribute(w4a32_gemv_stream_kernel<M_MAX>, cudaFuncAttributePreferredSharedMemoryCarveout,
                           (int)cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64) configured[dev] = true;
  return cudaSuccess;
}

// How many clusters of `s` CTAs (one CTA per SM) the current device runs at once: clusters are placed
// inside a GPC, so sizes that do not divide a GPC's SM count leave SMs idle, and a grid with more clusters
// than this runs in waves.  Asked from the driver once per device and size; 148 / s when it cannot be asked
// (no device: host-only plan checks).
static int gs_cluster_capacity(int s) {
  static int cache[64][kGsMaxCluster + 1] = {};
  if (s <= 1) return 148;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return 148 / s;
  }
  if (cache[dev][s] == 0) {
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(s * 148), 1, 1);
    cfg.blockDim = dim3(kGsThreads, 1, 1);
    cfg.dynamicSmemBytes = 120 * 1024;  // more than half of an SM: one CTA per SM
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)s;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (gs_configure<1>() != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, w4a32_gemv_stream_kernel<1>, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = 148 / s;
    }
    cache[dev][s] = n;
  }
  return cache[dev][s];
}

// groups[i], panels[i]: K-groups and 32-row panels of matrix i.
static bool gs_make_plan(int m_max, int count, const int* groups, const int* panels, GsPlan* plan) {
  if (count < 1 || count > kGsMaxProblems) return false;
  long long total_cells = 0;
  int g_max = 0;
  for (int i = 0; i < count; ++i) {
    total_cells += (long long)groups[i] * panels[i];
    g_max = std::max(g_max, groups[i]);
  }
  (void)total_cells;
  const int sms = 148;  // one CTA per SM and launch: the second slot of an SM belongs to the next launch of a chain
  // Clusters of matrix i for a given cluster size and budget: every matrix gets one, then the matrix whose
  // busiest CTA has the most cells gets the next, until the budget is spent or nobody can use more.
  auto allocate = [&](int s, int budget, int* c) {
    for (int i = 0; i < count; ++i) c[i] = 1;
    int used = count;
#ifndef MLLMB200_GS_QUANT_CELLS
#define MLLMB200_GS_QUANT_CELLS 0.3
#endif
    // cells of the busiest CTA, plus what quantizing a row of that many K-groups costs it before its first cell
    // (in cells' worth of time: every CTA of a matrix quantizes the row for itself)
    auto busiest = [&](int i) {
      return (double)((panels[i] + c[i] - 1) / c[i]) * groups[i] / s + MLLMB200_GS_QUANT_CELLS * groups[i];
    };
    while (used < budget) {
      int pick = -1;
      double worst = -1.0;
      for (int i = 0; i < count; ++i)
        if (c[i] < panels[i] && busiest(i) > worst) {
          worst = busiest(i);
          pick = i;
        }
      if (pick < 0) break;
      ++c[pick];
      ++used;
    }
    double w = 0.0;
    for (int i = 0; i < count; ++i) w = std::max(w, busiest(i));
    return w;
  };
  // Cluster size by a small cost model (microseconds): the busiest CTA's main loop (about 5 ns per cell
  // with 8 compute warps), what a cluster adds (its barrier and the exchange over DSMEM), and for runs
  // too long to sit in the ring all at once the time an SM needs to pull the bytes in.
  int S = 1;
  double best = 1e30;
  int c[kGsMaxProblems];
  for (int s = 1; s <= kGsMaxCluster; ++s) {
    const double cells = allocate(s, std::max(count, std::min(sms / s, gs_cluster_capacity(s))), c);
    const double t_loop = cells * 0.005;
    const double t_bw = cells > 224.0 ? cells * kCellBytes / (6.5e6 / 148) : 0.0;  // bytes / (bytes per us per SM)
    const double t = std::max(t_loop, t_bw) + (s > 1 ? 0.4 + 0.02 * s : 0.0);
    if (t < best) {
      best = t;
      S = s;
    }
  }
  allocate(S, std::max(count, std::min(sms / S, gs_cluster_capacity(S))), c);
  // a CTA's run may touch at most kGsMaxSlots / m_max panels: more, smaller clusters for a matrix until it does
  int np_max = 1, rmax = 1;
  long long stages_bound = 1;  // ring stages the busiest CTA walks through (exact for S == 1, an upper bound otherwise)
  for (int i = 0; i < count; ++i) {
    const int G = groups[i], P = panels[i];
    const long long blocks = (G + kGsBlockGroups - 1) / kGsBlockGroups;  // stages of a whole band
    for (;;) {
      const long long per_cluster = (P + c[i] - 1) / c[i];
      const long long Lc = (per_cluster * G + S - 1) / S;
      const int np = (int)std::min<long long>(per_cluster, (Lc + G - 2) / G + 1);
      if (np * m_max <= kGsMaxSlots) {
        np_max = std::max(np_max, np);
        if (S == 1) {
          if (per_cluster >= 2) rmax = 2;
          stages_bound = std::max(stages_bound, ((per_cluster + 1) / 2) * blocks);
        } else {
          if (Lc >= 2LL * G) rmax = 2;
          // every panel the run touches is walked in blocks of kGsBlockGroups groups: at most one short block per panel
          stages_bound = std::max(stages_bound, (Lc + kGsBlockGroups - 1) / kGsBlockGroups + (np - 1));
        }
        break;
      }
      if (c[i] >= P) return false;
      c[i] = std::min(P, c[i] * 2);
    }
    if ((long long)((P + c[i] - 1) / c[i]) * G * S >= (1LL << 31)) return false;
    if ((long long)P * (c[i] + 1) >= (1LL << 31)) return false;
  }
  // ring: the whole run in flight when it fits in kGsRingBytes, else as many stages as fit in that (at least 2),
  // wrapping - of single panels when two stages of panel pairs would not fit
  long long stage_bytes = (long long)rmax * kGsBandBytes;
  int stages = (int)std::min<long long>(stages_bound, kGsMaxStages);
  const long long ring_cap = stages_bound * stage_bytes > kGsLongRunBytes ? kGsRingBytesLong : kGsRingBytes;
  if (stages_bound * stage_bytes > ring_cap) {
    if (rmax == 2 && 2 * stage_bytes > ring_cap) {
      rmax = 1;
      stage_bytes = kGsBandBytes;
    }
    stages = (int)std::min<long long>(kGsMaxStages, std::max<long long>(2, ring_cap / stage_bytes));
  }
  for (;;) {
    const GsSmem L = gs_smem_layout(m_max, g_max, S, rmax, stages, np_max);
    if (L.total <= kGsSmemBudget) {
      plan->smem = L.total;
      break;
    }
    if (stages > 2) --stages;
    else return false;
  }
  int begin = 0;
  for (int i = 0; i < count; ++i) {
    plan->cl_begin[i] = begin;
    plan->clusters[i] = c[i];
    begin += c[i];
  }
  plan->total_clusters = begin;
  plan->cluster_size = S;
  plan->rmax = rmax;
  plan->stages = stages;
  plan->np_max = np_max;
  plan->g_max = g_max;
  return true;
}

static bool g_gs_trace_on = false;
static int g_gs_trace_next = 0, g_gs_trace_cap = 0;

// Development aid: record %globaltimer stamps of the first and last CTA of the next `capacity` launches
// into dev_buf (8-byte words: [0] unused, then per launch 2 x kGsTraceStamps stamps).  nullptr switches it off.
cudaError_t w4a32_gemv_stream_set_trace(unsigned long long* dev_buf, int capacity) {
  cudaError_t e = cudaMemcpyToSymbol(g_gs_trace, &dev_buf, sizeof(dev_buf));
  if (e != cudaSuccess) return e;
  e = cudaMemcpyToSymbol(g_gs_trace_capacity, &capacity, sizeof(capacity));
  if (e != cudaSuccess) return e;
  g_gs_trace_on = dev_buf != nullptr && capacity > 0;
  g_gs_trace_next = 0;
  g_gs_trace_cap = capacity;
  return cudaSuccess;
}

template <int M_MAX>
static cudaError_t gs_launch_t(const GsParams& prm, int grid, size_t smem, cudaStream_t stream) {
  const cudaError_t e = gs_configure<M_MAX>();
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(kGsThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (prm.cluster_size > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = (unsigned)prm.cluster_size;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
  }
  if (prm.use_pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = (unsigned)na;
  return cudaLaunchKernelEx(&cfg, w4a32_gemv_stream_kernel<M_MAX>, prm);
}

// One launch for `count` (1..8) weight matrices [n[i], k[i]], each with its own activations [m, k[i]]:
// fp32 x[i] (quantized inside the kernel; matrices may share a pointer) or, where x[i] == nullptr,
// records + row headers already quantized (a_rec[i], a_hdr[i]).
// Returns cudaErrorInvalidValue when the call has no plan (the caller uses the GEMM path).
cudaError_t launch_w4a32_gemv_stream(int count, const float* const* x, const int* ldx, const uint8_t* const* a_rec,
                                     const float2* const* a_hdr, int m, const int* k, const void* const* tiled,
                                     float* const* y, const int* n, const int* ldy, int use_pdl, cudaStream_t stream,
                                     int num_peers, float* const* y_peers) {
  if (count < 1 || count > kGsMaxProblems || m < 1 || m > kGsMaxM) return cudaErrorInvalidValue;
  const int m_max = m <= 1 ? 1 : (m <= 2 ? 2 : 4);
  int groups[kGsMaxProblems], panels[kGsMaxProblems];
  for (int i = 0; i < count; ++i) {
    const bool has_x = x != nullptr && x[i] != nullptr;
    if (!has_x && (a_rec == nullptr || a_hdr == nullptr || a_rec[i] == nullptr || a_hdr[i] == nullptr))
      return cudaErrorInvalidValue;
    groups[i] = (k[i] + kGroup - 1) / kGroup;
    panels[i] = (n[i] + kPanelRows - 1) / kPanelRows;
  }
  GsPlan plan;
  if (!gs_make_plan(m_max, count, groups, panels, &plan)) return cudaErrorInvalidValue;
  GsParams prm = {};
  prm.m = m;
  prm.cluster_size = plan.cluster_size;
  prm.rmax = plan.rmax;
  prm.stages = plan.stages;
  prm.np_max = plan.np_max;
  prm.g_max = plan.g_max;
  prm.use_pdl = use_pdl & 1;
  prm.num_problems = count;
  prm.trace = 0;
  if (g_gs_trace_on && g_gs_trace_next < g_gs_trace_cap) prm.trace = ++g_gs_trace_next;
  for (int i = 0; i < count; ++i) {
    const TiledHeader th = make_tiled_header(n[i], k[i], 0, 0);
    GsProblem& q = prm.prob[i];
    const bool has_x = x != nullptr && x[i] != nullptr;
    q.x = has_x ? x[i] : nullptr;
    q.a_rec = has_x ? nullptr : a_rec[i];
    q.a_hdr = has_x ? nullptr : a_hdr[i];
    q.tiled = static_cast<const uint8_t*>(tiled[i]);
    q.y = y[i];
    q.ldx = has_x ? ldx[i] : 0;
    q.ldy = ldy[i];
    q.n = n[i];
    q.k = k[i];
    q.num_groups = groups[i];
    q.num_panels = panels[i];
    q.cl_begin = plan.cl_begin[i];
    q.clusters = plan.clusters[i];
    q.zsum_off = th.zsum_off;
    q.bias_off = th.bias_off;
    q.num_peers = 0;
    if (num_peers > 0 && y_peers != nullptr) {  // (single-matrix calls only: the same offsets in every peer's buffer)
      if (count != 1 || num_peers > kGsMaxPeers) return cudaErrorInvalidValue;
      q.num_peers = num_peers;
      for (int j = 0; j < num_peers; ++j) q.y_peer[j] = y_peers[j];
    }
  }
  const int grid = plan.total_clusters * plan.cluster_size;
  switch (m_max) {
    case 1: return gs_launch_t<1>(prm, grid, plan.smem, stream);
    case 2: return gs_launch_t<2>(prm, grid, plan.smem, stream);
    default: return gs_launch_t<4>(prm, grid, plan.smem, stream);
  }
}

bool w4a32_gemv_stream_supported(int m, int count, const int* k, const int* n) {
  if (m < 1 || m > kGsMaxM || count < 1 || count > kGsMaxProblems) return false;
  int groups[kGsMaxProblems], panels[kGsMaxProblems];
  for (int i = 0; i < count; ++i) {
    groups[i] = (k[i] + kGroup - 1) / kGroup;
    panels[i] = (n[i] + kPanelRows - 1) / kPanelRows;
  }
  GsPlan plan;
  return gs_make_plan(m <= 1 ? 1 : (m <= 2 ? 2 : 4), count, groups, panels, &plan);
}

// Host-only self-check of the work decomposition for a call: replays, with the kernel's own integer
// arithmetic, which cells every CTA requests, which cell every warp consumes under which K-group and
// panel slot, which K-groups of the activations a CTA quantizes, and where every panel is finished.
// Verifies that each weight cell is requested and consumed exactly once, that a run touches at most
// np_max panels, that every consumed cell's activation group was quantized by its CTA, and that every
// panel is finished exactly once with the parts of exactly the CTAs that hold its cells.  Returns 0
// when the plan is sound, a positive code naming the first violated property otherwise, -1 when the
// call has no plan.
int w4a32_gemv_stream_plan_check(int m, int count, const int* k, const int* n, int* clusters, int* cluster_size, int* cpc,
                                 int* stages, size_t* smem) {
  if (count < 1 || count > kGsMaxProblems || m < 1 || m > kGsMaxM) return -1;
  const int m_max = m <= 1 ? 1 : (m <= 2 ? 2 : 4);
  int groups[kGsMaxProblems], panels[kGsMaxProblems];
  for (int i = 0; i < count; ++i) {
    groups[i] = (k[i] + kGroup - 1) / kGroup;
    panels[i] = (n[i] + kPanelRows - 1) / kPanelRows;
  }
  GsPlan plan = {};
  if (!gs_make_plan(m_max, count, groups, panels, &plan)) return -1;
  if (clusters) *clusters = plan.total_clusters;
  if (cluster_size) *cluster_size = plan.cluster_size;
  if (cpc) *cpc = plan.rmax * kGsBlockGroups;
  if (stages) *stages = plan.stages;
  if (smem) *smem = plan.smem;
  if (plan.np_max * m_max > kGsMaxSlots) return 1;
  const int S = plan.cluster_size;
  long long worst_stages = 0;
  for (int pi = 0; pi < count; ++pi) {
    const int G = groups[pi], P = panels[pi], C = plan.clusters[pi];
    if (G > plan.g_max) return 1;
    std::vector<uint8_t> requested((size_t)P * G, 0), consumed((size_t)P * G, 0);
    std::vector<uint8_t> finished((size_t)P, 0);
    for (int q = 0; q < C; ++q) {
      const int p0 = (int)(((uint32_t)q * (uint32_t)P) / (uint32_t)C);
      const int p1 = (int)(((uint32_t)(q + 1) * (uint32_t)P) / (uint32_t)C);
      const uint32_t T = (uint32_t)(p1 - p0) * (uint32_t)G;
      auto cta_begin = [&](uint32_t r) { return S > 1 ? (int)((r * T) / (uint32_t)S) : (int)(r * T); };
      std::vector<std::vector<int>> senders(S), readers(S);
      std::vector<int> sent_panel(S, -1), kept_panel(S, -1);
      for (int rank = 0; rank < S; ++rank) {
        const int cb = cta_begin(rank), ce = cta_begin(rank + 1);
        const int Lc = ce - cb;
        const int pa = cb / G;
        const int np_run = Lc > 0 ? (ce - 1) / G - pa + 1 : 0;
        if (np_run > plan.np_max) return 2;
        const int np_cta = np_run;
        (void)np_cta;
        const int g_lo = np_run == 1 ? cb - pa * G : 0;
        const int g_hi = np_run == 1 ? ce - 1 - pa * G : G - 1;
        // the walk the producer and the compute warps share: stages, their copies, and who consumes which cell
        GsWalk w;
        w.init(cb, ce, G, (plan.rmax == 2 && np_run >= 2) ? 2 : 1);
        long long nst = 0;
        int last_slot_flushed = -1;
        while (w.next()) {
          ++nst;
          if (w.R < 1 || w.R > plan.rmax || w.cnt < 1 || w.cnt > kGsBlockGroups) return 3;
          for (int r = 0; r < w.R; ++r) {
            const int slot = w.panel + r - pa;
            if (slot < 0 || slot >= np_cta) return 6;
            for (int j = 0; j < w.cnt; ++j) {
              const int g = w.g0 + j;
              const long long cell = (long long)(w.panel + r) * G + g;  // cell of the cluster
              if (cell < cb || cell >= ce) return 4;
              if (g < g_lo || g > g_hi) return 16;  // its activation record was not produced
              const size_t gc = (size_t)p0 * G + (size_t)cell;
              if (requested[gc]++) return 5;
              // consumed by warp j % 8 as its item j / 8
              if (j >= kGsBlockGroups) return 7;
              if (consumed[gc]++) return 7;
            }
            if (w.band_end) {
              if (slot != last_slot_flushed + 1) return 17;  // every slot parked once, in order
              last_slot_flushed = slot;
            }
          }
        }
        if (Lc > 0 && last_slot_flushed != np_cta - 1) return 17;
        if (nst > worst_stages) worst_stages = nst;
        // the epilogue's ownership rules
        const bool own_first = cb == pa * G;
        int keeps = 0;
        for (int jp = 0; jp < np_cta; ++jp) {
          const int c_lo = (pa + jp) * G, c_hi = c_lo + G;
          const bool complete = cb <= c_lo && ce >= c_hi;
          if (jp == 0 && !own_first) {
            uint32_t owner = 0;
            for (uint32_t r = 1; r < (uint32_t)rank; ++r)
              if (cta_begin(r) <= c_lo && cta_begin(r + 1) > c_lo) owner = r;
            if (!(cta_begin(owner) <= c_lo && cta_begin(owner + 1) > c_lo)) return 8;
            senders[owner].push_back(rank);
            if (sent_panel[owner] >= 0 && sent_panel[owner] != pa + jp) return 9;
            sent_panel[owner] = pa + jp;
          } else if (!complete) {
            if (++keeps > 1 || jp != np_cta - 1) return 10;
            kept_panel[rank] = pa + jp;
            for (uint32_t r = rank + 1; r < (uint32_t)S; ++r)
              if (cta_begin(r) < c_hi && cta_begin(r + 1) > cta_begin(r)) readers[rank].push_back((int)r);
            if (finished[p0 + pa + jp]++) return 11;
          } else {
            if (finished[p0 + pa + jp]++) return 11;
          }
        }
      }
      for (int owner = 0; owner < S; ++owner) {  // senders and readers must agree
        if (senders[owner] != readers[owner]) return 12;
        if (!senders[owner].empty() && kept_panel[owner] != sent_panel[owner]) return 13;
      }
    }
    for (size_t i = 0; i < requested.size(); ++i)
      if (requested[i] != 1 || consumed[i] != 1) return 14;
    for (int i = 0; i < P; ++i)
      if (finished[i] != 1) return 15;
  }
  return 0;
}

}  // namespace mllmb200
