// Streaming W4A32 GEMV for decode (M <= 4 activation rows), sm_100a.
//
// Work unit: a CTA owns `pp` consecutive 32-row panels of one weight matrix and one contiguous
// slice of their K-groups.  In the tile layout (layout.h) that is ONE contiguous byte range, so
// thread 0 moves all of it into shared memory with a few bulk copies (cp.async.bulk, one mbarrier
// per chunk) issued before anything else: every weight byte the CTA will ever need is in flight
// from its first instructions.  That is what a kernel whose whole input is a few tens of KB per SM
// needs to get near the HBM roofline; there is no steady state to pipeline.
//
// While the weights fly the CTA stages the fp32 activation row(s) in shared memory (one more bulk
// copy), finds each row's min/max, and quantizes its K-slice to int8 (dynamic asymmetric
// quantization, reference: tests/Arm/KaiLinearTest.hpp:163-230) in the byte order the nibble unpack
// produces.  Then the warps of a panel take its cells (panel x K-group) round robin: lane = weight
// row, one 16-byte shared load = the row's 32 nibbles, two masks split them into byte vectors,
// eight dp4a give the exact int32 group sum, one FMA applies the group scale.  Partials meet in
// shared memory in a fixed order; when K is split over the CTAs of a thread-block cluster they
// are written into the leader's shared memory and summed there in rank order (deterministic).
//
//   y[m,n] = lhs_scale[m] * ( sum_b float(sum_{k in b} a_q[m,k] * w[n,k]) * s[n,b]  +  a_off[m] * zsum[n] ) + bias[n]
//
// equals the reference expression (KaiLinearTest.hpp:338-377) with the zero-point term
// a_off * sum_k w[n,k] s[n,b] taken out of the integer sum (zsum is precomputed per row at repack).
//
// Up to 4 weight matrices that share the same activations (q/k/v, gate/up) run as one launch.
#include "device_common.cuh"

namespace mllmb200 {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvMaxChunks = 16;
constexpr int kGemvMaxSplit = 8;
constexpr int kGemvMaxProblems = 4;
constexpr int kGemvTargetCtas = 2 * 148;

struct GemvProblem {
  const uint8_t* tiled;  // TiledHeader at offset 0
  float* y;
  int n, ldy;
  int cta_begin;            // first blockIdx.x of this problem
  size_t zsum_off, bias_off;  // byte offsets of the per-row arrays inside the tiled buffer
};

struct GemvParams {
  const float* x;
  int m, k, ldx;
  int num_groups;       // K-groups per row
  int cells_per_slice;  // K-groups per CTA
  int split;            // CTAs per panel group (= cluster size)
  int pp;               // panels per CTA (power of two <= 8; > 1 only when split == 1)
  int chunk_shift;      // cells per bulk copy = 1 << chunk_shift
  int stage_x;          // 1: activation rows are staged in shared memory by a bulk copy
  int use_pdl;
  int num_problems;
  GemvProblem prob[kGemvMaxProblems];
};

// shared memory carve-up (dynamic, 128-byte aligned base):
//   [0, 136)      kGemvMaxChunks + 1 mbarriers
//   [256, 512)    min/max scratch (64 floats)
//   [512, 576)    row params: M_MAX x {recip scale, a_off}
//   wbuf          pp * cells_per_slice * 576   weights (bulk copy destination)
//   abuf          M_MAX * cells_per_slice * 48 permuted int8 activations + (-8 * group sum)
//   red           kGemvWarps * M_MAX * 32 floats
//   cred          kGemvMaxSplit * M_MAX * 32 floats (cluster leader only)
//   xbuf          M_MAX * k_pad4 floats (only when stage_x)
struct GemvSmem {
  size_t wbuf, abuf, red, cred, xbuf, total;
};
__host__ __device__ inline GemvSmem gemv_smem_layout(int m_max, int pp, int cells_per_slice, int k, int stage_x) {
  GemvSmem s;
  size_t off = 576;
  off = (off + 127) & ~size_t(127);
  s.wbuf = off;
  off += (size_t)pp * cells_per_slice * kCellBytes;
  s.abuf = off;
  off += (size_t)m_max * cells_per_slice * kActRecordBytes;
  s.red = off;
  off += (size_t)kGemvWarps * m_max * 32 * 4;
  s.cred = off;
  off += (size_t)kGemvMaxSplit * m_max * 32 * 4;
  off = (off + 15) & ~size_t(15);
  s.xbuf = off;
  if (stage_x) off += (size_t)m_max * (size_t)k * 4;
  s.total = off + 128;  // slack for the base alignment
  return s;
}

template <int M_MAX>
__global__ void __launch_bounds__(kGemvThreads) w4a32_gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const GemvSmem L = gemv_smem_layout(M_MAX, p.pp, p.cells_per_slice, p.k, p.stage_x);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [kGemvMaxChunks] weights, [kGemvMaxChunks] activations
  float* mm_scratch = reinterpret_cast<float*>(smem + 256);
  float* rowp = reinterpret_cast<float*>(smem + 512);
  uint8_t* wbuf = smem + L.wbuf;
  uint8_t* abuf = smem + L.abuf;
  float* red = reinterpret_cast<float*>(smem + L.red);
  float* cred = reinterpret_cast<float*>(smem + L.cred);
  float* xbuf = reinterpret_cast<float*>(smem + L.xbuf);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- which problem / panels / K-slice is ours
  int pi = 0;
#pragma unroll
  for (int i = 1; i < kGemvMaxProblems; ++i)
    if (i < p.num_problems && (int)blockIdx.x >= p.prob[i].cta_begin) pi = i;
  const GemvProblem& pr = p.prob[pi];
  const int local_cta = (int)blockIdx.x - pr.cta_begin;
  const int unit = local_cta / p.split;                 // index of the panel group
  const int slice = local_cta - unit * p.split;
  const int num_panels = (pr.n + kPanelRows - 1) / kPanelRows;
  const int panel0 = unit * p.pp;
  const int npanels = min(p.pp, num_panels - panel0);   // >= 1
  const int g0 = slice * p.cells_per_slice;             // first K-group of this CTA
  const int ncells = min(p.cells_per_slice, p.num_groups - g0);  // >= 1 by construction
  // with pp > 1 the slice is the whole K range, so the panels' cells are one contiguous run
  const int total_cells = npanels * ncells;
  const int cells_per_chunk = 1 << p.chunk_shift;
  const int nchunks = (total_cells + cells_per_chunk - 1) >> p.chunk_shift;

  const TiledHeader* hdr = reinterpret_cast<const TiledHeader*>(pr.tiled);

  // ---- 1. get every weight byte of this CTA in flight
  if (tid == 0) {
    for (int c = 0; c < nchunks; ++c) mbar_init(&bars[c], 1);
    mbar_init(&bars[kGemvMaxChunks], 1);
    mbar_fence_init();
    const uint8_t* src = pr.tiled + sizeof(TiledHeader) + ((size_t)panel0 * p.num_groups + g0) * kCellBytes;
    for (int c = 0; c < nchunks; ++c) {
      const int c0 = c << p.chunk_shift;
      const uint32_t bytes = (uint32_t)(min(cells_per_chunk, total_cells - c0) * kCellBytes);
      mbar_arrive_expect_tx(&bars[c], bytes);
      bulk_g2s(wbuf + (size_t)c0 * kCellBytes, src + (size_t)c0 * kCellBytes, bytes, &bars[c]);
    }
  }
  // the next kernel in the stream may start fetching its own (constant) weights now
  if (p.use_pdl) pdl_launch_dependents();
  // header word and per-row constants: requested now, consumed after the main loop
  const uint32_t hdr_magic = hdr->magic, hdr_n = hdr->n, hdr_k = hdr->k, scale_mode = hdr->scale_mode;
  const int rm = warp;  // activation row this warp finishes in the reductions (valid when < M_MAX)
  float zs[8], bs[8];   // per-row constants of the epilogue, one per panel of the CTA
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    zs[q] = 0.0f;
    bs[q] = 0.0f;
    if (rm < M_MAX && q < npanels) {
      const int n_pad = (panel0 + q) * kPanelRows + lane;  // always inside the padded per-row arrays
      zs[q] = reinterpret_cast<const float*>(pr.tiled + pr.zsum_off)[n_pad];
      bs[q] = reinterpret_cast<const float*>(pr.tiled + pr.bias_off)[n_pad];
    }
  }
  bool ok = true;
  // the weights are constant; the activations may come from the kernel before us
  if (p.use_pdl) pdl_wait_prior();

  // ---- 2. activations: stage (optional), min/max, quantize this CTA's K-slice
  if (p.stage_x) {
    if (tid == 0) {
      const uint32_t row_bytes = (uint32_t)p.k * 4u;
      mbar_arrive_expect_tx(&bars[kGemvMaxChunks], row_bytes * (uint32_t)p.m);
      for (int m = 0; m < p.m; ++m)
        bulk_g2s(xbuf + (size_t)m * p.k, p.x + (size_t)m * p.ldx, row_bytes, &bars[kGemvMaxChunks]);
    }
    __syncthreads();  // barrier initialisation visible to the waiters
    ok = mbar_wait_bounded(&bars[kGemvMaxChunks], 0);  // on a timeout: keep going (barriers below), store nothing
  } else {
    __syncthreads();
  }
#pragma unroll
  for (int m = 0; m < M_MAX; ++m) {
    if (m < p.m) {
      const float* row = p.stage_x ? (xbuf + (size_t)m * p.k) : (p.x + (size_t)m * p.ldx);
      float mn, mx;
      block_row_minmax(row, p.k, mm_scratch, mn, mx);
      const ActQuantParams q = act_quant_params(mn, mx);
      if (tid == 0) {
        rowp[m * 2 + 0] = q.recip_scale;
        rowp[m * 2 + 1] = (float)(-q.nzp);
      }
      // item = (cell, word pair i): 8 consecutive k -> low-half word i and high-half word i.
      // The loop bound is uniform over the CTA so that the quad shuffles below see full warps.
      for (int base = 0; base < ncells * 4; base += kGemvThreads) {
        const int item = base + tid;
        const bool valid = item < ncells * 4;
        const int c = item >> 2, i = item & 3;
        const int kbase = (g0 + c) * kGroup + i * 8;
        int q8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int kk = kbase + j;
          q8[j] = (valid && kk < p.k) ? act_quant_value(row[kk], q) : 0;
        }
        const uint32_t lo = ((uint32_t)q8[0] & 0xFFu) | (((uint32_t)q8[2] & 0xFFu) << 8) |
                            (((uint32_t)q8[4] & 0xFFu) << 16) | (((uint32_t)q8[6] & 0xFFu) << 24);
        const uint32_t hi = ((uint32_t)q8[1] & 0xFFu) | (((uint32_t)q8[3] & 0xFFu) << 8) |
                            (((uint32_t)q8[5] & 0xFFu) << 16) | (((uint32_t)q8[7] & 0xFFu) << 24);
        int s = q8[0] + q8[1] + q8[2] + q8[3] + q8[4] + q8[5] + q8[6] + q8[7];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (valid) {
          uint32_t* rec = reinterpret_cast<uint32_t*>(abuf + ((size_t)m * p.cells_per_slice + c) * kActRecordBytes);
          rec[i] = lo;
          rec[4 + i] = hi;
          if (i == 0) rec[8] = (uint32_t)(-8 * s);
        }
      }
    }
  }
  __syncthreads();

  // ---- 3. main loop.  The kGemvWarps / pp warps of a panel take its cells round robin; lane = weight row.
  const int wpp = kGemvWarps / p.pp;       // warps per panel
  const int pl = warp / wpp;               // panel (local) of this warp
  const int wr = warp - pl * wpp;          // rank of this warp inside its panel's group
  float acc[M_MAX];
#pragma unroll
  for (int m = 0; m < M_MAX; ++m) acc[m] = 0.0f;
  if (pl < npanels && ok) {
    int ready_chunk = -1;
    for (int c = wr; c < ncells; c += wpp) {
      const int lin = pl * ncells + c;
      const int chunk = lin >> p.chunk_shift;
      if (chunk != ready_chunk) {
        ok = mbar_wait_bounded(&bars[chunk], 0);
        if (!ok) break;
        ready_chunk = chunk;
      }
      const uint8_t* cell = wbuf + (size_t)lin * kCellBytes;
      const uint4 wq = *reinterpret_cast<const uint4*>(cell + lane * 16);
      const uint32_t sraw = *reinterpret_cast<const uint16_t*>(cell + kCellNibbleBytes + lane * 2);
      const float s = decode_scale(sraw, scale_mode);
      const int lo0 = (int)(wq.x & 0x0F0F0F0Fu), hi0 = (int)((wq.x >> 4) & 0x0F0F0F0Fu);
      const int lo1 = (int)(wq.y & 0x0F0F0F0Fu), hi1 = (int)((wq.y >> 4) & 0x0F0F0F0Fu);
      const int lo2 = (int)(wq.z & 0x0F0F0F0Fu), hi2 = (int)((wq.z >> 4) & 0x0F0F0F0Fu);
      const int lo3 = (int)(wq.w & 0x0F0F0F0Fu), hi3 = (int)((wq.w >> 4) & 0x0F0F0F0Fu);
#pragma unroll
      for (int m = 0; m < M_MAX; ++m) {
        if (m < p.m) {
          const uint8_t* rec = abuf + ((size_t)m * p.cells_per_slice + c) * kActRecordBytes;
          const int4 alo = *reinterpret_cast<const int4*>(rec);
          const int4 ahi = *reinterpret_cast<const int4*>(rec + 16);
          int iacc = *reinterpret_cast<const int*>(rec + 32);  // -8 * sum(a_q): nibbles are q+8
          iacc = __dp4a(alo.x, lo0, iacc);
          iacc = __dp4a(ahi.x, hi0, iacc);
          iacc = __dp4a(alo.y, lo1, iacc);
          iacc = __dp4a(ahi.y, hi1, iacc);
          iacc = __dp4a(alo.z, lo2, iacc);
          iacc = __dp4a(ahi.z, hi2, iacc);
          iacc = __dp4a(alo.w, lo3, iacc);
          iacc = __dp4a(ahi.w, hi3, iacc);
          acc[m] = fmaf((float)iacc, s, acc[m]);
        }
      }
    }
  }

  // ---- 4. warps -> CTA partials in shared memory
#pragma unroll
  for (int m = 0; m < M_MAX; ++m) red[(warp * M_MAX + m) * 32 + lane] = acc[m];
  __syncthreads();
  const bool hdr_ok = hdr_magic == kTiledMagic && hdr_n == (uint32_t)pr.n && hdr_k == (uint32_t)p.k;
  if (!hdr_ok && tid == 0) atomicOr(&g_device_status, kDevStatusBadHeader);

  // ---- 5. reduction + epilogue.  Warp rm (< M_MAX) finishes activation row rm for every panel of the CTA.
  const uint32_t rank = p.split > 1 ? cluster_ctarank() : 0u;
  if (p.split > 1) {
    // pp == 1 here: one panel, one partial per (row, lane)
    if (rm < M_MAX) {
      float part = 0.0f;
#pragma unroll
      for (int w = 0; w < kGemvWarps; ++w) part += red[(w * M_MAX + rm) * 32 + lane];
      st_cluster_f32(map_to_cta(&cred[(rank * M_MAX + rm) * 32 + lane], 0), part);
    }
    cluster_sync_all();
    if (rank != 0) return;
  }
  if (rm < M_MAX && rm < p.m && ok && hdr_ok) {
    const float lhs_scale = rowp[rm * 2 + 0], a_off = rowp[rm * 2 + 1];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (q >= npanels) break;
      float part = 0.0f;
      if (p.split > 1) {
        for (int r = 0; r < p.split; ++r) part += cred[(r * M_MAX + rm) * 32 + lane];
      } else {
        for (int w = q * wpp; w < (q + 1) * wpp; ++w) part += red[(w * M_MAX + rm) * 32 + lane];
      }
      const int n_pad = (panel0 + q) * kPanelRows + lane;
      if (n_pad < pr.n) {
        float v = fmaf(a_off, zs[q], part);
        v = fmaf(v, lhs_scale, bs[q]);
        pr.y[(size_t)rm * pr.ldy + n_pad] = clamp_flt_max(v);
      }
    }
  }
}

// ---- host side ---------------------------------------------------------------------------------
struct GemvPlan {
  int split, cells_per_slice, pp, chunk_shift, stage_x;
  size_t smem;
};

// total_panels: panels of all problems of the launch together.
static bool gemv_make_plan(int m_max, int m, int k, int ldx, const float* x, int num_groups, int total_panels,
                           GemvPlan* plan) {
  int split = 1, pp = 1;
  auto cps = [&](int s) { return (num_groups + s - 1) / s; };
  if (total_panels >= kGemvTargetCtas) {
    // enough panels: several panels per CTA so the activation prologue is paid ~300 times, not thousands
    while (pp < 8 && total_panels / (pp * 2) >= kGemvTargetCtas / 2 + 20 &&
           (size_t)(pp * 2) * num_groups * kCellBytes <= 64 * 1024)
      pp *= 2;
  } else {
    // few panels: split K over the CTAs of a cluster, keeping at least 12 K-groups per CTA
    while (split < kGemvMaxSplit && total_panels * split < (kGemvTargetCtas * 3) / 4 && cps(split * 2) >= 12) split *= 2;
  }
  // a slice larger than ~96 KB does not fit beside the rest: split further if possible
  while (split < kGemvMaxSplit && pp == 1 && (size_t)cps(split) * kCellBytes > 96 * 1024) split *= 2;
  int cells = cps(split);
  split = (num_groups + cells - 1) / cells;  // drop empty trailing slices
  const int total_cells = pp * cells;
  int shift = 2;
  while (((total_cells + (1 << shift) - 1) >> shift) > kGemvMaxChunks) ++shift;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (k % 4) == 0 && (m == 1 || (ldx % 4) == 0);
  int stage = aligned && (size_t)m_max * k * 4 <= 40 * 1024;
  GemvSmem L = gemv_smem_layout(m_max, pp, cells, k, stage);
  if (L.total > 200 * 1024 && stage) {
    stage = 0;
    L = gemv_smem_layout(m_max, pp, cells, k, stage);
  }
  if (L.total > 200 * 1024) return false;
  plan->split = split;
  plan->cells_per_slice = cells;
  plan->pp = pp;
  plan->chunk_shift = shift;
  plan->stage_x = stage;
  plan->smem = L.total;
  return true;
}

template <int M_MAX>
static cudaError_t launch_gemv_t(const GemvParams& prm, size_t smem, int grid, cudaStream_t stream) {
  static bool configured[64] = {};  // per device, per M_MAX instantiation
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (smem > 48 * 1024 && !(dev >= 0 && dev < 64 && configured[dev])) {
    e = cudaFuncSetAttribute(w4a32_gemv_kernel<M_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(200 * 1024 + 512));
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(kGemvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (prm.split > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = (unsigned)prm.split;
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
  return cudaLaunchKernelEx(&cfg, w4a32_gemv_kernel<M_MAX>, prm);
}

// One launch for `count` (1..4) weight matrices that share x [m, k].
// Returns cudaErrorInvalidValue when the shape has no GEMV plan (the caller uses the GEMM path).
cudaError_t launch_w4a32_gemv_grouped(const float* x, int m, int k, int ldx, int count, const void* const* tiled,
                                      float* const* y, const int* n, const int* ldy, int use_pdl,
                                      cudaStream_t stream) {
  if (count < 1 || count > kGemvMaxProblems || m < 1 || m > 4) return cudaErrorInvalidValue;
  const int num_groups = (k + kGroup - 1) / kGroup;
  const int m_max = m <= 1 ? 1 : (m <= 2 ? 2 : 4);
  int total_panels = 0;
  for (int i = 0; i < count; ++i) total_panels += (n[i] + kPanelRows - 1) / kPanelRows;
  GemvPlan plan;
  if (!gemv_make_plan(m_max, m, k, ldx, x, num_groups, total_panels, &plan)) return cudaErrorInvalidValue;
  GemvParams prm = {};
  prm.x = x;
  prm.m = m;
  prm.k = k;
  prm.ldx = ldx;
  prm.num_groups = num_groups;
  prm.cells_per_slice = plan.cells_per_slice;
  prm.split = plan.split;
  prm.pp = plan.pp;
  prm.chunk_shift = plan.chunk_shift;
  prm.stage_x = plan.stage_x;
  prm.use_pdl = use_pdl;
  prm.num_problems = count;
  int cta = 0;
  for (int i = 0; i < count; ++i) {
    const int panels = (n[i] + kPanelRows - 1) / kPanelRows;
    const TiledHeader th = make_tiled_header(n[i], k, 0, 0);
    prm.prob[i].tiled = static_cast<const uint8_t*>(tiled[i]);
    prm.prob[i].y = y[i];
    prm.prob[i].n = n[i];
    prm.prob[i].ldy = ldy[i];
    prm.prob[i].cta_begin = cta;
    prm.prob[i].zsum_off = th.zsum_off;
    prm.prob[i].bias_off = th.bias_off;
    cta += ((panels + plan.pp - 1) / plan.pp) * plan.split;
  }
  switch (m_max) {
    case 1: return launch_gemv_t<1>(prm, plan.smem, cta, stream);
    case 2: return launch_gemv_t<2>(prm, plan.smem, cta, stream);
    default: return launch_gemv_t<4>(prm, plan.smem, cta, stream);
  }
}

cudaError_t launch_w4a32_gemv(const float* x, const void* tiled, float* y, int m, int k, int n, int ldx, int ldy,
                              int use_pdl, cudaStream_t stream) {
  return launch_w4a32_gemv_grouped(x, m, k, ldx, 1, &tiled, &y, &n, &ldy, use_pdl, stream);
}

bool w4a32_gemv_supported(int m, int k, int n) {
  if (m < 1 || m > 4) return false;
  GemvPlan plan;
  // alignment only decides staging, never support: probe with the worst case (no staging)
  return gemv_make_plan(m <= 1 ? 1 : (m <= 2 ? 2 : 4), m, k, k | 1, nullptr, (k + kGroup - 1) / kGroup,
                        (n + kPanelRows - 1) / kPanelRows, &plan);
}

}  // namespace mllmb200
