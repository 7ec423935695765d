// Streaming W4A32 GEMV for decode (M <= 4 activation rows), sm_100a.
//
// Work unit: a CTA owns `pp` consecutive 32-row panels of one weight matrix and one contiguous
// slice of their K-groups; the `split` CTAs that cover the K range of the same panels form a
// thread-block cluster.  In the tile layout (layout.h) a CTA's weights are ONE contiguous byte
// range, so warp 0 moves all of it into shared memory with a few bulk copies (cp.async.bulk, one
// mbarrier per chunk) issued before anything else: every weight byte the CTA will ever need is in
// flight from its first instructions.  Under programmatic dependent launch this prefetch overlaps
// the kernel in front (weights are constants); only what depends on x waits for it.
//
// The activations arrive already quantized (act_quant.cu: int8 records in the byte order the
// nibble unpack produces + one {lhs_scale, a_off} header per row; dynamic asymmetric int8 per row
// as in the reference project, tests/Arm/KaiLinearTest.hpp:163-230).  The CTA's K-slice of them is
// one more bulk copy.  Quantizing inside this kernel was measured and lost: every CTA repeats the
// row reduction, and at 1-3 us per launch that prologue costs more than the second launch.
//
// Main loop: the warps of a panel take its cells (panel x K-group) round robin; lane = weight row,
// one 16-byte shared load = the row's 32 nibbles, two masks split them into byte vectors, eight
// dp4a on two chains give the exact int32 group sum, one FMA applies the group scale.  Partials
// meet in shared memory in a fixed order; across the cluster they are written into the leader's
// shared memory and summed in rank order, so results are deterministic.
//
//   y[m,n] = lhs_scale[m] * ( sum_b float(sum_{k in b} a_q[m,k] * w[n,k]) * s[n,b]  +  a_off[m] * zsum[n] ) + bias[n]
//
// equals the reference expression (tests/Arm/KaiLinearTest.hpp:338-377) with the zero-point term
// a_off * sum_k w[n,k] s[n,b] taken out of the integer sum (zsum is precomputed per row at repack).
//
// Up to 4 weight matrices that share the same activations (q/k/v, gate/up) run as one launch.
#include "device_common.cuh"

namespace mllmb200 {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvMaxChunks = 8;
constexpr int kGemvMaxSplit = 8;
constexpr int kGemvMaxProblems = 4;
constexpr int kGemvMaxM = 4;
constexpr int kGemvCtasPerSm = 4;  // __launch_bounds__ below caps registers at 64 to allow this

struct GemvProblem {
  const uint8_t* tiled;  // TiledHeader at offset 0
  float* y;
  int n, ldy;
  int cta_begin;              // first blockIdx.x of this problem
  size_t zsum_off, bias_off;  // byte offsets of the per-row arrays inside the tiled buffer
};

struct GemvParams {
  const uint8_t* a_rec;  // [m][num_groups] 48-byte activation records
  const float2* a_hdr;   // [m] {lhs_scale, a_off bits}
  int m, k;
  int num_groups;       // K-groups per row
  int cells_per_slice;  // K-groups per CTA
  int split;            // CTAs per panel group (= cluster size)
  int pp;               // panels per CTA (power of two <= 8; > 1 only when split == 1)
  int chunk_shift;      // cells per weight bulk copy = 1 << chunk_shift
  int use_pdl;
  int num_problems;
  GemvProblem prob[kGemvMaxProblems];
};

// shared memory carve-up (dynamic, 128-byte aligned base):
//   [0, 72)        kGemvMaxChunks weight barriers + 1 activation barrier
//   wbuf           pp * cells_per_slice * 576            weights (bulk copy destination)
//   abuf           M_MAX * cells_per_slice * 48          quantized activation records (bulk copy destination)
//   red            kGemvWarps * M_MAX * 32 floats        cross-warp partials
//   cred           kGemvMaxSplit * M_MAX * 32 floats     cross-CTA partials (cluster leader)
struct GemvSmem {
  size_t wbuf, abuf, red, cred, total;
};
__host__ __device__ inline GemvSmem gemv_smem_layout(int m_max, int pp, int cells_per_slice) {
  GemvSmem s;
  size_t off = 128;
  s.wbuf = off;
  off += (size_t)pp * cells_per_slice * kCellBytes;
  s.abuf = off;
  off += (size_t)m_max * cells_per_slice * kActRecordBytes;
  s.red = off;
  off += (size_t)kGemvWarps * m_max * 32 * 4;
  s.cred = off;
  off += (size_t)kGemvMaxSplit * m_max * 32 * 4;
  s.total = off + 128;  // slack for the base alignment
  return s;
}

template <int M_MAX>
__global__ void __launch_bounds__(kGemvThreads, kGemvCtasPerSm) w4a32_gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const GemvSmem L = gemv_smem_layout(M_MAX, p.pp, p.cells_per_slice);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  uint8_t* wbuf = smem + L.wbuf;
  uint8_t* abuf = smem + L.abuf;
  float* red = reinterpret_cast<float*>(smem + L.red);
  float* cred = reinterpret_cast<float*>(smem + L.cred);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- which problem / panels / K-slice is ours
  int pi = 0;
#pragma unroll
  for (int i = 1; i < kGemvMaxProblems; ++i)
    if (i < p.num_problems && (int)blockIdx.x >= p.prob[i].cta_begin) pi = i;
  const GemvProblem& pr = p.prob[pi];
  const int local_cta = (int)blockIdx.x - pr.cta_begin;
  const uint32_t rank = p.split > 1 ? cluster_ctarank() : 0u;  // == local_cta % split (cta_begin is a multiple of split)
  const int unit = p.split > 1 ? (local_cta - (int)rank) / p.split : local_cta;
  const int num_panels = (pr.n + kPanelRows - 1) / kPanelRows;
  const int panel0 = unit * p.pp;
  const int npanels = min(p.pp, num_panels - panel0);             // >= 1
  const int g0 = (int)rank * p.cells_per_slice;                   // first K-group of this CTA
  const int ncells = min(p.cells_per_slice, p.num_groups - g0);   // >= 1 by construction
  const int total_cells = npanels * ncells;  // with pp > 1 the slice is all of K: one contiguous run
  const int cells_per_chunk = 1 << p.chunk_shift;
  const int nchunks = (total_cells + cells_per_chunk - 1) >> p.chunk_shift;

  // Peers write into the leader's shared memory at the end; they may only do so once it runs.
  // Arrive now, wait just before the remote stores: the barrier latency hides behind the work.
  if (p.split > 1) cluster_arrive_relaxed();

  // ---- 1. every weight byte of this CTA in flight: lane c of warp 0 owns chunk c.
  // The tile header is checked first: a call whose N or K exceeds the buffer must not read past its end.
  const TiledHeader* hdr = reinterpret_cast<const TiledHeader*>(pr.tiled);
  const uint4 hdr4 = *reinterpret_cast<const uint4*>(pr.tiled);  // magic, version, n, k
  const uint32_t hdr_magic = hdr4.x, hdr_n = hdr4.z, hdr_k = hdr4.w, scale_mode = hdr->scale_mode;
  const bool hdr_ok = hdr_magic == kTiledMagic && hdr_n == (uint32_t)pr.n && hdr_k == (uint32_t)p.k;
  if (warp == 0) {
    if (lane < nchunks) mbar_init(&bars[lane], 1);
    if (lane == 31) mbar_init(&bars[kGemvMaxChunks], 1);
    mbar_fence_init();
    __syncwarp();
    if (lane < nchunks && hdr_ok) {
      const uint8_t* src = pr.tiled + sizeof(TiledHeader) + ((size_t)panel0 * p.num_groups + g0) * kCellBytes;
      const int c0 = lane << p.chunk_shift;
      const uint32_t bytes = (uint32_t)(min(cells_per_chunk, total_cells - c0) * kCellBytes);
      mbar_arrive_expect_tx(&bars[lane], bytes);
      bulk_g2s(wbuf + (size_t)c0 * kCellBytes, src + (size_t)c0 * kCellBytes, bytes, &bars[lane]);
    }
  }
  // the next kernel in the stream may start fetching its own (constant) weights now
  if (p.use_pdl) pdl_launch_dependents();
  // the weights are constant; the activations may come from the kernel before us
  if (p.use_pdl) pdl_wait_prior();

  // ---- 2. this CTA's slice of the quantized activations: one bulk copy per row (lane m of warp 0)
  if (warp == 0) {
    if (lane == 31) mbar_arrive_expect_tx(&bars[kGemvMaxChunks], (uint32_t)(ncells * kActRecordBytes * p.m));
    __syncwarp();
    if (lane < p.m)
      bulk_g2s(abuf + (size_t)lane * p.cells_per_slice * kActRecordBytes,
               p.a_rec + ((size_t)lane * p.num_groups + g0) * kActRecordBytes, (uint32_t)(ncells * kActRecordBytes),
               &bars[kGemvMaxChunks]);
  }
  const int rm = warp;  // activation row this warp finishes in the epilogue (valid when < M_MAX)
  float lhs_scale = 0.0f, a_off = 0.0f;
  if (rm < M_MAX && rm < p.m) {
    const float2 h = p.a_hdr[rm];
    lhs_scale = h.x;
    a_off = (float)__float_as_int(h.y);
  }
  __syncthreads();  // barrier initialisation visible to the waiters
  bool ok = mbar_wait_bounded(&bars[kGemvMaxChunks], 0) && hdr_ok;  // on a timeout or a bad header: keep going (barriers below), store nothing

  // ---- 3. main loop.  The kGemvWarps / pp warps of a panel take its cells round robin; lane = weight row.
  const int wpp = kGemvWarps / p.pp;  // warps per panel
  const int pl = warp / wpp;          // panel (local) of this warp
  const int wr = warp - pl * wpp;     // rank of this warp inside its panel's group
  float acc[M_MAX];
#pragma unroll
  for (int m = 0; m < M_MAX; ++m) acc[m] = 0.0f;
  // One cell: 16-byte load of the lane's row, masks, dp4a on two independent chains, scale, FMA.
  auto do_cell = [&](int c, int lin) {
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
      if (M_MAX == 1 || m < p.m) {
        const uint8_t* rec = abuf + ((size_t)m * p.cells_per_slice + c) * kActRecordBytes;
        const int4 alo = *reinterpret_cast<const int4*>(rec);
        const int4 ahi = *reinterpret_cast<const int4*>(rec + 16);
        int ia = *reinterpret_cast<const int*>(rec + 32);  // -8 * sum(a_q): nibbles are q+8
        int ib = 0;
        ia = __dp4a(alo.x, lo0, ia);
        ib = __dp4a(ahi.x, hi0, ib);
        ia = __dp4a(alo.y, lo1, ia);
        ib = __dp4a(ahi.y, hi1, ib);
        ia = __dp4a(alo.z, lo2, ia);
        ib = __dp4a(ahi.z, hi2, ib);
        ia = __dp4a(alo.w, lo3, ia);
        ib = __dp4a(ahi.w, hi3, ib);
        acc[m] = fmaf((float)(ia + ib), s, acc[m]);
      }
    }
  };
  if (pl < npanels && ok) {
    int ready_chunk = -1;  // each chunk barrier is waited for at most once per warp
    auto need = [&](int lin) {
      const int chunk = lin >> p.chunk_shift;
      for (; ready_chunk < chunk && ok; ++ready_chunk) ok = mbar_wait_bounded(&bars[ready_chunk + 1], 0);
    };
    int c = wr;
    for (; c + wpp < ncells && ok; c += 2 * wpp) {  // two independent cells per trip
      const int lin0 = pl * ncells + c, lin1 = lin0 + wpp;
      need(lin1);
      if (!ok) break;
      do_cell(c, lin0);
      do_cell(c + wpp, lin1);
    }
    if (c < ncells && ok) {
      const int lin0 = pl * ncells + c;
      need(lin0);
      if (ok) do_cell(c, lin0);
    }
  }

  // ---- 4. warps -> CTA partials in shared memory
#pragma unroll
  for (int m = 0; m < M_MAX; ++m) red[(warp * M_MAX + m) * 32 + lane] = acc[m];
  __syncthreads();
  if (!hdr_ok && tid == 0) atomicOr(&g_device_status, kDevStatusBadHeader);

  // ---- 5. reduction + epilogue.  Warp rm (< M_MAX) finishes activation row rm for every panel of the CTA.
  if (p.split > 1) {
    cluster_wait();  // every CTA of the cluster has started
    // pp == 1 here: one panel, one partial per (row, lane)
    if (rm < M_MAX) {
      float part = 0.0f;
#pragma unroll
      for (int w = 0; w < kGemvWarps; ++w) part += red[(w * M_MAX + rm) * 32 + lane];
      st_cluster_f32(map_to_cta(&cred[((int)rank * M_MAX + rm) * 32 + lane], 0), part);
    }
    cluster_sync_all();
    if (rank != 0) return;
  }
  if (rm < M_MAX && rm < p.m && ok && hdr_ok) {
    const float* zsum = reinterpret_cast<const float*>(pr.tiled + pr.zsum_off);
    const float* bias = reinterpret_cast<const float*>(pr.tiled + pr.bias_off);
    for (int q = 0; q < npanels; ++q) {
      const int n_pad = (panel0 + q) * kPanelRows + lane;  // always inside the padded per-row arrays
      const float zs = zsum[n_pad], bs = bias[n_pad];
      float part = 0.0f;
      if (p.split > 1) {
        for (int r = 0; r < p.split; ++r) part += cred[(r * M_MAX + rm) * 32 + lane];
      } else {
        for (int w = q * wpp; w < (q + 1) * wpp; ++w) part += red[(w * M_MAX + rm) * 32 + lane];
      }
      if (n_pad < pr.n) {
        float v = fmaf(a_off, zs, part);
        v = fmaf(v, lhs_scale, bs);
        pr.y[(size_t)rm * pr.ldy + n_pad] = clamp_flt_max(v);
      }
    }
  }
}

// ---- host side ---------------------------------------------------------------------------------
struct GemvPlan {
  int split, cells_per_slice, pp, chunk_shift;
  size_t smem;
};

// total_panels: panels of all problems of the launch together.
static bool gemv_make_plan(int m_max, int num_groups, int total_panels, GemvPlan* plan) {
  // Everything a CTA does is serialized behind its own prologue, so the whole grid should be
  // resident at once: at most kGemvCtasPerSm CTAs per SM (registers), i.e. one wave of 592.  Small
  // matrices are split along K (cluster) until they have about that many CTAs; big ones give
  // each CTA several panels.
  int split = 1, pp = 1;
  auto cps = [&](int s) { return (num_groups + s - 1) / s; };
  const int target = kGemvCtasPerSm * 148;
  if (total_panels > target) {
    while (pp < 8 && (total_panels + pp - 1) / pp > target && (size_t)(pp * 2) * num_groups * kCellBytes <= 96 * 1024)
      pp *= 2;
  } else {
    while (split < kGemvMaxSplit && total_panels * (split + 1) <= target && cps(split + 1) >= 6) ++split;
  }
  // a slice larger than ~64 KB: split further if possible
  while (split < kGemvMaxSplit && pp == 1 && (size_t)cps(split) * kCellBytes > 64 * 1024) ++split;
  int cells = cps(split);
  split = (num_groups + cells - 1) / cells;  // drop empty trailing slices
  const int total_cells = pp * cells;
  int shift = 2;
  while (((total_cells + (1 << shift) - 1) >> shift) > kGemvMaxChunks) ++shift;
  const GemvSmem L = gemv_smem_layout(m_max, pp, cells);
  if (L.total > 200 * 1024) return false;
  plan->split = split;
  plan->cells_per_slice = cells;
  plan->pp = pp;
  plan->chunk_shift = shift;
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
cudaError_t launch_w4a32_gemv_grouped(const uint8_t* a_rec, const float2* a_hdr, int m, int k, int count,
                                      const void* const* tiled, float* const* y, const int* n, const int* ldy,
                                      int use_pdl, cudaStream_t stream) {
  if (count < 1 || count > kGemvMaxProblems || m < 1 || m > kGemvMaxM) return cudaErrorInvalidValue;
  const int num_groups = (k + kGroup - 1) / kGroup;
  const int m_max = m <= 1 ? 1 : (m <= 2 ? 2 : 4);
  int total_panels = 0;
  for (int i = 0; i < count; ++i) total_panels += (n[i] + kPanelRows - 1) / kPanelRows;
  GemvPlan plan;
  if (!gemv_make_plan(m_max, num_groups, total_panels, &plan)) return cudaErrorInvalidValue;
  GemvParams prm = {};
  prm.a_rec = a_rec;
  prm.a_hdr = a_hdr;
  prm.m = m;
  prm.k = k;
  prm.num_groups = num_groups;
  prm.cells_per_slice = plan.cells_per_slice;
  prm.split = plan.split;
  prm.pp = plan.pp;
  prm.chunk_shift = plan.chunk_shift;
  prm.use_pdl = use_pdl & 1;
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

bool w4a32_gemv_supported(int m, int k, int n) {
  if (m < 1 || m > kGemvMaxM) return false;
  GemvPlan plan;
  return gemv_make_plan(m <= 1 ? 1 : (m <= 2 ? 2 : 4), (k + kGroup - 1) / kGroup, (n + kPanelRows - 1) / kPanelRows,
                        &plan);
}

}  // namespace mllmb200
