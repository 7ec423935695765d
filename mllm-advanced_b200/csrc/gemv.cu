// Streaming W4A32 GEMV for decode (M <= 4 activation rows), sm_100a.
//
// One CTA owns one 32-row panel of the weight matrix and one contiguous slice of its K-groups.
// The slice is a contiguous byte range in the tile layout (layout.h), so thread 0 moves all of it
// into shared memory with a handful of bulk copies (cp.async.bulk, each completing on its own
// mbarrier) issued before anything else: every byte the CTA will ever need is in flight from the
// first instructions, which is what a kernel whose whole input is a few tens of KB per SM needs
// to approach the HBM roofline.  While the copies fly, the CTA quantizes the activation row(s)
// (dynamic asymmetric int8, reference: tests/Arm/KaiLinearTest.hpp:163-230) into shared memory in
// the byte order the nibble unpack produces.  Then each warp takes cells (panel x K-group) round
// robin: lane = weight row, one 16-byte shared load = the row's 32 nibbles, masks split them into
// two byte vectors, eight dp4a accumulate the exact int32 group sum, and one fp32 FMA applies the
// group scale.  Partial sums meet in shared memory (fixed order); when K is split over the CTAs of
// a thread-block cluster the per-CTA partials are written into the cluster leader's shared memory
// and summed there in rank order, so the result is deterministic.
//
//   y[m,n] = lhs_scale[m] * ( sum_b float(sum_{k in b} a_q[m,k] * w[n,k]) * s[n,b]  +  a_off[m] * zsum[n] ) + bias[n]
//
// which equals the reference expression (KaiLinearTest.hpp:338-377) with the zero-point term
// a_off * sum_k w[n,k] s[n,b] taken out of the integer sum (zsum is precomputed per row at repack).
#include "device_common.cuh"

namespace mllmb200 {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvMaxChunks = 8;
constexpr int kGemvMaxSplit = 8;

struct GemvParams {
  const float* x;
  const uint8_t* tiled;  // TiledHeader at offset 0
  float* y;
  int m, k, n, ldx, ldy;
  int num_groups;        // K-groups per row
  int cells_per_cta;     // K-groups per CTA slice
  int split;             // CTAs per panel (= cluster size)
  int cells_per_chunk;   // cells per bulk copy
  int use_pdl;
  size_t zsum_off, bias_off;  // byte offsets of the per-row arrays inside the tiled buffer
};

// shared memory carve-up (dynamic):
//   [0, 64)                                  kGemvMaxChunks mbarriers
//   [64, 64+256)                             min/max scratch (64 floats)
//   [320, 320+64)                            row params: M_MAX x {scale0, recip, nzp, pad}
//   wbuf   cells_per_cta * 576               weights (bulk copy destination, 128-byte aligned)
//   abuf   M_MAX * cells_per_cta * 48        permuted int8 activations + (-8 * group sum)
//   red    kGemvWarps * M_MAX * 32 floats    cross-warp partials
//   cred   kGemvMaxSplit * M_MAX * 32 floats cross-CTA partials (leader only)
__host__ __device__ inline size_t gemv_smem_bytes(int m_max, int cells_per_cta) {
  size_t off = 384;
  off += (size_t)cells_per_cta * kCellBytes;
  off += (size_t)m_max * cells_per_cta * kActRecordBytes;
  off += (size_t)kGemvWarps * m_max * 32 * 4;
  off += (size_t)kGemvMaxSplit * m_max * 32 * 4;
  return off + 128;
}

template <int M_MAX>
__global__ void __launch_bounds__(kGemvThreads) w4a32_gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // align the carve-up to 128 bytes whatever the runtime gives us
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  float* mm_scratch = reinterpret_cast<float*>(smem + 64);
  float* rowp = reinterpret_cast<float*>(smem + 320);
  uint8_t* wbuf = smem + 384;
  uint8_t* abuf = wbuf + (size_t)p.cells_per_cta * kCellBytes;
  float* red = reinterpret_cast<float*>(abuf + (size_t)M_MAX * p.cells_per_cta * kActRecordBytes);
  float* cred = red + kGemvWarps * M_MAX * 32;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int panel = blockIdx.x / p.split;
  const int slice = blockIdx.x % p.split;
  const int g0 = slice * p.cells_per_cta;                       // first K-group of this CTA
  const int ncells = min(p.cells_per_cta, p.num_groups - g0);   // >= 1 by construction
  const int nchunks = (ncells + p.cells_per_chunk - 1) / p.cells_per_chunk;

  const TiledHeader* hdr = reinterpret_cast<const TiledHeader*>(p.tiled);
  const uint8_t* cells = p.tiled + sizeof(TiledHeader);

  // ---- 1. get every weight byte of this CTA in flight
  if (tid == 0) {
    for (int c = 0; c < nchunks; ++c) mbar_init(&bars[c], 1);
    mbar_fence_init();
    const uint8_t* src = cells + ((size_t)panel * p.num_groups + g0) * kCellBytes;
    for (int c = 0; c < nchunks; ++c) {
      const int c0 = c * p.cells_per_chunk;
      const uint32_t bytes = (uint32_t)(min(p.cells_per_chunk, ncells - c0) * kCellBytes);
      mbar_arrive_expect_tx(&bars[c], bytes);
      bulk_g2s(wbuf + (size_t)c0 * kCellBytes, src + (size_t)c0 * kCellBytes, bytes, &bars[c]);
    }
  }
  // the next kernel in the stream may start fetching its own (constant) weights now
  if (p.use_pdl) pdl_launch_dependents();
  const uint32_t scale_mode = hdr->scale_mode;
  const bool hdr_ok = hdr->magic == kTiledMagic && hdr->n == (uint32_t)p.n && hdr->k == (uint32_t)p.k;
  if (!hdr_ok && tid == 0) atomicOr(&g_device_status, kDevStatusBadHeader);
  // per-row constants for the epilogue, fetched now so their latency hides behind the main loop
  const int rm = tid >> 5;  // activation row this thread finishes in the reduction
  float row_zsum = 0.0f, row_bias = 0.0f;
  if (rm < M_MAX) {
    const int n_pad = panel * kPanelRows + lane;  // always inside the padded arrays
    row_zsum = reinterpret_cast<const float*>(p.tiled + p.zsum_off)[n_pad];
    row_bias = reinterpret_cast<const float*>(p.tiled + p.bias_off)[n_pad];
  }

  // the weights are constant; the activations may come from the kernel before us
  if (p.use_pdl) pdl_wait_prior();

  // ---- 2. quantize the activation rows (all of K for min/max, this CTA's slice for the values)
#pragma unroll
  for (int m = 0; m < M_MAX; ++m) {
    if (m < p.m) {
      const float* row = p.x + (size_t)m * p.ldx;
      float mn, mx;
      block_row_minmax(row, p.k, mm_scratch, mn, mx);
      const ActQuantParams q = act_quant_params(mn, mx);
      if (tid == 0) {
        rowp[m * 4 + 0] = q.recip_scale;
        rowp[m * 4 + 1] = (float)(-q.nzp);
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
          uint32_t* rec = reinterpret_cast<uint32_t*>(abuf + ((size_t)m * p.cells_per_cta + c) * kActRecordBytes);
          rec[i] = lo;
          rec[4 + i] = hi;
          if (i == 0) rec[8] = (uint32_t)(-8 * s);
        }
      }
    }
  }
  __syncthreads();

  // ---- 3. cells round robin over warps; lane = weight row
  float acc[M_MAX];
#pragma unroll
  for (int m = 0; m < M_MAX; ++m) acc[m] = 0.0f;
  bool ok = hdr_ok;
  int ready_chunk = -1;
  for (int c = warp; c < ncells && ok; c += kGemvWarps) {
    const int chunk = c / p.cells_per_chunk;
    if (chunk != ready_chunk) {
      ok = mbar_wait_bounded(&bars[chunk], 0);
      ready_chunk = chunk;
      if (!ok) break;
    }
    const uint8_t* cell = wbuf + (size_t)c * kCellBytes;
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
        const uint8_t* rec = abuf + ((size_t)m * p.cells_per_cta + c) * kActRecordBytes;
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

  // ---- 4. warps -> CTA partial (fixed order)
#pragma unroll
  for (int m = 0; m < M_MAX; ++m) red[(warp * M_MAX + m) * 32 + lane] = acc[m];
  __syncthreads();
  float part = 0.0f;
  if (rm < M_MAX) {
#pragma unroll
    for (int w = 0; w < kGemvWarps; ++w) part += red[(w * M_MAX + rm) * 32 + lane];
  }

  // ---- 5. CTAs of the cluster -> leader (fixed order), then the epilogue
  if (p.split > 1) {
    const uint32_t rank = cluster_ctarank();
    if (rm < M_MAX) {
      const uint32_t dst = map_to_cta(&cred[(rank * M_MAX + rm) * 32 + lane], 0);
      st_cluster_f32(dst, part);
    }
    cluster_sync_all();
    if (rank != 0) return;
    if (rm < M_MAX) {
      part = 0.0f;
      for (int r = 0; r < p.split; ++r) part += cred[(r * M_MAX + rm) * 32 + lane];
    }
  }
  if (rm < M_MAX && rm < p.m && ok) {
    const int n = panel * kPanelRows + lane;
    if (n < p.n) {
      const float lhs_scale = rowp[rm * 4 + 0], a_off = rowp[rm * 4 + 1];
      float v = fmaf(a_off, row_zsum, part);
      v = fmaf(v, lhs_scale, row_bias);
      p.y[(size_t)rm * p.ldy + n] = clamp_flt_max(v);
    }
  }
}

// ---- host launcher -------------------------------------------------------------------------
struct GemvPlan {
  int split, cells_per_cta, cells_per_chunk;
  size_t smem;
};

inline bool gemv_make_plan(int m_max, int num_groups, int num_panels, GemvPlan* plan) {
  // Start from one CTA per panel and split K while a CTA's slice is larger than ~32 KB or the grid
  // is too small to keep 148 SMs busy, as long as a slice keeps at least 4 K-groups.
  int split = 1;
  auto cpc = [&](int s) { return (num_groups + s - 1) / s; };
  while (split < kGemvMaxSplit && cpc(split * 2) >= 4 &&
         (cpc(split) * kCellBytes > 32 * 1024 || (long long)num_panels * split < 2 * 148))
    split *= 2;
  int cells = cpc(split);
  split = (num_groups + cells - 1) / cells;  // drop empty trailing slices
  const size_t smem = gemv_smem_bytes(m_max, cells);
  if (smem > 200 * 1024) return false;
  plan->split = split;
  plan->cells_per_cta = cells;
  plan->cells_per_chunk = (cells + kGemvMaxChunks - 1) / kGemvMaxChunks;
  plan->smem = smem;
  return true;
}

template <int M_MAX>
static cudaError_t launch_gemv_t(const GemvParams& prm, const GemvPlan& plan, int num_panels, cudaStream_t stream) {
  static bool configured[64] = {};  // per device, per M_MAX instantiation
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (plan.smem > 48 * 1024 && !(dev >= 0 && dev < 64 && configured[dev])) {
    e = cudaFuncSetAttribute(w4a32_gemv_kernel<M_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(200 * 1024 + 512));
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(num_panels * plan.split), 1, 1);
  cfg.blockDim = dim3(kGemvThreads, 1, 1);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (plan.split > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = (unsigned)plan.split;
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

// Returns cudaErrorInvalidValue when the shape has no GEMV plan (caller falls back to the GEMM path).
cudaError_t launch_w4a32_gemv(const float* x, const void* tiled, float* y, int m, int k, int n, int ldx, int ldy,
                              int use_pdl, cudaStream_t stream) {
  const int num_groups = (k + kGroup - 1) / kGroup;
  const int num_panels = (n + kPanelRows - 1) / kPanelRows;
  const int m_max = m <= 1 ? 1 : (m <= 2 ? 2 : 4);
  GemvPlan plan;
  if (m > 4 || !gemv_make_plan(m_max, num_groups, num_panels, &plan)) return cudaErrorInvalidValue;
  GemvParams prm;
  prm.x = x;
  prm.tiled = static_cast<const uint8_t*>(tiled);
  prm.y = y;
  prm.m = m;
  prm.k = k;
  prm.n = n;
  prm.ldx = ldx;
  prm.ldy = ldy;
  prm.num_groups = num_groups;
  prm.cells_per_cta = plan.cells_per_cta;
  prm.split = plan.split;
  prm.cells_per_chunk = plan.cells_per_chunk;
  prm.use_pdl = use_pdl;
  const TiledHeader th = make_tiled_header(n, k, 0, 0);
  prm.zsum_off = th.zsum_off;
  prm.bias_off = th.bias_off;
  switch (m_max) {
    case 1: return launch_gemv_t<1>(prm, plan, num_panels, stream);
    case 2: return launch_gemv_t<2>(prm, plan, num_panels, stream);
    default: return launch_gemv_t<4>(prm, plan, num_panels, stream);
  }
}

bool w4a32_gemv_supported(int m, int k, int n) {
  if (m < 1 || m > 4) return false;
  GemvPlan plan;
  return gemv_make_plan(m <= 1 ? 1 : (m <= 2 ? 2 : 4), (k + kGroup - 1) / kGroup, (n + kPanelRows - 1) / kPanelRows,
                        &plan);
}

}  // namespace mllmb200
