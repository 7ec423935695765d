// tcgen05 (5th-generation tensor core) W4A32 GEMM for prefill-sized M, sm_100a.
//
// The reference quantizes activations to int8 per row and accumulates every 32-wide K-group in
// int32 before applying that group's weight scale (tests/Arm/KaiLinearTest.hpp:338-373 of the
// reference project).  This kernel keeps exactly that arithmetic on the tensor cores:
// tcgen05.mma kind::i8 (int8 x int8 -> int32 in tensor memory), one MMA per K-group (K = 32 is the
// instruction's K for 8-bit types) with a fresh accumulator, and an epilogue that converts the
// exact group sums to fp32 and applies s[n,b] with one FMA per element, in K order.
//
// Operand roles are swapped with respect to the usual GEMM so that the per-row weight scale is a
// per-thread scalar in the epilogue:
//   A (M_mma = 128) = 128 weight rows (4 panels of the tile layout), int8 = 16 * (nibble - 8),
//                     written to shared memory by the dequant warps from the raw cells;
//   B (N_mma = NT)  = NT activation rows, int8, pre-arranged by the quantization kernel in the
//                     canonical K-major core-matrix layout, so one bulk copy per K-group delivers a
//                     ready operand (no tensor map needed);
//   D (tensor memory) = [128 lanes = weight rows] x [NT columns = activation rows], int32.
// Both operands use the same permutation of k inside a K-group (the order the nibble masks
// produce), which leaves every dot product unchanged.
//
// Warp roles (704 threads, one CTA per SM):
//   warps 0-15  epilogue: warp w reads TMEM lanes 32*(w%4).. (its quadrant) and columns
//               (w/4)*NT/4 ..; accumulators stay in registers for the whole K loop
//   warps 16-19 dequant: thread j expands weight row j of the tile, 4 K-groups per stage
//   warp 20     producer: bulk copies (cp.async.bulk) of raw weight cells and activation blocks
//   warp 21     MMA issuer (one elected lane) and tensor-memory allocation
// Shared memory: 8 stages of loaded data {raw cells 9 KB, B operand NT*128 B} and 3 stages of the
// dequantized A operand (16 KB each).  Tensor memory:
// all 512 columns, as 512/(4*NT) batches of 4 accumulators (one per K-group of a stage); a batch
// is handed to the epilogue with one commit and handed back with one arrive per warp, so the
// MMA -> epilogue -> MMA round trip (thousands of cycles) is paid once per 4 K-groups and several
// batches are in flight.  NT is 64 or 32.  Every mbarrier wait is bounded (device_common.cuh).
#include "device_common.cuh"
#include "tcgen05_common.cuh"

namespace mllmb200 {

constexpr int kTcEpiWarps = 16;     // 4 per TMEM lane quadrant, each a quarter of the columns
constexpr int kTcThreads = (kTcEpiWarps + 6) * 32;  // + 4 dequant warps + producer + MMA issuer
constexpr int kTcStages = 8;        // shared-memory stages of loaded data (raw weight cells + B operand): deep, to cover HBM latency
constexpr int kTcAStages = 3;       // shared-memory stages of the dequantized A operand (produced on chip: shallow)
constexpr int kTcGroupsPerStage = 4;  // K-groups (of 32) per stage
constexpr int kTcTileRows = 128;    // weight rows per CTA (= 4 panels)
constexpr int kTcTmemCols = 512;    // all of tensor memory: accumulator batches of 4 K-groups x NT columns

struct TcParams {
  const uint8_t* a_blocks;  // activations, [num_groups][m8_pad][256 bytes] canonical blocks
  const float2* a_hdr;      // [m] {lhs_scale, a_off bits}
  const uint8_t* tiled;     // weights (TiledHeader at offset 0)
  float* y;
  int m, n, k, ldy;
  int num_groups, num_panels, m8_pad;
  size_t zsum_off, bias_off;
};

template <int NT>
struct TcSmem {
  static constexpr int kRawBytes = 4 * kTcGroupsPerStage * kCellBytes;  // 9216
  static constexpr int kBBytes = kTcGroupsPerStage * NT * 32;
  static constexpr int kABytes = kTcGroupsPerStage * kTcTileRows * 32;  // 16384
  static constexpr int kStageBytes = kRawBytes + kBBytes;  // one loaded stage
  static constexpr int kBarBytes = 256;
  static constexpr int kAOffset = kBarBytes + kTcStages * kStageBytes;
  static constexpr int kTotal = kAOffset + kTcAStages * kABytes + 1024;  // + alignment slack
};

template <int NT>
__global__ void __launch_bounds__(kTcThreads, 1) w4a32_gemm_tc_kernel(const TcParams p) {
  using S = TcSmem<NT>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  if (!tiled_header_ok_cta(p.tiled, p.n, p.k)) return;  // before any copy, barrier or tensor-memory allocation
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem);  // [kTcStages]
  uint64_t* mma_done = raw_full + kTcStages;               // [kTcStages] the MMAs of a stage completed
  uint64_t* a_full = mma_done + kTcStages;                 // [kTcAStages]
  // accumulators are handed over in batches of one shared-memory stage (4 K-groups): one barrier
  // round trip per 4 MMAs instead of per MMA, and kSlots batches in flight
  constexpr int kSlots = kTcTmemCols / (kTcGroupsPerStage * NT);
  uint64_t* acc_empty = a_full + kTcAStages;               // [kSlots]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_empty + kSlots);
  uint8_t* stages = smem + S::kBarBytes;
  uint8_t* a_stages = smem + S::kAOffset;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile_n = blockIdx.x;  // 128 weight rows
  const int tile_m = blockIdx.y;  // NT activation rows
  const int panel0 = tile_n * 4;
  const int m0 = tile_m * NT;
  const int k_tiles = (p.num_groups + kTcGroupsPerStage - 1) / kTcGroupsPerStage;

  if (tid == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&mma_done[s], 1);
    }
    for (int s = 0; s < kTcAStages; ++s) mbar_init(&a_full[s], 128);
    for (int t = 0; t < kSlots; ++t) {
      mbar_init(&acc_empty[t], kTcEpiWarps);  // one arrival per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == kTcEpiWarps + 5) {
    tmem_alloc(tmem_base_slot, (uint32_t)kTcTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == kTcEpiWarps + 4) {
    // ------------------------------------------------------------ producer
    // lanes 0-3 copy one panel's cells each, lanes 4-7 one K-group's activation block each: the eight
    // copies of a stage are issued side by side (one thread issuing them all was the kernel's bottleneck)
    const int np = min(4, p.num_panels - panel0);
    for (int it = 0; it < k_tiles; ++it) {
      const int s = it % kTcStages;
      const uint32_t ph = (uint32_t)(it / kTcStages) & 1u;
      // warp-uniform outcome: a timed-out lane must not leave the others at the __syncwarp below
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(&mma_done[s], ph ^ 1u))) break;
      const int g0 = it * kTcGroupsPerStage;
      const int ng = min(kTcGroupsPerStage, p.num_groups - g0);
      uint8_t* st = stages + (size_t)s * S::kStageBytes;
      if (lane == 0) mbar_arrive_expect_tx(&raw_full[s], (uint32_t)(np * ng * kCellBytes + ng * NT * 32));
      __syncwarp();
      if (lane < np) {
        bulk_g2s(st + lane * kTcGroupsPerStage * kCellBytes,
                 p.tiled + sizeof(TiledHeader) + ((size_t)(panel0 + lane) * p.num_groups + g0) * kCellBytes,
                 (uint32_t)(ng * kCellBytes), &raw_full[s]);
      } else if (lane >= 4 && lane < 4 + ng) {
        const int g = lane - 4;
        bulk_g2s(st + S::kRawBytes + g * NT * 32, p.a_blocks + ((size_t)(g0 + g) * p.m8_pad + (m0 >> 3)) * 256,
                 (uint32_t)(NT * 32), &raw_full[s]);
      }
    }
  } else if (warp == kTcEpiWarps + 5) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: D = s32, A = B = signed int8, both K-major, N = NT, M = 128
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) | ((128u >> 4) << 24);
      bool ok = true;
      for (int it = 0; it < k_tiles && ok; ++it) {
        const int s = it % kTcStages;
        const uint32_t ph = (uint32_t)(it / kTcStages) & 1u;
        const int slot = it % kSlots;
        const int sa = it % kTcAStages;
        ok = mbar_wait_bounded(&raw_full[s], ph) && mbar_wait_bounded(&a_full[sa], (uint32_t)(it / kTcAStages) & 1u) &&
             mbar_wait_bounded(&acc_empty[slot], ((uint32_t)(it / kSlots) & 1u) ^ 1u);
        if (!ok) break;
        tc_fence_after();
        const int ng = min(kTcGroupsPerStage, p.num_groups - it * kTcGroupsPerStage);
        uint8_t* st = stages + (size_t)s * S::kStageBytes;
        const uint32_t b_addr = smem_u32(st + S::kRawBytes), a_addr = smem_u32(a_stages + (size_t)sa * S::kABytes);
        const uint64_t a_desc = make_kmajor_desc(a_addr, 128, 256), b_desc = make_kmajor_desc(b_addr, 128, 256);
#pragma unroll
        for (int g = 0; g < kTcGroupsPerStage; ++g) {
          if (g >= ng) break;
          // the start-address field counts 16-byte units: the next K-group is a constant further on
          tc_mma_i8(tmem_base + (uint32_t)((slot * kTcGroupsPerStage + g) * NT),
                    a_desc + (uint64_t)(g * (kTcTileRows * 32 / 16)), b_desc + (uint64_t)(g * (NT * 32 / 16)), idesc);
        }
        // one commit per K-tile: its accumulators are complete (epilogue), its loaded stage may be
        // refilled (producer) and its A stage rewritten (dequant); waiters pick the phase they need
        tc_commit(&mma_done[s]);
      }
    }
  } else if (warp >= kTcEpiWarps) {
    // ------------------------------------------------------------ dequant: thread j = weight row j of the tile
    const int j = tid - kTcEpiWarps * 32;
    const int q = j >> 5, r = j & 31;  // panel of the tile, row in the panel
    const bool have_panel = panel0 + q < p.num_panels;
    bool ok = true;
    for (int it = 0; it < k_tiles && ok; ++it) {
      const int s = it % kTcStages;
      const uint32_t ph = (uint32_t)(it / kTcStages) & 1u;
      ok = mbar_wait_bounded(&raw_full[s], ph);
      const int sa = it % kTcAStages;
      if (ok && it >= kTcAStages) {  // the A stage is free once the MMAs of K-tile it - kTcAStages are done
        const int prev = it - kTcAStages;
        ok = mbar_wait_bounded(&mma_done[prev % kTcStages], (uint32_t)(prev / kTcStages) & 1u);
      }
      if (!ok) break;
      const int ng = min(kTcGroupsPerStage, p.num_groups - it * kTcGroupsPerStage);
      uint8_t* st = stages + (size_t)s * S::kStageBytes;
      const uint8_t* raw = st + q * kTcGroupsPerStage * kCellBytes;
      uint8_t* a_out = a_stages + (size_t)sa * S::kABytes + (j >> 3) * 256 + (j & 7) * 16;
#pragma unroll
      for (int g = 0; g < kTcGroupsPerStage; ++g) {
        if (g >= ng) break;
        uint4 w = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
        if (have_panel) w = *reinterpret_cast<const uint4*>(raw + g * kCellBytes + r * 16);
        // byte = 16 * (nibble - 8) as signed int8: low nibbles shifted up, high nibbles in place, flip bit 7
        uint4 c0, c1;
        c0.x = ((w.x << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
        c0.y = (w.x & 0xF0F0F0F0u) ^ 0x80808080u;
        c0.z = ((w.y << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
        c0.w = (w.y & 0xF0F0F0F0u) ^ 0x80808080u;
        c1.x = ((w.z << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
        c1.y = (w.z & 0xF0F0F0F0u) ^ 0x80808080u;
        c1.z = ((w.w << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
        c1.w = (w.w & 0xF0F0F0F0u) ^ 0x80808080u;
        *reinterpret_cast<uint4*>(a_out + g * kTcTileRows * 32) = c0;        // K chunk 0
        *reinterpret_cast<uint4*>(a_out + g * kTcTileRows * 32 + 128) = c1;  // K chunk 1
      }
      fence_proxy_async_smem();  // make the generic-proxy stores visible to the tensor core
      mbar_arrive(&a_full[sa]);
    }
  } else {
    // ------------------------------------------------------------ epilogue
    constexpr int CW = NT / 4;  // columns per warp
    const int quad = warp & 3, half = warp >> 2;  // half = which quarter of the columns
    const int row = quad * 32 + lane;                // weight row inside the tile == TMEM lane
    const int n = tile_n * kTcTileRows + row;
    const bool have_panel = panel0 + quad < p.num_panels;
    const TiledHeader* hdr = reinterpret_cast<const TiledHeader*>(p.tiled);
    const uint32_t scale_mode = hdr->scale_mode;
    const uint8_t* scale_ptr = p.tiled + sizeof(TiledHeader) + (size_t)(panel0 + quad) * p.num_groups * kCellBytes +
                               kCellNibbleBytes + lane * 2;
    float acc[CW];
#pragma unroll
    for (int c = 0; c < CW; ++c) acc[c] = 0.0f;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(half * CW);
    // Group scales come from global memory (L2: the producer just fetched the same cells).  They are
    // requested kScaleAhead groups early so that their latency never sits in front of the math.
    constexpr int kScaleAhead = 8;
    uint32_t sraw[kScaleAhead];
#pragma unroll
    for (int i = 0; i < kScaleAhead; ++i)
      sraw[i] = (have_panel && i < p.num_groups) ? *reinterpret_cast<const uint16_t*>(scale_ptr + (size_t)i * kCellBytes) : 0u;
    bool ok = true;
    static_assert(kScaleAhead == 2 * kTcGroupsPerStage, "the scale ring covers two batches");
    for (int it2 = 0; it2 < k_tiles && ok; it2 += 2) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int it = it2 + h;
        if (it >= k_tiles || !ok) break;
        const int slot = it % kSlots;
        ok = mbar_wait_bounded(&mma_done[it % kTcStages], (uint32_t)(it / kTcStages) & 1u);
        if (!ok) break;
        tc_fence_after();
        const int ng = min(kTcGroupsPerStage, p.num_groups - it * kTcGroupsPerStage);
        // kLoadGroups accumulators into registers per wait (register budget: 704 threads share the
        // file); after the batch's last load its slot goes back to the MMA issuer
        constexpr int kLoadGroups = CW == 16 ? 2 : 4;
#pragma unroll
        for (int g0 = 0; g0 < kTcGroupsPerStage; g0 += kLoadGroups) {
          if (g0 >= ng) break;
          uint32_t v[kLoadGroups][CW];
#pragma unroll
          for (int j = 0; j < kLoadGroups; ++j)
            if (g0 + j < ng) tmem_ld_cols<CW>(lane_addr + (uint32_t)((slot * kTcGroupsPerStage + g0 + j) * NT), v[j]);
          tmem_ld_wait();
          if (g0 + kLoadGroups >= ng) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[slot]);
          }
#pragma unroll
          for (int j = 0; j < kLoadGroups; ++j) {
            const int g = g0 + j;
            if (g >= ng) break;
            const int u = h * kTcGroupsPerStage + g;
            const int cnt = it * kTcGroupsPerStage + g;
            // group scale / 16 (the A operand carries 16 * weight); exact: a power-of-two factor
            const float s16 = decode_scale(sraw[u], scale_mode) * 0.0625f;
            const int nxt = cnt + kScaleAhead;
            sraw[u] = (have_panel && nxt < p.num_groups) ? *reinterpret_cast<const uint16_t*>(scale_ptr + (size_t)nxt * kCellBytes) : 0u;
            // |group sum| <= 16 * 32 * 128 * 8 < 2^24: the int32 -> fp32 conversion is exact
#pragma unroll
            for (int i = 0; i < CW; ++i) acc[i] = fmaf((float)(int)v[j][i], s16, acc[i]);
          }
        }
      }
    }
    // y[m, n] = lhs_scale[m] * (acc + a_off[m] * zsum[n]) + bias[n]; lanes = consecutive n: coalesced per m
    if (ok && n < p.n) {
      const int n_pad = n;  // inside the padded per-row arrays
      const float zs = reinterpret_cast<const float*>(p.tiled + p.zsum_off)[n_pad];
      const float bs = reinterpret_cast<const float*>(p.tiled + p.bias_off)[n_pad];
#pragma unroll
      for (int c = 0; c < CW; ++c) {
        const int m = m0 + half * CW + c;
        if (m < p.m) {
          const float2 h = p.a_hdr[m];
          float v = fmaf((float)__float_as_int(h.y), zs, acc[c]);
          v = fmaf(v, h.x, bs);
          p.y[(size_t)m * p.ldy + n] = clamp_flt_max(v);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kTcEpiWarps + 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)kTcTmemCols);
  }
}

template <int NT>
static cudaError_t launch_tc_t(const TcParams& prm, cudaStream_t stream) {
  using S = TcSmem<NT>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (!(dev >= 0 && dev < 64 && configured[dev])) {
    e = cudaFuncSetAttribute(w4a32_gemm_tc_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid((unsigned)((prm.num_panels + 3) / 4), (unsigned)((prm.m + NT - 1) / NT), 1);
  w4a32_gemm_tc_kernel<NT><<<grid, kTcThreads, S::kTotal, stream>>>(prm);
  return cudaGetLastError();
}

// Rows of the activation block array are padded to a multiple of the largest NT.
int w4a32_gemm_tc_m_pad(int m) { return (m + 63) / 64 * 64; }

bool w4a32_gemm_tc_supported(int m, int k, int n) {
  // one CTA per SM holds 128 KB+ of shared memory and all tensor memory it allocates; any K, any N.
  // Below ~17 rows the GEMV / SIMT paths are the better fit.
  return m >= 17 && k >= 1 && n >= 1 && (size_t)((m + 127) / 128) <= 65535;
}

cudaError_t launch_w4a32_gemm_tc(const uint8_t* a_blocks, const float2* a_hdr, const void* tiled, float* y, int m, int k,
                                 int n, int ldy, cudaStream_t stream) {
  TcParams prm;
  prm.a_blocks = a_blocks;
  prm.a_hdr = a_hdr;
  prm.tiled = static_cast<const uint8_t*>(tiled);
  prm.y = y;
  prm.m = m;
  prm.n = n;
  prm.k = k;
  prm.ldy = ldy;
  prm.num_groups = (k + kGroup - 1) / kGroup;
  prm.num_panels = (n + kPanelRows - 1) / kPanelRows;
  prm.m8_pad = w4a32_gemm_tc_m_pad(m) / 8;
  const TiledHeader th = make_tiled_header(n, k, 0, 0);
  prm.zsum_off = th.zsum_off;
  prm.bias_off = th.bias_off;
  // Tile width along the activation rows.  A tile's time is dominated by per-K-tile costs that do
  // not depend on its width (dequantization of the 128 weight rows, copy and MMA issue), measured
  // ~51 us for K = 8192 at either width, so the wide tile wins whenever M has the rows for it.
  const int best_nt = m > 32 ? 64 : 32;
  if (best_nt == 32) return launch_tc_t<32>(prm, stream);
  return launch_tc_t<64>(prm, stream);
}

}  // namespace mllmb200
