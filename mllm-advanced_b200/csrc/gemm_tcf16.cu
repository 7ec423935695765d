// tcgen05 W4A32 GEMM with fp16 operands and fp32 accumulation over ALL of K in tensor memory
// (sm_100a) - the high-throughput prefill path.
//
// The int8 path (gemm_tc.cu) keeps the reference's per-group int32 sums and therefore pays one
// conversion and one FMA per (row, column, K-group) on the CUDA cores, which bounds it far below
// the tensor cores.  Here the group scale moves INTO the weight operand:
//   A[n, k] = fp16( (u[n,k] - 8) * s[n, group(k)] * 2^E )      B[m, k] = fp16( a_q[m, k] + a_off[m] )
// B is exact: |a_q + a_off| <= 255 fits fp16 (so the zero point needs no correction term and nothing
// cancels).  A is exact for bf16-encoded scales (the reference's encoding and the default,
// MLLMB200_SCALE_BF16_TRUNC / _RNE): (u - 8) has at most 3 significant bits, a bf16 scale 8, the
// product at most 11 = what fp16 holds; 2^E (one exponent per matrix, from the largest |scale| recorded
// in the tile header by the repack) keeps the products in fp16's normal range.  Every product a_q * A is
// then exact in fp32, and the only difference to the reference (tests/Arm/KaiLinearTest.hpp:338-377 of
// the reference project) is the order and rounding of the fp32 additions, which the GEMV and SIMT paths
// change as well.  Stated bound: max|diff| <= 1e-3 * rms(y), the bar of every other path; measured
// ~1e-6 * rms.  With fp16-ENCODED scales (MLLMB200_SCALE_FP16: 11 significant bits) the product needs up
// to 14 bits and the HMUL2 below rounds it to 11: a relative error of at most 2^-12 per weight, which
// shows up as about 1.5e-4 * rms(y) per output; stated bound for that mode 2e-3 * rms(y) (the exact
// kernels 1-3 remain available for it).  Scales more than 2^24 below the matrix maximum fall into fp16
// subnormals and lose low bits (contribution < 2^-24 of the largest group's).
//
//   y[m,n] = lhs_scale[m] * 2^-E * sum_k A[n,k] B[m,k] + bias[n]
//
// Tile: 128 weight rows (MMA M, tensor-memory lanes) x NT activation rows (MMA N, columns), one
// accumulator for the whole K loop, one CTA per SM.  Warp roles (576 threads):
//   warps 0-15 dequant: thread = weight row 32 (w % 4) + lane of the tile; the four warps of a row set take turns
//              over the K-groups (16 bytes of nibbles -> 64 bytes of fp16 per K-group: shift / mask-or / one
//              fused multiply-add on pairs of nibbles 16 bits apart) and write the row's 16 columns of the
//              A operand into TENSOR memory with tcgen05.st (256-row tiles: two warps per row set, operand in
//              shared memory in the canonical K-major core-matrix layout); after the loop the same warps run
//              the epilogue (warp w owns tensor-memory lanes 32 (w % 4).. and a quarter of the columns)
//   warp 16    producer: bulk copies (cp.async.bulk) of the raw weight cells (evict-first: each is read once
//              per wave) and of the activation blocks, which act_quant_blocks_f16_kernel already wrote in
//              operand layout
//   warp 17    MMA issuer and tensor-memory owner: the whole warp runs the loop, one elected lane issues
//              (two K=16 instructions per K-group, A from tensor memory, B through a shared-memory descriptor)
// Stages of 2 (NT = 256) or 4 K-groups: a ring of 5-7 loaded-data stages {raw cells, B operand NT*64 B per
// group} in shared memory and up to as many operand stages in tensor-memory columns [NT, 512).  Every wait
// (mbarrier, split-K flag) is bounded.  CTAs are renumbered so that the row tiles of one weight tile are
// dispatched side by side; launches that would fill less than half of the SMs, and the tiles left over after a
// launch's last full wave, split K between two CTAs per output tile.
// Measured at M = 512 on the Qwen2-1.5B layer shapes (cold caches, one launch each): q,k,v grouped 17 us,
// o 17 us, gate+up grouped 36 us, down 34 us; config 4 (28672 x 8192, M = 2048): 0.80 ms = 1202 TFLOP/s.
#include <cuda_fp16.h>

#include "device_common.cuh"
#include "layout_a16.h"
#include "tcgen05_common.cuh"

// Build-time switches (each 1 = the measured choice; 0 restores the form it replaced, for comparisons):
#ifndef MLLMB200_TF_WEIGHT_HINT  // evict-first L2 hint on the weight-cell copies
#define MLLMB200_TF_WEIGHT_HINT 1
#endif
#ifndef MLLMB200_TF_FUSED_DEQUANT  // one fused multiply-add per pair of nibbles (bf16-encoded scales)
#define MLLMB200_TF_FUSED_DEQUANT 1
#endif
#ifndef MLLMB200_TF_SMALL_M  // "fastest" picks this kernel from M = 64 for wide matrices with a short K
#define MLLMB200_TF_SMALL_M 1
#endif
#ifndef MLLMB200_TF_SPLIT_K  // K split in two on short grids and left-over tiles
#define MLLMB200_TF_SPLIT_K 1
#endif
#ifndef MLLMB200_TF_ATM  // dequantized weight operand in tensor memory (128-row tiles)
#define MLLMB200_TF_ATM 1
#endif
#ifndef MLLMB200_TF_ATM_A16  // the same for the W4A16 instantiation (measured: no faster - its fp32 dequant is the bound)
#define MLLMB200_TF_ATM_A16 0
#endif
#ifndef MLLMB200_TF_WIDE  // 256-row tiles (two accumulators, operand in shared memory) where tf_tile_for picks them
#define MLLMB200_TF_WIDE 1
#endif

namespace mllmb200 {

#ifdef MLLMB200_TF_TRACE
extern __device__ unsigned long long* g_gs_trace;  // development build only: clock stamps of one CTA per K-tile
// MLLMB200_TF_TRACE = 1: every stamp; 2: only the MMA warp's (slots 4-6) and the top of the dequant loop (7)
#define TF_STAMP(it, slot) do { if ((MLLMB200_TF_TRACE == 1 || (slot) >= 4) && traced && (it) < 100) g_gs_trace[17 + (it) * 8 + (slot)] = (unsigned long long)clock64(); } while (0)
#define TF_STAMP0(slot) do { if (traced) g_gs_trace[1 + (slot)] = (unsigned long long)clock64(); } while (0)
#else
#define TF_STAMP(it, slot) do { } while (0)
#define TF_STAMP0(slot) do { } while (0)
#endif

#ifndef MLLMB200_TF_DQ_WARPS
#define MLLMB200_TF_DQ_WARPS 16
#endif
// Dequant warps (a multiple of 8).  The warps that share a set of 32 weight rows take turns over the K-groups; one
// K-group costs a warp a chain of waits, loads, ~80 ALU instructions and a tensor-memory store of several hundred
// cycles, so it takes several warps per row set to keep that chain off the critical path (measured with 8 warps:
// ~900 cycles per K-tile of 2 groups against 512 cycles of tensor-core time).
constexpr int kTfDequantWarps = MLLMB200_TF_DQ_WARPS;
constexpr int kTfThreads = (kTfDequantWarps + 2) * 32;
constexpr int kTfTileRows = 128;   // weight rows per MMA (tensor-memory lanes); a CTA tile is ROWS = 128 or 256 of them

constexpr int kTfMaxProblems = 4;
constexpr int kTfMaxPeers = 7;
struct TfProblem {          // one weight matrix of a launch; all problems share x (M, K, the activation blocks)
  const uint8_t* tiled;     // TiledHeader at offset 0
  void* y;                  // fp32 [M, ldy] (W4A32) or fp16 [M, ldy] (W4A16)
  int n, ldy, num_panels;
  int tile_begin;           // first blockIdx.x of this problem
  size_t bias_off;
  // tensor parallelism (W4A32 only): every element is also stored at y_peer[i][m * ldy + n], i < num_peers - the
  // output buffers of the other GPUs mapped into this process; plain stores that cross NVLink tile by tile
  int num_peers;
  float* y_peer[kTfMaxPeers];
};
struct TfParams {
  const uint8_t* a_blocks;  // activations, [num_groups][m8_pad][512 bytes] fp16 canonical blocks
  const float2* a_hdr;      // [m] {lhs_scale, a_off bits}; unused (may be null) on the W4A16 path
  int m, k, num_groups, m8_pad, num_problems;
  int use_pdl;  // programmatic dependent launch: everything up to the first read of the activations overlaps the previous kernel
  // Grid: one CTA per output tile for tiles [0, split_begin), two per tile from there on (m_tiles = tiles along M).
  // K split in two (grids that would leave most SMs idle, and the tiles left over after the last full wave): the
  // two CTAs of an output tile each take half of the K-tiles; whichever finishes its half first parks its raw
  // accumulators in the tile's place in y, the other one adds them to its own and runs the epilogue.
  // split_sync: two zeroed ints per split output tile {arrivals, parked}.
  int m_tiles, split_begin;
  int* split_sync;
  TfProblem prob[kTfMaxProblems];
};

// A16 = the W4A16 sibling format (layout_a16.h): 768-byte cells with an fp32 scale and an fp32 zero term per
// row and K-group, A = fp16( ((u - 8) * s + z) * 2^E ) (one rounding), B = fp16( a_q * a_s ) per 32-element
// block (one rounding), fp16 output.
//
// ATM = the dequantized weight operand lives in TENSOR memory, not in shared memory: the dequant warps write their
// rows with tcgen05.st (thread = lane = weight row, two fp16 per 32-bit column) and the MMA takes A from there.
// Shared memory then carries only the loaded data - per K-group of a 128 x 256 tile 16 KB of B read by the MMAs
// plus 18.6 KB written by the copies, instead of 24 + 8 + 18.6 KB - and the room of the operand stages goes to a
// deeper ring.  Columns: [0, NT) the accumulator, then kAStages x kGroups x 16 of operand (512 allocated).
template <int NT, int ROWS, bool A16 = false, bool ATM = false>
struct TfSmem {
  static_assert(!ATM || ROWS == 128, "the tensor-memory operand is for single-accumulator tiles");
  static constexpr int kCell = A16 ? kCellBytesA16 : kCellBytes;
  // K-groups per stage.  Every stage costs the MMA-issuing warp a barrier wait and a commit.
  static constexpr int kGroups = (NT >= 256 || ROWS > 128) ? 2 : 4;
  static constexpr int kPanels = ROWS / kPanelRows;
  static constexpr int kRawBytes = kPanels * kGroups * kCell;
  static constexpr int kBBytes = kGroups * NT * 64;
  static constexpr int kStageBytes = kRawBytes + kBBytes;
  static constexpr int kBarBytes = 256;
  static constexpr int kHdrBytes = NT * 8;  // {lhs_scale, a_off} of the tile's activation rows
  static constexpr int kFitStages = (227 * 1024 - 1024 - kBarBytes - kHdrBytes) / kStageBytes;
  // A K-tile passes through a chain of hand-offs (copy landed -> dequantized -> MMAs issued -> MMAs
  // committed -> stage free) of well over a thousand cycles; its cost per tile is the chain divided by
  // the number of tiles in flight, so both rings are as deep as shared memory allows.
  static constexpr int kStages = ATM ? (kFitStages < 7 ? kFitStages : 7) : (NT >= 256 && ROWS == 128) ? 4 : 3;
  // must not exceed kStages (the dequant warps wait on mma_done of tile it - kAStages); the 768-byte cells of the
  // W4A16 format leave room for two operand stages of 4 K-groups
  static constexpr int kAColsPerStage = kGroups * 16;  // tensor-memory columns of one operand stage (ATM)
  static constexpr int kATmemStages = (512 - NT) / kAColsPerStage;
  static constexpr int kAStages = ATM ? (kATmemStages < kStages ? kATmemStages : kStages) : (A16 && NT < 256) ? 2 : kStages;
  static constexpr int kGroupABytes = ROWS * kGroup * 2;  // one K-group of the A operand (8 or 16 KB)
  static constexpr int kABytes = ATM ? 0 : kGroups * kGroupABytes;
  static constexpr int kAOffset = kBarBytes + kHdrBytes + kStages * kStageBytes;
  static constexpr int kTotal = kAOffset + kAStages * kABytes + 1024;
  static_assert(kTotal <= 227 * 1024, "shared memory");
};

// ROWS = 256: two 128-row accumulators side by side in tensor memory share every activation block
// that is loaded - the activation (B) operand is re-read from L2 once per weight tile, which bounds
// the 128-row tile on large grids.
template <int NT, int ROWS, bool A16, bool ATM>
__global__ void __launch_bounds__(kTfThreads, 1) w4a32_gemm_tcf16_kernel(const TfParams p) {
  using S = TfSmem<NT, ROWS, A16, ATM>;
  constexpr int kCell = S::kCell;
  static_assert(sizeof(TiledHeader) == sizeof(TiledHeaderA16), "both formats keep their cells 256 bytes in");
  constexpr int kPanels = S::kPanels, kHalves = ROWS / kTfTileRows, kTfGroupABytes = S::kGroupABytes;
  constexpr int kStages = S::kStages, kTfAStages = S::kAStages, kTfGroupsPerStage = S::kGroups;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  static_assert((2 * S::kStages + kTfAStages + 1) * 8 + 8 <= S::kBarBytes, "barrier area");
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem);  // [kStages]   loaded data arrived
  uint64_t* mma_done = raw_full + kStages;                 // [kStages]   the MMAs that read a stage completed
  uint64_t* a_full = mma_done + kStages;                   // [kTfAStages] dequantized operand written
  uint64_t* acc_done = a_full + kTfAStages;                // [1]         all MMAs of the tile completed
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  float2* s_hdr = reinterpret_cast<float2*>(smem + S::kBarBytes);
  uint8_t* stages = smem + S::kBarBytes + S::kHdrBytes;
  uint8_t* a_stages = smem + S::kAOffset;

  const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // (warp-uniform for the compiler)
  if (p.use_pdl) pdl_launch_dependents();  // the next kernel waits for this whole grid before it touches anything we use
  // CTAs are dispatched in order of blockIdx.x.  Output tiles are numbered so that the tiles that share a weight tile
  // (same columns of W, different rows of x) are neighbours in that order: they run in the same wave, the weight tile
  // comes from DRAM once and the rest of them find it in L2, while the activation blocks, which every wave reads in
  // full, stay resident.  The two halves of a split tile are neighbours too.
  const int linear = (int)blockIdx.x;
  const bool split_k = linear >= p.split_begin;
  const int tile_lin = split_k ? p.split_begin + ((linear - p.split_begin) >> 1) : linear;
  const int split = split_k ? ((linear - p.split_begin) & 1) : 0;
  const int bx = tile_lin / p.m_tiles, tile_m = tile_lin % p.m_tiles;
#ifdef MLLMB200_TF_TRACE
  const bool traced = linear == (int)gridDim.x / 2 && lane == 0 && (warp == 0 || warp >= kTfDequantWarps) && g_gs_trace != nullptr;
  if (warp == 0) TF_STAMP0(0);
#endif
  int pi = 0;
#pragma unroll
  for (int i = 1; i < kTfMaxProblems; ++i)
    if (i < p.num_problems && bx >= p.prob[i].tile_begin) pi = i;
  const TfProblem& pr = p.prob[pi];
  if constexpr (!A16) {  // (the W4A16 launcher's kernels check their own header format)
    if (!tiled_header_ok_cta(pr.tiled, pr.n, p.k)) return;  // before any copy, barrier or tensor-memory allocation
  }
  const int tile_n = bx - pr.tile_begin;
  const int panel0 = tile_n * kPanels, m0 = tile_m * NT;
  const int k_tiles_all = (p.num_groups + kTfGroupsPerStage - 1) / kTfGroupsPerStage;
  // this CTA's K-tiles: [it0, it0 + k_tiles) of the matrix; `it` below counts from 0 within them
  const int it0 = split == 0 ? 0 : k_tiles_all / 2;
  const int k_tiles = !split_k ? k_tiles_all : (split == 0 ? k_tiles_all / 2 : k_tiles_all - k_tiles_all / 2);
  constexpr uint32_t kTmemCols = ATM ? 512u : (uint32_t)(kHalves * NT) < 32u ? 32u : (uint32_t)(kHalves * NT);
  constexpr uint32_t kAColBase = (uint32_t)NT;  // first operand column (ATM)
  // Dequant work: kRowSets sets of 32 weight rows, kDqShare warps per set; K-group g of K-tile it goes to the warp
  // number (it * groups per tile + g) mod kDqShare of its row set.
  constexpr int kRowSets = ROWS / 32, kDqShare = kTfDequantWarps / kRowSets;
  static_assert(kDqShare >= 1 && (kDqShare % kTfGroupsPerStage == 0 || kTfGroupsPerStage % kDqShare == 0), "turn-taking");
  constexpr int kDqArrivals = kRowSets * (kDqShare < kTfGroupsPerStage ? kDqShare : kTfGroupsPerStage);

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&mma_done[s], 1);
    }
    for (int s = 0; s < kTfAStages; ++s) mbar_init(&a_full[s], kDqArrivals);  // one arrival per warp that has a K-group in the tile
    mbar_init(acc_done, 1);
    mbar_fence_init();
  }
  if (warp == kTfDequantWarps + 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base_any = *tmem_base_slot;
  const TiledHeader* hdr = reinterpret_cast<const TiledHeader*>(pr.tiled);

  if (warp == kTfDequantWarps) {
    // ------------------------------------------------------------ producer
    const int np = min(kPanels, pr.num_panels - panel0);
#if MLLMB200_TF_WEIGHT_HINT
    const uint64_t stream_once = l2_policy_evict_first();
#endif
    // One K-tile into its stage: `parts` bit 0 = the weight cells, bit 1 = the activation blocks.  The barrier is armed
    // for both together, with the first part that is requested.
    auto request = [&](int it, int parts) {
      const int s = it % kStages;
      const int g0 = (it0 + it) * kTfGroupsPerStage;
      const int ng = min(kTfGroupsPerStage, p.num_groups - g0);
      uint8_t* st = stages + (size_t)s * S::kStageBytes;
      if ((parts & 1) && lane == 0) mbar_arrive_expect_tx(&raw_full[s], (uint32_t)(np * ng * kCell + ng * NT * 64));
      __syncwarp();
      if ((parts & 1) && lane < np) {
        // the weights pass through once per tile row; the activation blocks are what every tile row re-reads:
        // first in line for eviction, so that a wave of weight tiles does not push the blocks out of L2
#if MLLMB200_TF_WEIGHT_HINT
        bulk_g2s_hint(st + lane * kTfGroupsPerStage * kCell,
                      pr.tiled + sizeof(TiledHeader) + ((size_t)(panel0 + lane) * p.num_groups + g0) * kCell,
                      (uint32_t)(ng * kCell), &raw_full[s], stream_once);
#else
        bulk_g2s(st + lane * kTfGroupsPerStage * kCell,
                 pr.tiled + sizeof(TiledHeader) + ((size_t)(panel0 + lane) * p.num_groups + g0) * kCell,
                 (uint32_t)(ng * kCell), &raw_full[s]);
#endif
      } else if ((parts & 2) && lane >= kPanels && lane < kPanels + ng) {
        const int g = lane - kPanels;
        bulk_g2s(st + S::kRawBytes + g * NT * 64, p.a_blocks + ((size_t)(g0 + g) * p.m8_pad + (m0 >> 3)) * 512,
                 (uint32_t)(NT * 64), &raw_full[s]);
      }
    };
    // The weights are constant, the activation blocks come from the kernel before this one: under programmatic
    // dependent launch the weight cells of the first lap are requested before the wait, the blocks after it.
    const int first_lap = min(k_tiles, kStages);
    if (p.use_pdl) {
      for (int it = 0; it < first_lap; ++it) request(it, 1);
      pdl_wait_prior();
      for (int it = 0; it < first_lap; ++it) request(it, 2);
    } else {
      for (int it = 0; it < first_lap; ++it) request(it, 3);
    }
    for (int it = first_lap; it < k_tiles; ++it) {
      const int s = it % kStages;
      const uint32_t ph = (uint32_t)(it / kStages) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(&mma_done[s], ph ^ 1u))) break;
      TF_STAMP(it, 0);
      request(it, 3);
    }
  } else if (warp == kTfDequantWarps + 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop (same waits, same addresses in every lane) and one elected lane issues: the
    // operands of tcgen05.mma are then warp-uniform values, not the private registers of a diverged lane.
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_base_any, 0);
    const bool issuer = elect_one_sync();
    {
      // instruction descriptor: D = f32, A = B = f16, both K-major, N = NT, M = 128
      const uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((128u >> 4) << 24);
      bool ok = true;
      uint32_t accumulate = 0;
      for (int it = 0; it < k_tiles && ok; ++it) {
        const int s = it % kStages, sa = it % kTfAStages;
        // a_full[sa] is arrived on by the dequant warps AFTER they saw raw_full[s] complete, so it also
        // orders this stage's bulk copies (the B operand) before the MMAs: one wait instead of two
        TF_STAMP(it, 4);
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&a_full[sa], (uint32_t)(it / kTfAStages) & 1u));
        if (!ok) break;
        TF_STAMP(it, 5);
        tc_fence_after();
        if (issuer) {
        const int ng = min(kTfGroupsPerStage, p.num_groups - (it0 + it) * kTfGroupsPerStage);
        uint8_t* st = stages + (size_t)s * S::kStageBytes;
        const uint32_t b_addr = smem_u32(st + S::kRawBytes), a_addr = smem_u32(a_stages + (size_t)sa * S::kABytes);
        // K-major, no swizzle: 16-byte K chunks of a row 128 bytes apart, 8-row groups 512 bytes apart
        const uint64_t a_desc = make_kmajor_desc(a_addr, 128, 512), b_desc = make_kmajor_desc(b_addr, 128, 512);
#pragma unroll
        for (int g = 0; g < kTfGroupsPerStage; ++g) {
          if (g >= ng) break;
#pragma unroll
          for (int h = 0; h < 2; ++h) {  // K = 16 per instruction: two chunks of 8; the start address counts 16-byte units
            if constexpr (ATM) {
              tc_mma_f16_ts(tmem_base, tmem_base + kAColBase + (uint32_t)(sa * S::kAColsPerStage + g * 16 + h * 8),
                            b_desc + (uint64_t)((g * NT * 64 + h * 256) >> 4), idesc, accumulate);
            } else {
#pragma unroll
              for (int rh = 0; rh < kHalves; ++rh)  // 128-row halves of the tile: own accumulator (NT columns each), same B
                tc_mma_f16(tmem_base + (uint32_t)(rh * NT),
                           a_desc + (uint64_t)((g * kTfGroupABytes + rh * (kTfTileRows * 64) + h * 256) >> 4),
                           b_desc + (uint64_t)((g * NT * 64 + h * 256) >> 4), idesc, accumulate);
            }
            accumulate = 1;
          }
        }
        tc_commit(&mma_done[s]);  // frees the loaded stage (producer) and the A stage (dequant)
        }
        __syncwarp();
        TF_STAMP(it, 6);
      }
      if (ok && issuer) tc_commit(acc_done);
    }
  } else {
    const uint32_t tmem_base = tmem_base_any;
    // ------------------------------------------------------------ dequant: thread j = weight row j of the tile.
    // ROWS = 128: rows are shared by warps w and w + 4, which alternate over the K-groups of a stage;
    // ROWS = 256: one row per thread, every group.
    const int j = (warp % kRowSets) * 32 + lane;
    const int turn = warp / kRowSets;
    const int q = j >> 5, r = j & 31;  // panel of the tile, row in the panel
    const bool have_panel = panel0 + q < pr.num_panels;
    const uint32_t scale_mode = hdr->scale_mode;
    // 2^E maps the largest |scale| of the matrix into [2^10, 2^11): (u - 8) * s * 2^E < 2^14, 24 * s * 2^E < 2^16 * 0.75.
    // (Read here, not before the role split: the producer must not wait for this load.)
    // W4A16: the header word at the same offset holds the bits of max (8 |s| + |z|) >= max |weight|,
    // mapped into [2^14, 2^15).
    const int emax = (int)(((A16 ? reinterpret_cast<const TiledHeaderA16*>(pr.tiled)->max_weight_bits : hdr->max_scale_bits) >> 23) & 0xFFu);
    const int E = emax == 0 ? 0 : (A16 ? 14 : 10) - (emax - 127);
    const bool fused_dequant = MLLMB200_TF_FUSED_DEQUANT && scale_mode != 2u;
    const float up = exp2f((float)E), down = exp2f((float)-E);
    if constexpr (!A16) {
      // the rows' {scale, offset} pairs, written by the quantization kernel in front of this one; read by these
      // same warps in the epilogue, after the barrier below
      if (p.use_pdl) pdl_wait_prior();
      for (int i = tid; i < NT; i += kTfDequantWarps * 32) s_hdr[i] = (m0 + i < p.m) ? p.a_hdr[m0 + i] : make_float2(0.0f, 0.0f);
      asm volatile("bar.sync 1, %0;" ::"n"(kTfDequantWarps * 32) : "memory");
    }
    bool ok = true;
    for (int it = 0; it < k_tiles && ok; ++it) {
      const int s = it % kStages, sa = it % kTfAStages;
      const int gsel = (turn + kDqShare - (it * kTfGroupsPerStage) % kDqShare) % kDqShare;  // (turns count from this CTA's first tile)  // this warp's first K-group of the tile
      if (gsel >= kTfGroupsPerStage) continue;                                              // none: not its turn
      TF_STAMP(it, 7);
      ok = mbar_wait_bounded(&raw_full[s], (uint32_t)(it / kStages) & 1u);
      TF_STAMP(it, 1);
      if (ok && it >= kTfAStages) {  // the A stage is free once the MMAs of K-tile it - kTfAStages are done
        const int prev = it - kTfAStages;
        ok = mbar_wait_bounded(&mma_done[prev % kStages], (uint32_t)(prev / kStages) & 1u);
      }
      if (!ok) break;
      TF_STAMP(it, 2);
      const int ng = min(kTfGroupsPerStage, p.num_groups - (it0 + it) * kTfGroupsPerStage);
      const uint8_t* raw = stages + (size_t)s * S::kStageBytes + q * kTfGroupsPerStage * kCell;
      uint8_t* a_out = a_stages + (size_t)sa * S::kABytes + (j >> 3) * 512 + (j & 7) * 16;
      // ATM: this warp's lanes of tensor memory (32 (warp % 4)..), first column of the operand stage
      const uint32_t a_tm = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + kAColBase + (uint32_t)(sa * S::kAColsPerStage);
#pragma unroll
      for (int g = gsel; g < kTfGroupsPerStage; g += kDqShare) {
        if (g < ng) {
        uint4 w = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
        float sc = 0.0f;
        uint32_t areg[16];  // ATM: the row's 32 fp16 of this K-group, column c * 4 + t = chunk c, pair t
        if constexpr (A16) {
          // fp32 all the way to one rounding: ((u - 8) * s + z) * 2^E; 0x4B000000 | u = 2^23 + u as a float
          float zr = 0.0f;
          if (have_panel) {
            w = *reinterpret_cast<const uint4*>(raw + g * kCell + r * 16);
            sc = *reinterpret_cast<const float*>(raw + g * kCell + kCellNibbleBytes + r * 4);
            zr = *reinterpret_cast<const float*>(raw + g * kCell + kCellNibbleBytes + kPanelRows * 4 + r * 4);
          }
          const float s_up = sc * up, z_up = zr * up;
          const uint32_t wa[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float f[8];
#pragma unroll
            for (int t = 0; t < 8; ++t)
              f[t] = fmaf(__uint_as_float(0x4B000000u | ((wa[c] >> (4 * t)) & 15u)) - 8388616.0f, s_up, z_up);
            uint32_t o[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {  // same element order as the W4A32 unpack: k = 8c + {0,4,1,5,2,6,3,7}
              const __half2 v = __floats2half2_rn(f[t], f[t + 4]);
              o[t] = *reinterpret_cast<const uint32_t*>(&v);
            }
            if constexpr (ATM) {
#pragma unroll
              for (int t = 0; t < 4; ++t) areg[c * 4 + t] = o[t];
            } else {
              *reinterpret_cast<uint4*>(a_out + g * kTfGroupABytes + c * 128) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        } else {
        if (have_panel) {
          w = *reinterpret_cast<const uint4*>(raw + g * kCellBytes + r * 16);
          sc = decode_scale(*reinterpret_cast<const uint16_t*>(raw + g * kCellBytes + kCellNibbleBytes + r * 2), scale_mode);
        }
        const float s_up = sc * up;                              // exact: a power-of-two multiple of a bf16 / fp16 value
        const __half2 s2 = __float2half2_rn(s_up);
        // (u - 8) * s2 below is exact for a bf16-encoded scale (3 + 8 bits); for an fp16-encoded one HMUL2 rounds it once
        const __half2 off = __floats2half2_rn(1032.0f, 1032.0f);  // 0x6400 | nibble = 1024 + nibble; weight = nibble - 8
        // bf16-encoded scales, one instruction less per pair: the nibble in mantissa bits 6..9 of 0x4400 reads
        // x = 4 + u / 4, and (u - 8) s = x (4 s) - 24 s as ONE fused multiply-add - 4 s and 24 s = 3 * 8 * s
        // (8 + 2 significant bits) are exact in fp16, and so is the result, so nothing is rounded
        const __half2 s4 = __float2half2_rn(4.0f * s_up), c24 = __float2half2_rn(-24.0f * s_up);
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // word c = k 8c..8c+7; half2 t = nibbles t and t + 4 (16 bits apart)
          uint32_t o[4];
          if (fused_dequant) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const uint32_t moved = t == 0 ? ws[c] << 6 : t == 1 ? ws[c] << 2 : t == 2 ? ws[c] >> 2 : ws[c] >> 6;
              const uint32_t bits = (moved & 0x03C003C0u) | 0x44004400u;
              const __half2 v = __hfma2(*reinterpret_cast<const __half2*>(&bits), s4, c24);
              o[t] = *reinterpret_cast<const uint32_t*>(&v);
            }
          } else {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const uint32_t bits = ((ws[c] >> (4 * t)) & 0x000F000Fu) | 0x64006400u;
            const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&bits), off), s2);
            o[t] = *reinterpret_cast<const uint32_t*>(&v);
          }
          }
          if constexpr (ATM) {
#pragma unroll
            for (int t = 0; t < 4; ++t) areg[c * 4 + t] = o[t];
          } else {
            *reinterpret_cast<uint4*>(a_out + g * kTfGroupABytes + c * 128) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        }
        if constexpr (ATM) tmem_st16(a_tm + (uint32_t)(g * 16), areg);
        }
      }
      if constexpr (ATM) {
        tmem_st_wait();     // the stores have landed ...
        tc_fence_before();  // ... and are ordered before the MMAs of the thread that sees the arrival below
      } else {
        fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core
      }
      __syncwarp();
      TF_STAMP(it, 3);
      if (lane == 0) mbar_arrive(&a_full[sa]);
    }
    // ------------------------------------------------------------ epilogue (same four warps)
    // tensor-memory loads are warp-wide: every lane takes part, only the stores are guarded
    ok = __all_sync(0xffffffffu, ok && mbar_wait_bounded(acc_done, 0));
    tc_fence_after();
    TF_STAMP0(1);
    // K split: 0 = whole K here; 1 = first of the tile's two CTAs to finish (parks its accumulators in y);
    // 2 = second (adds the parked ones).  The second waits - bounded - only for a CTA that is already in its epilogue.
    int role = 0;
    int* tile_sync = nullptr;
    if constexpr (!A16) {
      if (split_k) {
        tile_sync = p.split_sync + 2 * (tile_lin - p.split_begin);
        int* s_role = reinterpret_cast<int*>(tmem_base_slot + 1);
        if (tid == 0) {
          int r = atomicAdd(tile_sync, 1) == 0 ? 1 : 2;
          if (r == 2) {
            const long long t0 = clock64();
            while (ld_acquire_gpu(tile_sync + 1) == 0) {
              if (clock64() - t0 > (1ll << 31)) {
                atomicOr(&g_device_status, kDevStatusTimeout);
                r = 3;  // gave up: no result for this tile, the status word says so
                break;
              }
            }
          }
          *s_role = r;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kTfDequantWarps * 32) : "memory");
        role = *s_role;
        if (role == 3) ok = false;
      }
    }
    // warps w, w + 4, .. share tensor-memory lanes 32 (w % 4).. and split the columns
    constexpr int kColSplit = kTfDequantWarps / 4, kColsPerWarp = NT / kColSplit, kChunk = kColsPerWarp >= 32 ? 32 : 16;
    static_assert(kColsPerWarp % kChunk == 0, "column split");
    const int col_begin = (warp >> 2) * kColsPerWarp, col_end = col_begin + kColsPerWarp;
#pragma unroll 1
    for (int rh = 0; rh < kHalves; ++rh) {  // the 128-row halves of the tile: accumulators NT columns apart
      const int n = tile_n * ROWS + rh * kTfTileRows + (warp & 3) * 32 + lane;
      const bool live = n < pr.n;
      const float bs = live ? reinterpret_cast<const float*>(pr.tiled + pr.bias_off)[n] : 0.0f;
      const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(rh * NT);
      if (ok) {
#pragma unroll 1
        for (int c0 = col_begin; c0 < col_end && m0 + c0 < p.m; c0 += kChunk) {
          // all loads of the chunk first (tensor memory, the rows' scales), then the arithmetic, then the stores
          // back to back: lanes = consecutive n, one 128-byte line per store instruction
          uint32_t v[kChunk];
          tmem_ld16(lane_addr + (uint32_t)c0, reinterpret_cast<uint32_t(&)[16]>(v[0]));
          if constexpr (kChunk == 32) tmem_ld16(lane_addr + (uint32_t)(c0 + 16), reinterpret_cast<uint32_t(&)[16]>(v[16]));
          float sc[kChunk];
          if constexpr (!A16) {
#pragma unroll
            for (int i = 0; i < kChunk; i += 2) {
              const float4 h = *reinterpret_cast<const float4*>(&s_hdr[c0 + i]);  // {scale, offset} of two rows
              sc[i] = h.x, sc[i + 1] = h.z;
            }
          }
          tmem_ld_wait();
          const int m_left = p.m - (m0 + c0);
          if constexpr (A16) {
            __half* yp = static_cast<__half*>(pr.y) + (size_t)(m0 + c0) * pr.ldy + n;
#pragma unroll
            for (int i = 0; i < kChunk; ++i) {
              const float val = fmaf(__uint_as_float(v[i]), down, bs);
              if (live && i < m_left) yp[(size_t)i * pr.ldy] = __float2half_rn(fminf(fmaxf(val, -65504.0f), 65504.0f));
            }
          } else {
            const size_t at0 = (size_t)(m0 + c0) * pr.ldy + n;
            float* yp = static_cast<float*>(pr.y) + at0;
            if (role == 1) {  // park the raw sums
#pragma unroll
              for (int i = 0; i < kChunk; ++i)
                if (live && i < m_left) __stcg(yp + (size_t)i * pr.ldy, __uint_as_float(v[i]));
              continue;
            }
            if (role == 2) {  // a + b = b + a: the result does not depend on which half finished first
              float parked[kChunk];
#pragma unroll
              for (int i = 0; i < kChunk; ++i) parked[i] = (live && i < m_left) ? __ldcg(yp + (size_t)i * pr.ldy) : 0.0f;
#pragma unroll
              for (int i = 0; i < kChunk; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + parked[i]);
            }
#pragma unroll
            for (int i = 0; i < kChunk; ++i) v[i] = __float_as_uint(clamp_flt_max(fmaf(__uint_as_float(v[i]) * down, sc[i], bs)));
#pragma unroll
            for (int i = 0; i < kChunk; ++i)
              if (live && i < m_left) yp[(size_t)i * pr.ldy] = __uint_as_float(v[i]);
            for (int pe = 0; pe < pr.num_peers; ++pe) {  // tensor parallelism: the same tile into every peer's y
              float* yq = pr.y_peer[pe] + at0;
#pragma unroll
              for (int i = 0; i < kChunk; ++i)
                if (live && i < m_left) yq[(size_t)i * pr.ldy] = __uint_as_float(v[i]);
            }
          }
        }
      }
    }
    if (role == 1) {  // every parked value is visible before the flag is
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kTfDequantWarps * 32) : "memory");
      if (tid == 0) st_release_gpu(tile_sync + 1, 1);
    }
    tc_fence_before();
    TF_STAMP0(2);
  }
  __syncthreads();
  if (warp == kTfDequantWarps + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base_any, kTmemCols);
  }
}

template <int NT, int ROWS, bool A16 = false, bool ATM = false>
static cudaError_t launch_tf_t(const TfParams& prm, int total_tiles, cudaStream_t stream) {
  using S = TfSmem<NT, ROWS, A16, ATM>;
  static bool configured[64] = {};  // function attributes are per device
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (!(dev >= 0 && dev < 64 && configured[dev])) {
    e = cudaFuncSetAttribute(w4a32_gemm_tcf16_kernel<NT, ROWS, A16, ATM>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * total_tiles * prm.m_tiles - prm.split_begin), 1, 1);  // (split_begin = all tiles: no split)
  cfg.blockDim = dim3(kTfThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  if (prm.use_pdl) {
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, w4a32_gemm_tcf16_kernel<NT, ROWS, A16, ATM>, prm);
}

// Tile shape for a launch: weight rows per CTA (128, or 256 = two accumulators sharing every loaded
// activation block) and activation rows per tile.  128 x NT x 16 takes NT / 2 cycles of tensor-core time
// and the dequantization of a K-group costs the same whatever NT, so narrow activation tiles are bound by
// the dequant warps; on grids that fill the GPU the 128-row tile moves twice the bytes per FLOP through L2
// (the activation operand, which every weight tile re-reads) - config 4, M = 2048: 0.84 ms with either.
struct TfTile {
  int rows, nt;
};
static int tf_sm_count() {
  static int sms[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0 && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms[dev] = 148;
  return sms[dev];
}
static TfTile tf_tile_for(int m, int count, const int* n) {
  long long t128 = 0, t256 = 0;
  bool wide = true;  // 256-row tiles only for matrices with at least 4096 rows
  for (int i = 0; i < count; ++i) {
    t128 += (n[i] + 127) / 128;
    t256 += (n[i] + 255) / 256;
    wide = wide && n[i] >= 4096;
  }
  TfTile t;
  if (MLLMB200_TF_WIDE && wide && m >= 256 && t256 * ((m + 255) / 256) >= 100) {  // (256 rows x 128: measured slower than 128 x 256, 31 vs 24 us)
    t.rows = 256;
    t.nt = 256;
    return t;
  }
  t.rows = 128;
  t.nt = (m >= 256 && t128 * ((m + 255) / 256) >= 100) ? 256 : (m >= 128 ? 128 : 64);
  return t;
}
int w4a32_gemm_tcf16_tile(int m, int n) { return tf_tile_for(m, 1, &n).nt; }
int w4a32_gemm_tcf16_tile_grouped(int m, int count, const int* n) { return tf_tile_for(m, count, n).nt; }
int w4a32_gemm_tcf16_m_pad(int m, int n) {
  const int nt = w4a32_gemm_tcf16_tile(m, n);
  return (m + nt - 1) / nt * nt;
}
int w4a32_gemm_tcf16_m_pad_max(int m) { return (m + 255) / 256 * 256; }
bool w4a32_gemm_tcf16_supported(int m, int k, int n) { return m >= 64 && k >= 1 && n >= 1 && (m + 63) / 64 <= 65535; }
// Shapes on which this path is at least as fast as the int8 path (measured on the Qwen2-1.5B layer
// shapes at M = 512: 17 vs 18 us for N = 1536 / 256, 24 vs 60 us for N = 8960, 59 vs 68 us for K = 8960).
// At 64 <= M < 128 only where the weight tiles alone fill the GPU and K is short (gate / up of the 1.5B model, alone or
// grouped: 17 vs 30 us at M = 64 against the streaming small-batch GEMM); narrow or long-K matrices stay there.
bool w4a32_gemm_tcf16_preferred(int m, int k, int n) {
  if (!w4a32_gemm_tcf16_supported(m, k, n)) return false;
  return m >= 128 || (MLLMB200_TF_SMALL_M && n >= 8192 && k <= 4096);
}

// Up to four matrices that share x in ONE launch (their weight tiles side by side in the grid):
// the activation blocks must be padded to m_pad = a multiple of the tile width chosen by
// w4a32_gemm_tcf16_tile_grouped for the same arguments.
// split_sync (optional): split_sync_ints ints that are ZERO when the kernel starts (the quantization kernel in front of
// it clears them); with them, launches that would fill less than half of the GPU split K in two.
cudaError_t launch_w4a32_gemm_tcf16_grouped(const uint8_t* a_blocks, const float2* a_hdr, int m, int k, int count,
                                            const void* const* tiled, float* const* y, const int* n, const int* ldy,
                                            cudaStream_t stream, int num_peers, float* const* y_peers, int use_pdl,
                                            int* split_sync, int split_sync_ints) {
  if (count < 1 || count > kTfMaxProblems) return cudaErrorInvalidValue;
  if (num_peers > 0 && (count != 1 || num_peers > kTfMaxPeers || y_peers == nullptr)) return cudaErrorInvalidValue;
  const TfTile tile = tf_tile_for(m, count, n);
  const int nt = tile.nt;
  TfParams prm = {};
  prm.a_blocks = a_blocks;
  prm.a_hdr = a_hdr;
  prm.m = m, prm.k = k;
  prm.num_groups = (k + kGroup - 1) / kGroup;
  prm.m8_pad = (m + nt - 1) / nt * nt / 8;
  prm.num_problems = count;
  prm.use_pdl = use_pdl;
  int tiles = 0;
  for (int i = 0; i < count; ++i) {
    const TiledHeader th = make_tiled_header(n[i], k, 0, 0);
    prm.prob[i].tiled = static_cast<const uint8_t*>(tiled[i]);
    prm.prob[i].y = y[i];
    prm.prob[i].n = n[i];
    prm.prob[i].ldy = ldy[i];
    prm.prob[i].num_panels = (n[i] + kPanelRows - 1) / kPanelRows;
    prm.prob[i].tile_begin = tiles;
    prm.prob[i].bias_off = th.bias_off;
    prm.prob[i].num_peers = num_peers > 0 ? num_peers : 0;
    for (int j = 0; j < prm.prob[i].num_peers; ++j) prm.prob[i].y_peer[j] = y_peers[j];
    tiles += (n[i] + tile.rows - 1) / tile.rows;
  }
  prm.split_sync = split_sync;
  prm.m_tiles = (m + nt - 1) / nt;
  {
    // Which output tiles split K: all of them when two CTAs per tile still fit one wave; else the tiles left over
    // after the last full wave, when they are fewer than half a wave (config 4: 896 tiles = 6 waves + 8: a seventh
    // wave of 8 CTAs would cost as much as a full one).
    const int out_tiles = tiles * prm.m_tiles, sms = tf_sm_count();
    const int groups_per_tile = (nt >= 256 || tile.rows == 256) ? 2 : 4;  // (TfSmem::kGroups)
    const int k_tiles = (prm.num_groups + groups_per_tile - 1) / groups_per_tile;
    const int left_over = out_tiles % sms;
    int split_tiles = 0;
    if (MLLMB200_TF_SPLIT_K && split_sync != nullptr && k_tiles >= 8) {
      if (2 * out_tiles <= sms) split_tiles = out_tiles;
      else if (out_tiles > sms && 2 * left_over <= sms) split_tiles = left_over;
    }
    if (2 * split_tiles > split_sync_ints) split_tiles = 0;
    prm.split_begin = out_tiles - split_tiles;
  }
  if (tile.rows == 256) return launch_tf_t<256, 256>(prm, tiles, stream);
  constexpr bool kAtm = MLLMB200_TF_ATM != 0;
  switch (nt) {
    case 256: return launch_tf_t<256, 128, false, kAtm>(prm, tiles, stream);
    case 128: return launch_tf_t<128, 128, false, kAtm>(prm, tiles, stream);
    default: return launch_tf_t<64, 128, false, kAtm>(prm, tiles, stream);
  }
}

// W4A16: 128-row tiles; the activation blocks must be padded to a multiple of w4a16_gemm_tcf16_tile_grouped(...)
// rows.  Up to four matrices that share x ride in one launch (their weight tiles side by side in the grid).
int w4a16_gemm_tcf16_tile_grouped(int m, int count, const int* n) {
  long long t128 = 0;
  for (int i = 0; i < count; ++i) t128 += (n[i] + 127) / 128;
  return (m >= 256 && t128 * ((m + 255) / 256) >= 100) ? 256 : (m >= 128 ? 128 : 64);
}
int w4a16_gemm_tcf16_tile(int m, int n) { return w4a16_gemm_tcf16_tile_grouped(m, 1, &n); }
cudaError_t launch_w4a16_gemm_tcf16_grouped(const uint8_t* a_blocks, int m, int k, int count, const void* const* tiled,
                                            void* const* y_f16, const int* n, const int* ldy, cudaStream_t stream) {
  if (count < 1 || count > kTfMaxProblems) return cudaErrorInvalidValue;
  const int nt = w4a16_gemm_tcf16_tile_grouped(m, count, n);
  TfParams prm = {};
  prm.a_blocks = a_blocks;
  prm.a_hdr = nullptr;
  prm.m = m, prm.k = k;
  prm.num_groups = (k + kGroup - 1) / kGroup;
  prm.m8_pad = (m + nt - 1) / nt * nt / 8;
  prm.num_problems = count;
  prm.m_tiles = (m + nt - 1) / nt;
  int tiles = 0;
  for (int i = 0; i < count; ++i) {
    prm.prob[i].tiled = static_cast<const uint8_t*>(tiled[i]);
    prm.prob[i].y = y_f16[i];
    prm.prob[i].n = n[i];
    prm.prob[i].ldy = ldy[i];
    prm.prob[i].num_panels = (n[i] + kPanelRows - 1) / kPanelRows;
    prm.prob[i].tile_begin = tiles;
    prm.prob[i].bias_off = make_tiled_header_a16(n[i], k, 0).bias_off;
    tiles += (n[i] + 127) / 128;
  }
  prm.split_begin = tiles * prm.m_tiles;  // (no K split: fp16 output cannot hold parked sums)
  constexpr bool kAtm = MLLMB200_TF_ATM != 0 && MLLMB200_TF_ATM_A16 != 0;
  switch (nt) {
    case 256: return launch_tf_t<256, 128, true, kAtm>(prm, tiles, stream);
    case 128: return launch_tf_t<128, 128, true, kAtm>(prm, tiles, stream);
    default: return launch_tf_t<64, 128, true, kAtm>(prm, tiles, stream);
  }
}
cudaError_t launch_w4a16_gemm_tcf16(const uint8_t* a_blocks, const void* tiled, void* y_f16, int m, int k, int n, int ldy,
                                    cudaStream_t stream) {
  return launch_w4a16_gemm_tcf16_grouped(a_blocks, m, k, 1, &tiled, &y_f16, &n, &ldy, stream);
}

cudaError_t launch_w4a32_gemm_tcf16(const uint8_t* a_blocks, const float2* a_hdr, const void* tiled, float* y, int m, int k,
                                    int n, int ldy, cudaStream_t stream, int use_pdl, int* split_sync, int split_sync_ints) {
  return launch_w4a32_gemm_tcf16_grouped(a_blocks, a_hdr, m, k, 1, &tiled, &y, &n, &ldy, stream, 0, nullptr, use_pdl,
                                         split_sync, split_sync_ints);
}

}  // namespace mllmb200
