// Streaming W4A32 GEMM for small batches (5 <= M <= 64 activation rows), sm_100a.
//
//   y[m,n] = lhs_scale[m] * ( sum_b float(sum_{k in b} a_q[m,k] * w[n,k]) * s[n,b]  +  a_off[m] * zsum[n] ) + bias[n]
//
// the expression of the GEMV (gemv_stream.cu; reference project tests/Arm/KaiLinearTest.hpp:338-377, production call
// mllm/Backends/Arm/Kernels/kai_linear.cpp:350-398): exact int32 sums per K-group, one fp32 FMA with the group
// scale per (row, column, group).
//
// At these batch sizes the linear is a weight stream like the GEMV - every weight byte is read once and used for
// at most 64 rows - but 64 times the integer work of the GEMV does not fit the CUDA cores, and the tile GEMMs
// (128 weight rows x all of K per CTA) fill a fraction of the SMs: 12 CTAs for a 1536 x 1536 matrix.  Here the
// cells of the weight matrix (layout.h: [panel of 32 rows][K-group] x 576 bytes) are spread over all SMs as in the
// GEMV and the per-group integer products run on the tensor cores:
//   * work unit = one panel x one K-slice.  A cluster of S CTAs owns panels c, c + C, c + 2C, ...; CTA rank r of it
//     takes K-groups [r G / S, (r + 1) G / S) of every one of those panels.  S is the smallest size for which the
//     quantized activations of a K-slice (36 bytes per row and group) fit beside the weight ring in shared memory:
//     1 for K = 1536 at M = 64, 6 for K = 8960.  They are loaded once per CTA with one bulk copy.
//   * a producer warp streams the unit's cells through a ring of 16-group stages (cp.async.bulk + full / empty
//     mbarriers, weights marked evict-first in L2); under programmatic dependent launch the first stages are
//     requested before griddepcontrol.wait, the activations after it.
//   * 8 compute warps: warp (ks, ns) takes the K-groups ks, ks + KS, ... of a stage and the batch columns
//     [ns, ns + 1) * 8 NTW.  Per cell: 4 word loads = the A fragments of two mma.sync.m16n8k32 (u8 nibbles x s8
//     activations -> s32; low nibbles are k 0..15, high nibbles k 16..31 of the instruction, which is the byte order
//     of the activation blocks), accumulator start value -8 * sum(a_q) (the nibbles are stored +8) plus the bits of
//     12582912.0f, so that the s32 result read as a float is 12582912 + value exactly and one FADD and one FMA with
//     the row's group scale fold it into the fp32 accumulators.
//   * at the end of a unit the warps' partial sums meet in shared memory (added in K-slice order); with S > 1
//     ranks 1.. leave theirs in a double-buffered slot of their own shared memory, signal rank 0 through an
//     mbarrier in ITS shared memory, and rank 0 adds them in rank order through distributed-shared-memory loads:
//     deterministic.  Rank 0 (or the only CTA) applies zero-point term, row scale and bias and stores y.
// Every wait is bounded; a cluster leaves together (one cluster barrier at the end) so that no CTA's shared memory
// disappears under a peer.
#include <algorithm>

#include "device_common.cuh"

namespace mllmb200 {

#ifdef MLLMB200_MS_TRACE
extern __device__ unsigned long long* g_gs_trace;  // development build only: stamps of CTA 0 into the GEMV trace buffer
#define MS_STAMP(i, v) do { if (blockIdx.x == 0 && tid == 0 && g_gs_trace != nullptr) g_gs_trace[1 + (i)] = (unsigned long long)(v); } while (0)
#else
#define MS_STAMP(i, v) do { } while (0)
#endif

#ifndef MLLMB200_MS_WARPS
#define MLLMB200_MS_WARPS 8
#endif
constexpr int kMsCWarps = MLLMB200_MS_WARPS;  // compute warps (16 were measured 7 % slower than 8)
constexpr int kMsCThreads = kMsCWarps * 32;
constexpr int kMsThreads = kMsCThreads + 32;  // + the producer warp
constexpr int kMsBlockGroups = 16;            // K-groups per ring stage
constexpr int kMsStageBytes = kMsBlockGroups * kCellBytes;  // 9216
constexpr int kMsStages = kMsCWarps > 8 ? 4 : 6;
constexpr int kMsMaxProblems = 4;
constexpr int kMsMaxCluster = 8;
constexpr int kMsActRowBytes = 36;            // per activation row and K-group: 16 + 16 bytes of int8 and the -8 * sum word
constexpr size_t kMsActBudget = 112 * 1024;   // shared memory for the activations of a CTA's K-slice
constexpr int kMsMaxM = 64;
constexpr int kMsSlotsPerThread = kMsMaxM * 8 / kMsCThreads;  // float4 result slots of a unit per compute thread (2)

struct MsProblem {
  const uint8_t* tiled;  // TiledHeader at offset 0
  float* y;
  int n, ldy, num_panels, panel_begin;  // panels [panel_begin, panel_begin + num_panels) of the launch
  size_t zsum_off, bias_off;
};
struct MsParams {
  const uint8_t* acts;   // [num_groups][ m_pad x 16 (low words) | m_pad x 16 (high words) | m_pad x 4 (-8 * sum) ]
  const float2* a_hdr;   // [m] {lhs_scale, a_off bits}
  int m, m_pad, k, num_groups;
  int cluster_size, num_clusters, total_panels, num_problems, use_pdl;
  MsProblem prob[kMsMaxProblems];
};

struct MsSmem {
  size_t bars, hdr, flags, acts, ring, red, psum, total;
};
__host__ __device__ inline MsSmem ms_smem_layout(int m_pad, int groups_per_rank, int cluster_size, int ks) {
  MsSmem L;
  size_t off = 0;
  L.bars = off;
  off += 256;  // full[6], empty[6], act, peer_full[2], peer_free[2]
  L.hdr = off;
  off += (size_t)m_pad * 8;
  L.flags = off;
  off += 16;
  L.acts = off;
  off += (size_t)groups_per_rank * m_pad * kMsActRowBytes;
  off = (off + 127) & ~(size_t)127;
  L.ring = off;
  off += (size_t)kMsStages * kMsStageBytes;
  L.red = off;
  off += (size_t)ks * m_pad * 32 * 4;
  L.psum = off;
  if (cluster_size > 1) off += (size_t)2 * m_pad * 32 * 4;
  L.total = off;
  return L;
}

__device__ __forceinline__ uint32_t ms_lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 ms_lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t ms_lds16(uint32_t a) {
  uint32_t v;
  asm volatile("{\n\t.reg .u16 t;\n\tld.shared.u16 t, [%1];\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float4 ms_ld_cluster_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
// arrive on the same-named mbarrier of CTA `rank`; orders this CTA's earlier writes before it at cluster scope
__device__ __forceinline__ void ms_mbar_arrive_remote(uint64_t* local_bar, uint32_t rank) {
  const uint32_t addr = map_to_cta(local_bar, rank);
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ bool ms_mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool ms_mbar_wait_cluster_bounded(uint64_t* bar, uint32_t parity) {
  if (ms_mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  while (!ms_mbar_try_wait_cluster(bar, parity)) {
    if (clock64() - t0 > (1ll << 31)) {
      atomicOr(&g_device_status, kDevStatusTimeout);
      return false;
    }
  }
  return true;
}
// D (s32, 16 x 8) = A (u8, 16 x 32, row-major) * B (s8, 32 x 8, column-major) + C, where C holds c0 in the columns
// 2 (lane % 4) and c1 in the columns 2 (lane % 4) + 1 of both of the lane's rows
__device__ __forceinline__ void ms_mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, int c0, int c1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %10, %11};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}
__device__ __forceinline__ void ms_compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kMsCThreads) : "memory"); }

// NTW: 8-column tiles of the batch per warp (1, 2, 4); NS: warps side by side along the batch (1, 2).
// The other kMsCWarps / NS warps split the K-groups of a stage.
template <int NTW, int NS>
__global__ void __launch_bounds__(kMsThreads, 1) w4a32_gemm_stream_kernel(const __grid_constant__ MsParams p) {
  constexpr int KS = kMsCWarps / NS;
  extern __shared__ __align__(128) uint8_t ms_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int S = p.cluster_size, G = p.num_groups, m_pad = p.m_pad;
  const uint32_t rank = S > 1 ? cluster_ctarank() : 0u;
  const int cluster = (int)blockIdx.x / S;
  const int g_lo = (int)(((long long)rank * G) / S), g_hi = (int)(((long long)(rank + 1) * G) / S);
  const int ng = g_hi - g_lo;
  const MsSmem Lo = ms_smem_layout(m_pad, (G + S - 1) / S, S, KS);
  uint64_t* full = reinterpret_cast<uint64_t*>(ms_smem + Lo.bars);
  uint64_t* empty = full + kMsStages;
  uint64_t* act_bar = empty + kMsStages;
  uint64_t* peer_full = act_bar + 1;   // [2] rank 0: the other ranks' partial sums of a unit are in place
  uint64_t* peer_free = peer_full + 2; // [2] ranks 1..: rank 0 has read the slot
  float2* s_hdr = reinterpret_cast<float2*>(ms_smem + Lo.hdr);
  volatile int* flags = reinterpret_cast<volatile int*>(ms_smem + Lo.flags);
  uint8_t* acts = ms_smem + Lo.acts;
  uint8_t* ring = ms_smem + Lo.ring;
  float* red = reinterpret_cast<float*>(ms_smem + Lo.red);
  float* psum = reinterpret_cast<float*>(ms_smem + Lo.psum);
  const size_t group_bytes = (size_t)m_pad * kMsActRowBytes;

  MS_STAMP(0, clock64());
  if (p.use_pdl) pdl_launch_dependents();
  if (tid == 0) {
    for (int i = 0; i < kMsStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kMsCWarps);
    }
    mbar_init(act_bar, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&peer_full[i], (uint32_t)max(S - 1, 1));
      mbar_init(&peer_free[i], 1);
    }
    mbar_fence_init();
    // tile headers: checked before a single byte of a matrix is requested
    int bad = 0;
    for (int i = 0; i < p.num_problems; ++i) {
      const uint4 h = *reinterpret_cast<const uint4*>(p.prob[i].tiled);  // magic, version, n, k
      if (h.x != kTiledMagic || h.z != (uint32_t)p.prob[i].n || h.w != (uint32_t)p.k) bad = 1;
    }
    if (bad) atomicOr(&g_device_status, kDevStatusBadHeader);
    flags[0] = bad;  // 1: nothing is done
    flags[1] = 0;    // set when a wait ran out
  }
  __syncthreads();
  if (S > 1) cluster_sync_all();  // every CTA of the cluster runs and has its barriers initialised
  const bool run = flags[0] == 0;
  const int first_unit = run ? cluster : p.total_panels;

  auto problem_of = [&](int u) {
    int pi = 0;
#pragma unroll
    for (int i = 1; i < kMsMaxProblems; ++i)
      if (i < p.num_problems && u >= p.prob[i].panel_begin) pi = i;
    return pi;
  };

  if (warp == kMsCWarps) {
    // =============================== producer warp (one lane) ===============================
    if (lane == 0 && ng > 0) {
      const uint64_t stream_once = l2_policy_evict_first();
      int st = 0, issued = 0;
      uint32_t ph = 0;
      bool acts_requested = false;
      auto request_acts = [&] {
        if (p.use_pdl) pdl_wait_prior();  // the activation blocks come from the kernel before this one
        const uint32_t bytes = (uint32_t)((size_t)ng * group_bytes);
        mbar_arrive_expect_tx(act_bar, bytes);
        bulk_g2s(acts, p.acts + (size_t)g_lo * group_bytes, bytes, act_bar);
        acts_requested = true;
      };
      bool ok = true;
      for (int u = first_unit; u < p.total_panels && ok; u += p.num_clusters) {
        const int pi = problem_of(u);
        const MsProblem& pr = p.prob[pi];
        const uint8_t* panel_cells = pr.tiled + sizeof(TiledHeader) + (size_t)(u - pr.panel_begin) * G * kCellBytes;
        for (int b = g_lo; b < g_hi; b += kMsBlockGroups) {
          if (issued == kMsStages && !acts_requested) request_acts();  // the ring is full of weights: now the activations
          if (issued >= kMsStages) {
            if (!mbar_wait_bounded(&empty[st], ph ^ 1u)) {
              flags[1] = 1;
              ok = false;
              break;
            }
          }
          const uint32_t bytes = (uint32_t)(min(kMsBlockGroups, g_hi - b) * kCellBytes);
          mbar_arrive_expect_tx(&full[st], bytes);
          bulk_g2s_hint(ring + (size_t)st * kMsStageBytes, panel_cells + (size_t)b * kCellBytes, bytes, &full[st], stream_once);
          ++issued;
          if (++st == kMsStages) {
            st = 0;
            ph ^= 1u;
          }
        }
      }
      if (!acts_requested) request_acts();  // (also when there is no unit: the compute warps wait for it)
    }
    __syncwarp();
  } else {
    // =============================== compute warps ===============================
    const int ks = warp % KS, ns = warp / KS;
    const int g8 = lane >> 2, c4 = lane & 3;
    const int n_tiles = m_pad >> 3;
    MS_STAMP(1, clock64());
    if (p.use_pdl) pdl_wait_prior();
    MS_STAMP(2, clock64());
    for (int i = tid; i < m_pad; i += kMsCThreads) s_hdr[i] = i < p.m ? p.a_hdr[i] : make_float2(0.0f, 0.0f);
    bool ok = ng <= 0 || mbar_wait_bounded(act_bar, 0);  // also publishes nothing else: s_hdr is read after the first unit's barrier
    MS_STAMP(3, clock64());
    long long wait_full = 0, t_loop = 0, t_tail = 0;
    const uint32_t ring_s = smem_u32(ring), acts_s = smem_u32(acts), red_s = smem_u32(red);
    const uint32_t lo_off = (uint32_t)(g8 * 16 + c4 * 4);                  // this lane's word of a row block
    const uint32_t hi_base = (uint32_t)m_pad * 16, sum_base = (uint32_t)m_pad * 32;

    float acc[2][NTW][4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int t = 0; t < NTW; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][t][i] = 0.0f;

    int st = 0, unit_index = 0;
    uint32_t ph = 0;
    for (int u = first_unit; u < p.total_panels; u += p.num_clusters, ++unit_index) {
      const int pi = problem_of(u);
      const MsProblem& pr = p.prob[pi];
      const bool f16 = reinterpret_cast<const TiledHeader*>(pr.tiled)->scale_mode == 2u;
      // the per-row constants of the epilogue are requested now and used after the last stage of the unit
      const int slots = n_tiles * 64;  // float4 slots of a unit: (column tile, half, lane)
      const int panel = u - pr.panel_begin;
      float zs[kMsSlotsPerThread][2], bs[kMsSlotsPerThread][2];
#pragma unroll
      for (int q = 0; q < kMsSlotsPerThread; ++q) {
        const int e4 = tid + q * kMsCThreads;
        zs[q][0] = zs[q][1] = bs[q][0] = bs[q][1] = 0.0f;
        if (e4 < slots && rank == 0) {
          const int row0 = 16 * ((e4 >> 5) & 1) + ((e4 & 31) >> 2);
          const float* zsum = reinterpret_cast<const float*>(pr.tiled + pr.zsum_off) + (size_t)panel * kPanelRows;
          const float* bias = reinterpret_cast<const float*>(pr.tiled + pr.bias_off) + (size_t)panel * kPanelRows;
          zs[q][0] = zsum[row0], zs[q][1] = zsum[row0 + 8];
          bs[q][0] = bias[row0], bs[q][1] = bias[row0 + 8];
        }
      }
      const long long tl0 = clock64();
      for (int b = g_lo; b < g_hi && ok; b += kMsBlockGroups) {
        const long long tw0 = clock64();
        if (!mbar_wait_bounded(&full[st], ph)) {
          ok = false;
          break;
        }
        wait_full += clock64() - tw0;
        const int cnt = min(kMsBlockGroups, g_hi - b);
        // Two cells per trip (K-groups j and j + KS of the stage), their loads and tensor-core products interleaved:
        // with two warps per scheduler the dependent chain of a single cell would leave the pipes idle.
        // The accumulator of a product starts at 0x4B400000 - 8 * sum(a_q): the s32 result, read as a float, is then
        // 12582912 + value exactly (|value| <= 32768), and one FADD replaces the integer-to-float conversion.
        for (int j = ks; j < cnt; j += 2 * KS) {
          const bool two = j + KS < cnt;
          const uint32_t cell0 = ring_s + (uint32_t)st * kMsStageBytes + (uint32_t)j * kCellBytes;
          const uint32_t cell1 = two ? cell0 + (uint32_t)KS * kCellBytes : cell0;
          const uint32_t ag0 = acts_s + (uint32_t)(b - g_lo + j) * (uint32_t)group_bytes;
          const uint32_t ag1 = two ? ag0 + (uint32_t)KS * (uint32_t)group_bytes : ag0;
          // weights: rows g8, g8 + 8 of either 16-row half; 4 bytes = 8 nibbles = k {4 c4 .. 4 c4 + 3} low and high
          uint32_t w0[4], w1[4];
          uint32_t r0[4], r1[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            w0[i] = ms_lds32(cell0 + lo_off + (uint32_t)i * 128);
            w1[i] = ms_lds32(cell1 + lo_off + (uint32_t)i * 128);
            r0[i] = ms_lds16(cell0 + kCellNibbleBytes + (uint32_t)(g8 + 8 * i) * 2);
            r1[i] = ms_lds16(cell1 + kCellNibbleBytes + (uint32_t)(g8 + 8 * i) * 2);
          }
          float sc0[4], sc1[4];
          uint32_t a0[2][4], a1[2][4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            sc0[i] = f16 ? __half2float(__ushort_as_half((unsigned short)r0[i])) : __uint_as_float(r0[i] << 16);
            sc1[i] = f16 ? __half2float(__ushort_as_half((unsigned short)r1[i])) : __uint_as_float(r1[i] << 16);
            if (!two) sc1[i] = 0.0f;  // the second cell of an odd trip repeats the first with scale 0
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            a0[h][0] = w0[2 * h] & 0x0F0F0F0Fu, a0[h][1] = w0[2 * h + 1] & 0x0F0F0F0Fu;
            a0[h][2] = (w0[2 * h] >> 4) & 0x0F0F0F0Fu, a0[h][3] = (w0[2 * h + 1] >> 4) & 0x0F0F0F0Fu;
            a1[h][0] = w1[2 * h] & 0x0F0F0F0Fu, a1[h][1] = w1[2 * h + 1] & 0x0F0F0F0Fu;
            a1[h][2] = (w1[2 * h] >> 4) & 0x0F0F0F0Fu, a1[h][3] = (w1[2 * h + 1] >> 4) & 0x0F0F0F0Fu;
          }
          constexpr int kMagic = 0x4B400000;  // 12582912.0f: ulp 1 up to +-2^22 around it
#pragma unroll
          for (int t = 0; t < NTW; ++t) {
            const int nt = ns * NTW + t;
            if (nt < n_tiles) {
              const uint32_t col = (uint32_t)nt * 128 + lo_off;  // 8 rows x 16 bytes per column tile
              const uint32_t sum_at = sum_base + (uint32_t)(nt * 8 + 2 * c4) * 4;  // -8 * sum(a_q) of columns 2 c4, 2 c4 + 1
              const uint32_t p0 = ms_lds32(ag0 + col), q0 = ms_lds32(ag0 + hi_base + col);
              const uint32_t p1 = ms_lds32(ag1 + col), q1 = ms_lds32(ag1 + hi_base + col);
              const uint2 s0 = ms_lds64(ag0 + sum_at), s1 = ms_lds64(ag1 + sum_at);
              int d0[2][4], d1[2][4];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                ms_mma_u8s8(d0[h], a0[h], p0, q0, (int)s0.x + kMagic, (int)s0.y + kMagic);
                ms_mma_u8s8(d1[h], a1[h], p1, q1, (int)s1.x + kMagic, (int)s1.y + kMagic);
              }
#pragma unroll
              for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float f0 = __int_as_float(d0[h][i]) - 12582912.0f, f1 = __int_as_float(d1[h][i]) - 12582912.0f;
                  acc[h][t][i] = fmaf(f0, sc0[2 * h + (i >> 1)], acc[h][t][i]);
                  acc[h][t][i] = fmaf(f1, sc1[2 * h + (i >> 1)], acc[h][t][i]);
                }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
        if (++st == kMsStages) {
          st = 0;
          ph ^= 1u;
        }
      }
      const long long tl1 = clock64();
      t_loop += tl1 - tl0;
      // ---- end of the unit: the K-slices of the warps meet in shared memory
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int t = 0; t < NTW; ++t) {
          const int nt = ns * NTW + t;
          if (nt < n_tiles) {
            const uint32_t at = red_s + (uint32_t)(((ks * n_tiles + nt) * 2 + h) * 32 + lane) * 16;
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(at), "f"(acc[h][t][0]), "f"(acc[h][t][1]),
                         "f"(acc[h][t][2]), "f"(acc[h][t][3])
                         : "memory");
          }
          acc[h][t][0] = acc[h][t][1] = acc[h][t][2] = acc[h][t][3] = 0.0f;
        }
      ms_compute_sync();
      const int buf = unit_index & 1;
      // ranks 1..: the slot written two units ago must have been read by rank 0
      if (S > 1 && rank != 0 && unit_index >= 2 && ok)
        ok = ms_mbar_wait_cluster_bounded(&peer_free[buf], (uint32_t)((unit_index >> 1) - 1) & 1u);
      if (S > 1 && rank == 0 && ok) ok = ms_mbar_wait_cluster_bounded(&peer_full[buf], (uint32_t)(unit_index >> 1) & 1u);
#pragma unroll
      for (int q = 0; q < kMsSlotsPerThread; ++q) {
        const int e4 = tid + q * kMsCThreads;
        if (e4 >= slots) break;
        float4 v = *reinterpret_cast<const float4*>(red + (size_t)e4 * 4);
        for (int r = 1; r < KS; ++r) {
          const float4 o = *reinterpret_cast<const float4*>(red + ((size_t)r * slots + e4) * 4);
          v.x += o.x, v.y += o.y, v.z += o.z, v.w += o.w;
        }
        if (S > 1 && rank != 0) {
          *reinterpret_cast<float4*>(psum + ((size_t)buf * slots + e4) * 4) = v;
          continue;
        }
        if (S > 1 && ok) {
          for (uint32_t r = 1; r < (uint32_t)S; ++r) {
            const float4 o = ms_ld_cluster_f32x4(map_to_cta(psum + ((size_t)buf * slots + e4) * 4, r));
            v.x += o.x, v.y += o.y, v.z += o.z, v.w += o.w;
          }
        }
        // epilogue: slot = (column tile nt, half h, lane l): rows 16 h + l / 4 (+ 8), columns 8 nt + 2 (l % 4) (+ 1)
        const int nt = e4 >> 6, h = (e4 >> 5) & 1, l = e4 & 31;
        const int row0 = 16 * h + (l >> 2), col0 = 8 * nt + 2 * (l & 3);
        const float vals[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = row0 + (i >> 1) * 8, col = col0 + (i & 1);
          const int n = panel * kPanelRows + row;
          if (n < pr.n && col < p.m && ok) {
            const float2 hc = s_hdr[col];
            float o = fmaf((float)__float_as_int(hc.y), zs[q][i >> 1], vals[i]);
            o = fmaf(o, hc.x, bs[q][i >> 1]);
            pr.y[(size_t)col * pr.ldy + n] = clamp_flt_max(o);
          }
        }
      }
      ms_compute_sync();  // red (and, for rank 0, the peers' slots) are read: the next unit may overwrite them
      t_tail += clock64() - tl1;
      if (S > 1 && tid == 0) {
        if (rank != 0) ms_mbar_arrive_remote(&peer_full[buf], 0);  // our partial sums of this unit are in place
        else
          for (uint32_t r = 1; r < (uint32_t)S; ++r) ms_mbar_arrive_remote(&peer_free[buf], r);
      }
    }
    if (!ok && lane == 0) flags[1] = 1;
    MS_STAMP(4, clock64());
    MS_STAMP(5, wait_full);
    MS_STAMP(6, t_loop);
    MS_STAMP(7, t_tail);
    MS_STAMP(8, unit_index);
  }
  // Leave together: ranks 1.. hold partial sums that rank 0 reads, rank 0 holds the barriers they arrive on.
  __syncthreads();
  if (S > 1) cluster_sync_all();
}

// ------------------------------------------------------------------------------------------------ activations
// Per-row int8 quantization (the arithmetic of act_quant_records_kernel) into the layout above: for K-group g
// and row m the four low words (even k of each 8-value item) at [g][m][0..16), the four high words (odd k) at
// [g][m_pad + m] ... , -8 * sum at [g][2 m_pad ... ].  One CTA per row of the padded batch; padding rows are zeros.
constexpr int kMsQuantThreads = 256;
__global__ void __launch_bounds__(kMsQuantThreads) act_quant_mma_kernel(const float* __restrict__ x, int m_total, int m_pad,
                                                                        int k, int ldx, int num_groups,
                                                                        uint8_t* __restrict__ acts, float2* __restrict__ hdr,
                                                                        int use_pdl) {
  __shared__ float scratch[64];
  if (use_pdl) {
    pdl_launch_dependents();
    pdl_wait_prior();  // x may be the previous kernel's output, and that kernel may still read the blocks we overwrite
  }
  const int m = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool live = m < m_total;
  const float* row = x + (size_t)(live ? m : 0) * ldx;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
  const int num_items = num_groups * 4;
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
  if (live) {
    if (vec) {
      for (int i = tid; i < (k >> 2); i += kMsQuantThreads) {
        const float4 v = reinterpret_cast<const float4*>(row)[i];
        mn = fminf(mn, fminf(fminf(v.x, v.y), fminf(v.z, v.w)));
        mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
      }
      for (int i = (k & ~3) + tid; i < k; i += kMsQuantThreads) {
        mn = fminf(mn, row[i]);
        mx = fmaxf(mx, row[i]);
      }
    } else {
      for (int i = tid; i < k; i += kMsQuantThreads) {
        mn = fminf(mn, row[i]);
        mx = fmaxf(mx, row[i]);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0) {
    scratch[warp] = mn;
    scratch[32 + warp] = mx;
  }
  __syncthreads();
  mn = lane < kMsQuantThreads / 32 ? scratch[lane] : 3.402823466e+38f;
  mx = lane < kMsQuantThreads / 32 ? scratch[32 + lane] : -3.402823466e+38f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const ActQuantParams qp = act_quant_params(mn, mx);
  if (live && tid == 0) hdr[m] = make_float2(qp.recip_scale, __int_as_float(-qp.nzp));
  const size_t group_bytes = (size_t)m_pad * kMsActRowBytes;
  for (int base = 0; base < num_items; base += kMsQuantThreads) {  // uniform trip count: full warps at the shuffles
    const int item = base + tid;
    const bool valid = item < num_items;
    const int k0 = item * 8;
    int q8[8];
    if (live && valid && vec && k0 + 8 <= k) {
      const float4 a = *reinterpret_cast<const float4*>(row + k0);
      const float4 b = *reinterpret_cast<const float4*>(row + k0 + 4);
      const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) q8[j] = act_quant_value(f[j], qp);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) q8[j] = (live && valid && k0 + j < k) ? act_quant_value(row[k0 + j], qp) : 0;
    }
    const uint32_t lo = ((uint32_t)q8[0] & 0xFFu) | (((uint32_t)q8[2] & 0xFFu) << 8) | (((uint32_t)q8[4] & 0xFFu) << 16) |
                        (((uint32_t)q8[6] & 0xFFu) << 24);
    const uint32_t hi = ((uint32_t)q8[1] & 0xFFu) | (((uint32_t)q8[3] & 0xFFu) << 8) | (((uint32_t)q8[5] & 0xFFu) << 16) |
                        (((uint32_t)q8[7] & 0xFFu) << 24);
    int s = q8[0] + q8[1] + q8[2] + q8[3] + q8[4] + q8[5] + q8[6] + q8[7];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (valid) {
      const int g = item >> 2, i = item & 3;
      uint8_t* grp = acts + (size_t)g * group_bytes;
      reinterpret_cast<uint32_t*>(grp + (size_t)m * 16)[i] = lo;
      reinterpret_cast<uint32_t*>(grp + (size_t)m_pad * 16 + (size_t)m * 16)[i] = hi;
      if (i == 0) reinterpret_cast<int*>(grp + (size_t)m_pad * 32)[m] = -8 * s;
    }
  }
}

// ------------------------------------------------------------------------------------------------ host side
struct MsPlan {
  int m_pad, cluster_size, num_clusters, total_panels, ks, ntw, ns;
  size_t smem;
};

template <int NTW, int NS>
static cudaError_t ms_configure() {
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && configured[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(w4a32_gemm_stream_kernel<NTW, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64) configured[dev] = true;
  return cudaSuccess;
}

// clusters of `s` CTAs of this kernel that the current device runs at once (148 / s without a device)
template <int NTW, int NS>
static int ms_cluster_capacity(int s, size_t smem) {
  if (s <= 1) return 148;
  int n = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(s * 148), 1, 1);
  cfg.blockDim = dim3(kMsThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = (unsigned)s;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (ms_configure<NTW, NS>() != cudaSuccess ||
      cudaOccupancyMaxActiveClusters(&n, w4a32_gemm_stream_kernel<NTW, NS>, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = 148 / s;
  }
  return n;
}

static bool ms_shape_plan(int m, int k, int count, const int* n, MsPlan* plan) {
  if (m < 1 || m > kMsMaxM || count < 1 || count > kMsMaxProblems || k < 1) return false;
  const int G = (k + kGroup - 1) / kGroup;
  plan->m_pad = (m + 7) / 8 * 8;
  const int n_tiles = plan->m_pad / 8;
  plan->ntw = n_tiles <= 1 ? 1 : (n_tiles <= 2 ? 2 : 4);
  plan->ns = n_tiles > 4 ? 2 : 1;
  plan->ks = kMsCWarps / plan->ns;
  int S = 0;
  for (int s = 1; s <= kMsMaxCluster; ++s)
    if ((size_t)((G + s - 1) / s) * plan->m_pad * kMsActRowBytes <= kMsActBudget) {
      S = s;
      break;
    }
  if (S == 0 || S > G) return false;
  plan->cluster_size = S;
  long long panels = 0;
  for (int i = 0; i < count; ++i) {
    if (n[i] < 1) return false;
    panels += (n[i] + kPanelRows - 1) / kPanelRows;
  }
  if (panels >= (1ll << 30)) return false;
  plan->total_panels = (int)panels;
  plan->smem = ms_smem_layout(plan->m_pad, (G + S - 1) / S, S, plan->ks).total;
  return plan->smem <= 227 * 1024;
}

bool w4a32_gemm_stream_supported(int m, int k, int count, const int* n) {
  MsPlan plan;
  return m >= 1 && ms_shape_plan(m, k, count, n, &plan);
}

// bytes of the activation blocks for m rows of k values (rows padded to a multiple of 8)
size_t w4a32_gemm_stream_act_bytes(int m, int k) {
  return (size_t)((k + kGroup - 1) / kGroup) * (size_t)((m + 7) / 8 * 8) * kMsActRowBytes;
}

cudaError_t launch_act_quant_mma(const float* x, int m, int k, int ldx, uint8_t* acts, float2* hdr, int use_pdl,
                                 cudaStream_t stream) {
  const int m_pad = (m + 7) / 8 * 8, num_groups = (k + kGroup - 1) / kGroup;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)m_pad, 1, 1);
  cfg.blockDim = dim3(kMsQuantThreads, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  if (use_pdl) {
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, act_quant_mma_kernel, x, m, m_pad, k, ldx, num_groups, acts, hdr, use_pdl);
}

template <int NTW, int NS>
static cudaError_t ms_launch_t(MsParams& prm, const MsPlan& plan, cudaStream_t stream) {
  cudaError_t e = ms_configure<NTW, NS>();
  if (e != cudaSuccess) return e;
  const int S = plan.cluster_size;
  static int capacity[64][kMsMaxCluster + 1] = {};  // per device and cluster size (the largest shared-memory need is assumed)
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (capacity[dev][S] == 0) capacity[dev][S] = ms_cluster_capacity<NTW, NS>(S, 227 * 1024);
  prm.num_clusters = std::max(1, std::min(std::min(capacity[dev][S], 148 / S), plan.total_panels));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(prm.num_clusters * S), 1, 1);
  cfg.blockDim = dim3(kMsThreads, 1, 1);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (S > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = (unsigned)S;
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
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, w4a32_gemm_stream_kernel<NTW, NS>, prm);
}

// acts / a_hdr: output of launch_act_quant_mma for the same m and k.  Up to four matrices that share them.
cudaError_t launch_w4a32_gemm_stream(const uint8_t* acts, const float2* a_hdr, int m, int k, int count,
                                     const void* const* tiled, float* const* y, const int* n, const int* ldy, int use_pdl,
                                     cudaStream_t stream) {
  MsPlan plan;
  if (!ms_shape_plan(m, k, count, n, &plan)) return cudaErrorInvalidValue;
  MsParams prm = {};
  prm.acts = acts;
  prm.a_hdr = a_hdr;
  prm.m = m;
  prm.m_pad = plan.m_pad;
  prm.k = k;
  prm.num_groups = (k + kGroup - 1) / kGroup;
  prm.cluster_size = plan.cluster_size;
  prm.total_panels = plan.total_panels;
  prm.num_problems = count;
  prm.use_pdl = use_pdl;
  int begin = 0;
  for (int i = 0; i < count; ++i) {
    const TiledHeader th = make_tiled_header(n[i], k, 0, 0);
    prm.prob[i].tiled = static_cast<const uint8_t*>(tiled[i]);
    prm.prob[i].y = y[i];
    prm.prob[i].n = n[i];
    prm.prob[i].ldy = ldy[i];
    prm.prob[i].num_panels = (int)th.num_panels;
    prm.prob[i].panel_begin = begin;
    prm.prob[i].zsum_off = th.zsum_off;
    prm.prob[i].bias_off = th.bias_off;
    begin += (int)th.num_panels;
  }
  if (plan.ns == 2) return ms_launch_t<4, 2>(prm, plan, stream);
  switch (plan.ntw) {
    case 1: return ms_launch_t<1, 1>(prm, plan, stream);
    case 2: return ms_launch_t<2, 1>(prm, plan, stream);
    default: return ms_launch_t<4, 1>(prm, plan, stream);
  }
}

}  // namespace mllmb200
