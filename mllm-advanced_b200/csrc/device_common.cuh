// Device-side helpers shared by the sm_100a kernels: status word, bounded mbarrier waits,
// bulk-copy and cluster PTX wrappers, and the activation-quantization parameter math.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <cuda_fp16.h>

#include "layout.h"

namespace mllmb200 {

// Bits of the device status word (see mllmb200_check_device_status).
enum : unsigned {
  kDevStatusTimeout = 1u,    // a bounded wait on an mbarrier ran out
  kDevStatusBadHeader = 2u,  // tiled buffer header does not match the call's N/K
};

extern __device__ unsigned int g_device_status;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  // make barrier initialisation visible to the async proxy (bulk copies, tensor-core commits)
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity, at most ~2^31 clock ticks (about a second).
// Returns false and raises the timeout bit in the status word when the wait runs out, so a
// lost copy shows up as an error code on the host instead of a hung GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, long long limit_ticks = 1ll << 31) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > limit_ticks) {
      atomicOr(&g_device_status, kDevStatusTimeout);
      return false;
    }
  }
  return true;
}

// flag in global memory, written by one CTA and polled by another of the same GPU
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// 1-D bulk copy global -> shared of this CTA; completion counted in bytes on `bar`.
// src, dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// L2 replacement policy for bytes that are read once (a weight matrix streamed through): first in line for
// eviction, so that they do not push the activations, outputs and per-row constants out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Split form: arrive early, wait later (hides the barrier latency behind independent work).
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Address of `local_smem` in the shared memory of CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(const void* local_smem, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(local_smem)), "r"(rank));
  return out;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start its prologue, and
// wait for the previous kernel's memory before touching data it may have produced.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Every CTA checks the tile header before it requests a single byte of the matrix: true when magic, row
// count and K are what the call claims (a call whose N or K is larger than the buffer would otherwise read
// past its end).  Called by ALL threads of the CTA (it synchronizes them); on a mismatch the bad-header bit
// of the status word is raised and the CTA must return without touching the matrix.
__device__ __forceinline__ bool tiled_header_ok_cta(const uint8_t* tiled, int n, int k) {
  int bad = 0;
  if (threadIdx.x == 0) {
    const uint4 h = *reinterpret_cast<const uint4*>(tiled);  // magic, version, n, k
    bad = !(h.x == kTiledMagic && h.z == (uint32_t)n && h.w == (uint32_t)k);
    if (bad) atomicOr(&g_device_status, kDevStatusBadHeader);
  }
  return __syncthreads_or(bad) == 0;
}

// ------------------------------------------------------------------ scale decode
__device__ __forceinline__ float decode_scale(uint32_t raw16, uint32_t scale_mode) {
  const float as_bf16 = __uint_as_float(raw16 << 16);
  const float as_f16 = __half2float(__ushort_as_half((unsigned short)raw16));
  return scale_mode == 2u ? as_f16 : as_bf16;
}

// ------------------------------------------------------------------ activation quantization
// Per-row parameters of the dynamic asymmetric int8 quantization
// (reference project: tests/Arm/KaiLinearTest.hpp:163-205).  Every operation is a separately
// rounded fp32 operation (no fused multiply-add), as in the scalar reference.
struct ActQuantParams {
  float scale0;       // multiplier 255 / (rmax - rmin)
  float recip_scale;  // 1 / scale0, the "lhs_scale" applied to the output
  int nzp;            // nudged zero point; a_off = -nzp
};

__device__ __forceinline__ ActQuantParams act_quant_params(float min0, float max0) {
  const float qmin = -128.0f, qmax = 127.0f;
  const float rmin0 = min0 < 0.0f ? min0 : 0.0f;
  const float rmax0 = 0.0f < max0 ? max0 : 0.0f;
  const float scale0 = rmin0 == rmax0 ? 1.0f : __fdiv_rn(__fsub_rn(qmax, qmin), __fsub_rn(rmax0, rmin0));
  const float recip = scale0 != 0.0f ? __fdiv_rn(1.0f, scale0) : 0.0f;
  const float dmin = __fmul_rn(rmin0, scale0);
  const float dmax = __fmul_rn(rmax0, scale0);
  const float zp_min_err = __fadd_rn(qmin, dmin);
  const float zp_max_err = __fadd_rn(qmax, dmax);
  float zp = __fadd_rn(zp_min_err, zp_max_err) > 0.0f ? __fsub_rn(qmin, dmin) : __fsub_rn(qmax, dmax);
  zp = zp < qmin ? qmin : zp;
  zp = qmax < zp ? qmax : zp;
  ActQuantParams p;
  p.scale0 = scale0;
  p.recip_scale = recip;
  p.nzp = __float2int_rn(zp);  // lrintf: round half to even
  return p;
}

// a_q = clamp(round_half_away(x * scale0) + nzp, -128, 127)   (KaiLinearTest.hpp:217-226)
__device__ __forceinline__ int act_quant_value(float x, const ActQuantParams& p) {
  int v = (int)roundf(__fmul_rn(x, p.scale0));
  v += p.nzp;
  v = max(v, -128);
  v = min(v, 127);
  return v;
}

// Block-wide min and max over a row of `k` floats; every thread gets the result.
// scratch: 2 * 32 floats of shared memory.
__device__ __forceinline__ void block_row_minmax(const float* __restrict__ row, int k, float* scratch,
                                                 float& out_min, float& out_max) {
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
  const int tid = threadIdx.x, nt = blockDim.x;
  if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
    const int k4 = k >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(row);
    for (int i = tid; i < k4; i += nt) {
      const float4 v = r4[i];
      mn = fminf(mn, fminf(fminf(v.x, v.y), fminf(v.z, v.w)));
      mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
    }
    for (int i = (k4 << 2) + tid; i < k; i += nt) {
      mn = fminf(mn, row[i]);
      mx = fmaxf(mx, row[i]);
    }
  } else {
    for (int i = tid; i < k; i += nt) {
      mn = fminf(mn, row[i]);
      mx = fmaxf(mx, row[i]);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const int warp = tid >> 5, lane = tid & 31, nw = (nt + 31) >> 5;
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) {
    scratch[warp] = mn;
    scratch[32 + warp] = mx;
  }
  __syncthreads();
  mn = lane < nw ? scratch[lane] : 3.402823466e+38f;
  mx = lane < nw ? scratch[32 + lane] : -3.402823466e+38f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  out_min = mn;
  out_max = mx;
}

__device__ __forceinline__ float clamp_flt_max(float v) {
  // the reference clamps to [-FLT_MAX, FLT_MAX] (mllm/Backends/Arm/Kernels/kai_linear.cpp:393)
  v = v < -3.402823466e+38f ? -3.402823466e+38f : v;
  v = 3.402823466e+38f < v ? 3.402823466e+38f : v;
  return v;
}

}  // namespace mllmb200
