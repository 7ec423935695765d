// Tensor parallelism for the W4A32 linear over the GPUs of one node (one process per GPU).
//
// Output channels (rows of W) are sharded: rank r holds rows [r N/g, (r+1) N/g) in the tile layout (the repack
// takes a row range) and x is replicated, so a rank's result is the column block [:, r N/g : (r+1) N/g] of y and
// needs no reduction - only to be delivered to every rank.  The reference project has no multi-device path
// (its engine is single-device, mllm/Engine/Context.cpp:56-59); the contract here is the benchmark's: every rank
// ends up with the full fp32 y [M, N].
//
// Gather modes:
//   2  fused (the product): the output buffers of all ranks are mapped into every process (CUDA IPC, exchanged
//      once over the caller's NCCL communicator), and the kernels' epilogues store every finished element into
//      all of them at the rank's column offset - plain stores over NVLink / NVSwitch, tile by tile, while the
//      other tiles are still being computed.  A rank then tells every peer "my block has landed" by a flag in
//      the peer's memory and waits (bounded) for the peers' flags.
//   1  NCCL baseline: the rank's block goes to a contiguous staging buffer, ncclAllGather concatenates the
//      blocks as [g][M][N/g], a kernel re-assembles [M][N].
//   0  none: the rank's own column block only.
// No kernel of another library is ever handed a peer pointer; peer memory is only written with plain st.global.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>  // types and prototypes only: the entry points are looked up in the NCCL the process already loaded

#include <algorithm>
#include <cstring>
#include <vector>

#include "../../include/mllmb200.h"
#include "device_common.cuh"

namespace mllmb200 {
int record_cuda_failure(cudaError_t e);
size_t w4a32_ws_rec_bytes(int m, int k);
int* w4a32_ws_split_sync(void* ws_dev, int m, int k);
int w4a32_ws_split_sync_ints();
cudaError_t launch_w4a32_gemv_stream(int count, const float* const* x, const int* ldx, const uint8_t* const* a_rec,
                                     const float2* const* a_hdr, int m, const int* k, const void* const* tiled,
                                     float* const* y, const int* n, const int* ldy, int use_pdl, cudaStream_t stream,
                                     int num_peers, float* const* y_peers);
bool w4a32_gemv_stream_supported(int m, int count, const int* k, const int* n);
bool w4a32_gemm_tcf16_preferred(int m, int k, int n);
int w4a32_gemm_tcf16_m_pad(int m, int n);
cudaError_t launch_act_quant_blocks_f16(const float*, int, int, int, int, uint8_t*, float2*, cudaStream_t, int use_pdl = 0,
                                        int* clear_ints = nullptr, int clear_count = 0);
cudaError_t launch_w4a32_gemm_tcf16_grouped(const uint8_t*, const float2*, int, int, int, const void* const*, float* const*,
                                            const int*, const int*, cudaStream_t, int num_peers, float* const* y_peers,
                                            int use_pdl = 0, int* split_sync = nullptr, int split_sync_ints = 0);

constexpr int kTpMaxRanks = 8;
constexpr long long kTpWaitTicks = 1ll << 32;  // ~2 s: ranks reach a collective call milliseconds apart at worst

struct TpIpcBlob {  // what a rank publishes: its output buffer and its flag array
  cudaIpcMemHandle_t y, flags;
};

struct TpHandle {
  int nranks = 0, rank = 0;
  ncclComm_t comm = nullptr;
  ncclResult_t (*all_gather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*comm_count)(const ncclComm_t, int*) = nullptr;
  ncclResult_t (*comm_user_rank)(const ncclComm_t, int*) = nullptr;
  float* y_local = nullptr;
  size_t y_bytes = 0;
  unsigned* flags_local = nullptr;         // [nranks]: flags_local[p] = last epoch whose block from rank p has landed here
  float* y_rank[kTpMaxRanks] = {};         // every rank's output buffer as mapped here (own = y_local)
  unsigned* flags_rank[kTpMaxRanks] = {};  // every rank's flag array as mapped here
  float* send_stage = nullptr;             // NCCL mode: [M][N/g] and [g][M][N/g], allocated on first use
  float* recv_stage = nullptr;
  size_t stage_bytes = 0;
  unsigned epoch = 0;
  bool mapped = false;
};

// this rank's "my column block has landed everywhere" to every peer, after the kernels in front of it on the stream
struct TpFlagPtrs {
  unsigned* p[kTpMaxRanks];
};
// Thread p (one per peer): tells peer p that this rank's block of this epoch has landed there (everything the
// kernels in front of this one on the stream stored), then waits until peer p's block has landed here.  The wait is
// bounded: a peer that never arrives raises the timeout bit of the status word instead of hanging the GPU.
__global__ void tp_signal_wait_kernel(TpFlagPtrs f, const unsigned* flags_local, int nranks, int rank, unsigned epoch,
                                      long long limit_ticks) {
  const int p = threadIdx.x;
  if (p >= nranks || p == rank) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.p[p] + rank), "r"(epoch) : "memory");
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags_local + p) : "memory");
    if ((int)(v - epoch) >= 0) return;  // epochs only grow (wrap-safe comparison)
    if (clock64() - t0 > limit_ticks) {
      atomicOr(&g_device_status, kDevStatusTimeout);
      return;
    }
    __nanosleep(100);
  }
}
// [g][M][nl] -> [M][g * nl] (the NCCL mode's re-assembly)
__global__ void tp_reassemble_kernel(const float* __restrict__ gathered, float* __restrict__ y, int g, int m, int nl, int ldy) {
  const size_t total = (size_t)g * m * (nl / 4);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c4 = (int)(i % (nl / 4));
    const size_t rm = i / (nl / 4);
    const int row = (int)(rm % m), r = (int)(rm / m);
    const float4 v = reinterpret_cast<const float4*>(gathered)[i];
    *reinterpret_cast<float4*>(y + (size_t)row * ldy + (size_t)r * nl + c4 * 4) = v;
  }
}

static int tp_fail(cudaError_t e) { return record_cuda_failure(e); }

}  // namespace mllmb200

using namespace mllmb200;

extern "C" {

int mllmb200_w4a32_tp_init(int nranks, int rank, void* nccl_comm, void** handle) {
  if (!handle || nranks < 1 || nranks > kTpMaxRanks || rank < 0 || rank >= nranks) return MLLMB200_INVALID_ARG;
  auto* h = new TpHandle();
  h->nranks = nranks;
  h->rank = rank;
  h->comm = static_cast<ncclComm_t>(nccl_comm);
  if (h->comm) {
    // the communicator was created by the NCCL that is already in the process: use that very library
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW);
    if (lib) {
      h->all_gather = reinterpret_cast<decltype(h->all_gather)>(dlsym(lib, "ncclAllGather"));
      h->comm_count = reinterpret_cast<decltype(h->comm_count)>(dlsym(lib, "ncclCommCount"));
      h->comm_user_rank = reinterpret_cast<decltype(h->comm_user_rank)>(dlsym(lib, "ncclCommUserRank"));
    }
    if (!h->all_gather || !h->comm_count || !h->comm_user_rank) {
      delete h;
      return MLLMB200_UNSUPPORTED;  // no NCCL in the process
    }
    int cnt = -1, ur = -1;
    if (h->comm_count(h->comm, &cnt) != ncclSuccess || h->comm_user_rank(h->comm, &ur) != ncclSuccess || cnt != nranks ||
        ur != rank) {
      delete h;
      return MLLMB200_INVALID_ARG;
    }
  }
  *handle = h;
  return MLLMB200_OK;
}

int mllmb200_w4a32_tp_ipc_export(void* handle, size_t y_bytes, float** y_dev, void* blob_out) {
  auto* h = static_cast<TpHandle*>(handle);
  if (!h || !y_dev || !blob_out || y_bytes == 0 || h->y_local) return MLLMB200_INVALID_ARG;
  cudaError_t e = cudaMalloc(&h->y_local, y_bytes);
  if (e != cudaSuccess) return tp_fail(e);
  h->y_bytes = y_bytes;
  if ((e = cudaMalloc(&h->flags_local, 256)) != cudaSuccess) return tp_fail(e);
  if ((e = cudaMemset(h->flags_local, 0, 256)) != cudaSuccess) return tp_fail(e);
  TpIpcBlob blob;
  std::memset(&blob, 0, sizeof(blob));
  if (h->nranks > 1) {
    if ((e = cudaIpcGetMemHandle(&blob.y, h->y_local)) != cudaSuccess) return tp_fail(e);
    if ((e = cudaIpcGetMemHandle(&blob.flags, h->flags_local)) != cudaSuccess) return tp_fail(e);
  }
  std::memcpy(blob_out, &blob, sizeof(blob));
  *y_dev = h->y_local;
  return MLLMB200_OK;
}

int mllmb200_w4a32_tp_ipc_import(void* handle, const void* all_blobs) {
  auto* h = static_cast<TpHandle*>(handle);
  if (!h || !all_blobs || !h->y_local || h->mapped) return MLLMB200_INVALID_ARG;
  const auto* blobs = static_cast<const TpIpcBlob*>(all_blobs);
  for (int p = 0; p < h->nranks; ++p) {
    if (p == h->rank) {
      h->y_rank[p] = h->y_local;
      h->flags_rank[p] = h->flags_local;
      continue;
    }
    void* py = nullptr;
    void* pf = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&py, blobs[p].y, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return tp_fail(e);
    if ((e = cudaIpcOpenMemHandle(&pf, blobs[p].flags, cudaIpcMemLazyEnablePeerAccess)) != cudaSuccess) return tp_fail(e);
    h->y_rank[p] = static_cast<float*>(py);
    h->flags_rank[p] = static_cast<unsigned*>(pf);
  }
  h->mapped = true;
  return MLLMB200_OK;
}

int mllmb200_w4a32_tp_alloc_output(void* handle, size_t y_bytes, float** y_dev, void* stream) {
  auto* h = static_cast<TpHandle*>(handle);
  if (!h || !y_dev) return MLLMB200_INVALID_ARG;
  if (h->nranks > 1 && !h->comm) return MLLMB200_INVALID_ARG;  // without a communicator use ipc_export / ipc_import
  TpIpcBlob mine;
  int st = mllmb200_w4a32_tp_ipc_export(handle, y_bytes, y_dev, &mine);
  if (st != MLLMB200_OK) return st;
  std::vector<TpIpcBlob> all((size_t)h->nranks);
  all[h->rank] = mine;
  if (h->nranks > 1) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    void *send = nullptr, *recv = nullptr;
    cudaError_t e = cudaMalloc(&send, sizeof(TpIpcBlob));
    if (e != cudaSuccess) return tp_fail(e);
    if ((e = cudaMalloc(&recv, sizeof(TpIpcBlob) * h->nranks)) != cudaSuccess) return tp_fail(e);
    if ((e = cudaMemcpyAsync(send, &mine, sizeof(mine), cudaMemcpyHostToDevice, s)) != cudaSuccess) return tp_fail(e);
    if (h->all_gather(send, recv, sizeof(TpIpcBlob), ncclChar, h->comm, s) != ncclSuccess) return MLLMB200_CUDA_ERROR;
    if ((e = cudaMemcpyAsync(all.data(), recv, sizeof(TpIpcBlob) * h->nranks, cudaMemcpyDeviceToHost, s)) != cudaSuccess) return tp_fail(e);
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return tp_fail(e);
    cudaFree(send);
    cudaFree(recv);
  }
  return mllmb200_w4a32_tp_ipc_import(handle, all.data());
}

int mllmb200_w4a32_linear_forward_tp(void* handle, const float* x_dev, const void* tiled_shard_dev, void* ws_dev, int M,
                                     int K, int N_total, int ldx, int kernel, int gather_mode, void* stream) {
  auto* h = static_cast<TpHandle*>(handle);
  if (!h || !x_dev || !tiled_shard_dev || M <= 0 || K <= 0 || N_total <= 0 || ldx < K || gather_mode < 0 || gather_mode > 2)
    return MLLMB200_INVALID_ARG;
  if (!h->mapped || (size_t)M * N_total * 4 > h->y_bytes) return MLLMB200_INVALID_ARG;
  const int g = h->nranks, r = h->rank;
  if (N_total % (g * 32) != 0) return MLLMB200_UNSUPPORTED;  // equal shards of whole 32-row panels
  const int nl = N_total / g;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* y_blk = h->y_local + (size_t)r * nl;  // this rank's column block inside the full [M, N_total]
  const int use_pdl = (kernel >> 8) & 1;
  const int policy = kernel & 0xFF;

  if (gather_mode == 0 || g == 1) {
    return mllmb200_w4a32_linear_forward_ex(x_dev, tiled_shard_dev, y_blk, ws_dev, M, K, nl, ldx, N_total, kernel, stream);
  }
  if (gather_mode == 1) {  // NCCL baseline
    if (!h->comm) return MLLMB200_INVALID_ARG;
    const size_t need = (size_t)M * N_total * 4;
    if (need > h->stage_bytes) {
      cudaError_t e = cudaSuccess;
      if (h->send_stage) cudaFree(h->send_stage);
      if (h->recv_stage) cudaFree(h->recv_stage);
      h->send_stage = h->recv_stage = nullptr;
      if ((e = cudaMalloc(&h->send_stage, (size_t)M * nl * 4)) != cudaSuccess) return tp_fail(e);
      if ((e = cudaMalloc(&h->recv_stage, need)) != cudaSuccess) return tp_fail(e);
      h->stage_bytes = need;
    }
    int st = mllmb200_w4a32_linear_forward_ex(x_dev, tiled_shard_dev, h->send_stage, ws_dev, M, K, nl, ldx, nl, kernel, stream);
    if (st != MLLMB200_OK) return st;
    if (h->all_gather(h->send_stage, h->recv_stage, (size_t)M * nl, ncclFloat, h->comm, s) != ncclSuccess) return MLLMB200_CUDA_ERROR;
    const size_t total4 = (size_t)g * M * (nl / 4);
    const int blocks = (int)std::min<size_t>((total4 + 255) / 256, 148 * 8);
    tp_reassemble_kernel<<<blocks, 256, 0, s>>>(h->recv_stage, h->y_local, g, M, nl, N_total);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MLLMB200_OK : tp_fail(e);
  }

  // ---- gather_mode 2: the epilogue stores into every rank's y
  float* peers[kTpMaxRanks];
  int np = 0;
  for (int p = 0; p < g; ++p)
    if (p != r) peers[np++] = h->y_rank[p] + (size_t)r * nl;
  cudaError_t e = cudaSuccess;
  const void* tiled = tiled_shard_dev;
  int ldy = N_total;
  if (M <= 4 && (policy == 0 || policy == 1 || policy == 5) && w4a32_gemv_stream_supported(M, 1, &K, &nl)) {
    e = launch_w4a32_gemv_stream(1, &x_dev, &ldx, nullptr, nullptr, M, &K, &tiled, &y_blk, &nl, &ldy, use_pdl, s, np, peers);
  } else if ((policy == 4 || policy == 5) && w4a32_gemm_tcf16_preferred(M, K, nl)) {
    if (!ws_dev || (reinterpret_cast<uintptr_t>(ws_dev) & 255u)) return MLLMB200_INVALID_ARG;
    uint8_t* blocks = static_cast<uint8_t*>(ws_dev);
    float2* hdr = reinterpret_cast<float2*>(blocks + w4a32_ws_rec_bytes(M, K));
    // with the K-split counters, as the public forward: every gather mode computes a shard with the same launch
    int* sync = w4a32_ws_split_sync(ws_dev, M, K);
    const int sync_ints = w4a32_ws_split_sync_ints();
    e = launch_act_quant_blocks_f16(x_dev, M, w4a32_gemm_tcf16_m_pad(M, nl), K, ldx, blocks, hdr, s, 0, sync, sync_ints);
    if (e == cudaSuccess)
      e = launch_w4a32_gemm_tcf16_grouped(blocks, hdr, M, K, 1, &tiled, &y_blk, &nl, &ldy, s, np, peers, 0, sync, sync_ints);
  } else {
    // kernels without a peer epilogue: compute the block, then push it to every peer with strided device copies
    const int st = mllmb200_w4a32_linear_forward_ex(x_dev, tiled_shard_dev, y_blk, ws_dev, M, K, nl, ldx, N_total, kernel, stream);
    if (st != MLLMB200_OK) return st;
    for (int i = 0; i < np && e == cudaSuccess; ++i)
      e = cudaMemcpy2DAsync(peers[i], (size_t)N_total * 4, y_blk, (size_t)N_total * 4, (size_t)nl * 4, (size_t)M, cudaMemcpyDefault, s);
  }
  if (e != cudaSuccess) return tp_fail(e);
  // completion: tell every peer that this rank's block has landed, wait for theirs
  const unsigned epoch = ++h->epoch;
  TpFlagPtrs fp;
  for (int p = 0; p < kTpMaxRanks; ++p) fp.p[p] = p < g ? h->flags_rank[p] : nullptr;
  tp_signal_wait_kernel<<<1, 32, 0, s>>>(fp, h->flags_local, g, r, epoch, kTpWaitTicks);
  e = cudaGetLastError();
  return e == cudaSuccess ? MLLMB200_OK : tp_fail(e);
}

int mllmb200_w4a32_tp_output(void* handle, float** y_dev, size_t* bytes) {
  auto* h = static_cast<TpHandle*>(handle);
  if (!h) return MLLMB200_INVALID_ARG;
  if (y_dev) *y_dev = h->y_local;
  if (bytes) *bytes = h->y_bytes;
  return MLLMB200_OK;
}

void mllmb200_w4a32_tp_destroy(void* handle) {
  auto* h = static_cast<TpHandle*>(handle);
  if (!h) return;
  cudaDeviceSynchronize();
  for (int p = 0; p < h->nranks; ++p) {
    if (p == h->rank || !h->mapped) continue;
    if (h->y_rank[p]) cudaIpcCloseMemHandle(h->y_rank[p]);
    if (h->flags_rank[p]) cudaIpcCloseMemHandle(h->flags_rank[p]);
  }
  if (h->y_local) cudaFree(h->y_local);
  if (h->flags_local) cudaFree(h->flags_local);
  if (h->send_stage) cudaFree(h->send_stage);
  if (h->recv_stage) cudaFree(h->recv_stage);
  delete h;
}

}  // extern "C"
