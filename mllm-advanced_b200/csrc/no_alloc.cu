// mllmb200_w4a32_linear_forward_static: the forward for callers that must not allocate.
//
// Who that is: code that runs where device allocation is off limits - a serving loop whose
// memory budget was fixed at start-up, a host framework that owns every byte of device memory
// through its own pool (as the mllm engine does with its MemManager) and forbids plug-ins to go
// to the CUDA allocator behind its back, or a latency-critical step where cudaMalloc's implicit
// device synchronization is unacceptable.  Such a caller can hand over inputs and outputs it
// already owns, but has nowhere to get the workspace that mllmb200_w4a32_linear_forward needs for
// the quantized activations.
//
// This entry point keeps that workspace in a fixed array in the library's own device image, so the
// call allocates nothing: no cudaMalloc, no cudaFree, no allocating library routine.  The price
// is a fixed capacity and a shared buffer:
//  - every GPU that loads the library holds kStaticScratchBytes (1 MiB) until the process exits;
//  - a call whose workspace (mllmb200_w4a32_workspace_size(M, K)) exceeds that is refused with
//    MLLMB200_TOO_LARGE - batched-decode sizes fit (up to M = 256 at K = 1536, M = 63 at K = 8960),
//    a 512-token prefill does not.  Calls with M <= 4 take the single-launch GEMV, which quantizes
//    the activations in shared memory and does not touch the array at all;
//  - all calls on a device share the one array and it keeps whatever the last call left.  Nothing
//    in it has to start at zero (the quantization kernel overwrites every byte the matrix kernel
//    reads), but two calls that overlap on the GPU (different streams) race on it: serialize them.
//
// The array's name is only a host-side handle; kernels need its device address.  The first call on
// each device looks it up with cudaGetSymbolAddress while that device is current and caches it.
// Make that first call before any stream capture begins.
#include <cuda_runtime.h>

#include "../../include/mllmb200.h"

namespace mllmb200 {
int record_cuda_failure(cudaError_t e);  // c_api.cu: remembers the code for mllmb200_last_cuda_error()
}

namespace {

constexpr size_t kStaticScratchBytes = 1u << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device ordinal; filled on first use.  Not locked: two host
// threads that make the first call on a device at the same time both look the address up and both
// store the same value, and an aligned pointer store is not torn - a benign race.
void* g_scratch_addr[kMaxDevices] = {};

// Returns the device address of the scratch array on the current device (nullptr on failure).
void* scratch_address(int* cuda_error) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *cuda_error = (int)(e != cudaSuccess ? e : cudaErrorInvalidDevice);
    return nullptr;
  }
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);  // with `dev` current: each device has its own copy
    if (e != cudaSuccess || ptr == nullptr) {
      *cuda_error = (int)e;
      return nullptr;
    }
    g_scratch_addr[dev] = ptr;
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" {

int mllmb200_w4a32_static_scratch_bytes(size_t* bytes) {
  if (!bytes) return MLLMB200_INVALID_ARG;
  *bytes = kStaticScratchBytes;
  return MLLMB200_OK;
}

int mllmb200_w4a32_linear_forward_static(const float* x_dev, const void* tiled_dev, float* y_dev, int M, int K, int N,
                                         int ldx, int ldy, void* stream) {
  size_t need = 0;
  const int st = mllmb200_w4a32_workspace_size(M, K, &need);
  if (st != MLLMB200_OK) return st;
  if (need > kStaticScratchBytes) return MLLMB200_TOO_LARGE;
  int cuda_error = 0;
  void* scratch = scratch_address(&cuda_error);
  if (scratch == nullptr) return mllmb200::record_cuda_failure((cudaError_t)cuda_error);
  // same kernels as the ordinary forward; only the workspace comes from the static array
  return mllmb200_w4a32_linear_forward(x_dev, tiled_dev, y_dev, scratch, M, K, N, ldx, ldy, stream);
}

}  // extern "C"
