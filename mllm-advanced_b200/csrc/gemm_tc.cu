// tcgen05 (5th-generation tensor core) W4A32 GEMM for large M.  Placeholder until the kernel lands:
// reports "not supported" so that the dispatcher uses the SIMT path.
#include "device_common.cuh"

namespace mllmb200 {
bool w4a32_gemm_tc_supported(int, int, int) { return false; }
cudaError_t launch_w4a32_gemm_tc(const uint8_t*, const float2*, const void*, float*, int, int, int, int, cudaStream_t) {
  return cudaErrorNotSupported;
}
}  // namespace mllmb200
