// Device side of the W4A16 part of the C ABI (include/mllmb200.h): argument checks and launches.
#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/mllmb200.h"
#include "layout_a16.h"

namespace mllmb200 {
// w4a16.cu
size_t a16_workspace_bytes(int m, int k, int n);
cudaError_t launch_w4a16_linear(const void*, int, const void*, void*, void*, int, int, int, int, int, int, cudaStream_t);
cudaError_t launch_w4a16_linear_grouped(const void*, int, int, int, int, int, const void* const*, void* const*, const int*,
                                        const int*, void*, int, cudaStream_t);
cudaError_t launch_w4a16_repack(const void*, int, int, int, int, int, void*, cudaStream_t);
// c_api.cu
int record_cuda_failure(cudaError_t e);
}  // namespace mllmb200

using namespace mllmb200;

extern "C" {

int mllmb200_w4a16_tiled_size(int N_rows, int K, size_t* bytes) {
  if (!bytes || N_rows <= 0 || K <= 0) return MLLMB200_INVALID_ARG;
  *bytes = make_tiled_header_a16(N_rows, K, 0).total_bytes;
  return MLLMB200_OK;
}

int mllmb200_w4a16_repack_device(const void* blob_dev, int N, int K, int has_bias, int row_begin, int row_count,
                                 void* tiled_dev, void* stream) {
  if (!blob_dev || !tiled_dev || N <= 0 || K <= 0 || row_count <= 0 || row_begin < 0 || row_begin + row_count > N)
    return MLLMB200_INVALID_ARG;
  if (((uintptr_t)blob_dev & 15) || ((uintptr_t)tiled_dev & 15)) return MLLMB200_INVALID_ARG;
  const cudaError_t e = launch_w4a16_repack(blob_dev, N, K, has_bias ? 1 : 0, row_begin, row_count, tiled_dev,
                                            (cudaStream_t)stream);
  return e == cudaSuccess ? MLLMB200_OK : record_cuda_failure(e);
}

int mllmb200_w4a16_workspace_size(int M, int K, int N, size_t* bytes) {
  if (!bytes || M <= 0 || K <= 0 || N <= 0) return MLLMB200_INVALID_ARG;
  *bytes = a16_workspace_bytes(M, K, N);
  return MLLMB200_OK;
}

int mllmb200_w4a16_linear_forward(const void* x_dev, int x_dtype, const void* tiled_dev, void* y_dev, void* ws_dev,
                                  int M, int K, int N, int ldx, int ldy, void* stream) {
  return mllmb200_w4a16_linear_forward_ex(x_dev, x_dtype, tiled_dev, y_dev, ws_dev, M, K, N, ldx, ldy, 0, stream);
}

int mllmb200_w4a16_linear_forward_ex(const void* x_dev, int x_dtype, const void* tiled_dev, void* y_dev, void* ws_dev,
                                     int M, int K, int N, int ldx, int ldy, int kernel, void* stream) {
  const int family = kernel & 0xff;
  if ((kernel & ~0x1ff) || (family != 0 && family != 2 && family != 4)) return MLLMB200_INVALID_ARG;
  if (family == 4 && M < 8) return MLLMB200_UNSUPPORTED;
  if (!x_dev || !tiled_dev || !y_dev || !ws_dev || M <= 0 || K <= 0 || N <= 0 || ldx < K || ldy < N)
    return MLLMB200_INVALID_ARG;
  if (x_dtype != MLLMB200_DTYPE_F32 && x_dtype != MLLMB200_DTYPE_F16) return MLLMB200_INVALID_ARG;
  if (((uintptr_t)tiled_dev & 15) || ((uintptr_t)ws_dev & 255) || ((uintptr_t)y_dev & 1) ||
      ((uintptr_t)x_dev & (x_dtype == MLLMB200_DTYPE_F16 ? 1 : 3)))
    return MLLMB200_INVALID_ARG;
  if (M > 65535) return MLLMB200_UNSUPPORTED;  // rows of x ride on gridDim.y
  const cudaError_t e =
      launch_w4a16_linear(x_dev, x_dtype, tiled_dev, y_dev, ws_dev, M, K, N, ldx, ldy, kernel, (cudaStream_t)stream);
  return e == cudaSuccess ? MLLMB200_OK : record_cuda_failure(e);
}

int mllmb200_w4a16_linear_forward_grouped(const void* x_dev, int x_dtype, int M, int K, int ldx, int count,
                                          const void* const* tiled_dev, void* const* y_dev, const int* N, const int* ldy,
                                          void* ws_dev, int flags, void* stream) {
  if (!x_dev || !tiled_dev || !y_dev || !N || !ldy || !ws_dev || M <= 0 || K <= 0 || ldx < K || count < 1 || count > 4)
    return MLLMB200_INVALID_ARG;
  if (x_dtype != MLLMB200_DTYPE_F32 && x_dtype != MLLMB200_DTYPE_F16) return MLLMB200_INVALID_ARG;
  if ((flags & ~0x100) || ((uintptr_t)ws_dev & 255) || ((uintptr_t)x_dev & (x_dtype == MLLMB200_DTYPE_F16 ? 1 : 3)))
    return MLLMB200_INVALID_ARG;
  if (M > 65535) return MLLMB200_UNSUPPORTED;
  for (int i = 0; i < count; ++i) {
    if (!tiled_dev[i] || !y_dev[i] || N[i] <= 0 || ldy[i] < N[i]) return MLLMB200_INVALID_ARG;
    if (((uintptr_t)tiled_dev[i] & 15) || ((uintptr_t)y_dev[i] & 1)) return MLLMB200_INVALID_ARG;
  }
  const cudaError_t e = launch_w4a16_linear_grouped(x_dev, x_dtype, M, K, ldx, count, tiled_dev, y_dev, N, ldy, ws_dev,
                                                    flags, (cudaStream_t)stream);
  return e == cudaSuccess ? MLLMB200_OK : record_cuda_failure(e);
}

}  // extern "C"
