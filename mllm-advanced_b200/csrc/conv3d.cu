// Conv3D as a W4A32 linear (Qwen2VL patch embedding): im2col of the activation, the quantized
// linear on [positions, C*kt*kh*kw], and the permutation of the result to [B, O, T', H', W'] -
// the flow of the reference project's mllm/Backends/Arm/Ops/Conv3DOp.cpp:31-170 (no padding,
// dilation 1; im2col column order c, kt, kh, kw as in mllm/Backends/Arm/Kernels/conv3d.cpp:15-79).
// For the patch embedding K = 3*2*14*14 = 1176 is not a multiple of the 32-wide scale group: the
// linear's ragged last group is exercised here.
#include <cuda_runtime.h>

#include <algorithm>

#include "../../include/mllmb200.h"
#include "device_common.cuh"

namespace mllmb200 {

struct Conv3dDims {
  int batch, in_ch, t, h, w, kt, kh, kw, st, sh, sw, ot, oh, ow, out_ch;
};

// One thread per im2col element: z[(b, ot, oh, ow)][(c, kt, kh, kw)] = x[b][c][ot*st + kt][oh*sh + kh][ow*sw + kw]
__global__ void conv3d_im2col_kernel(const float* __restrict__ x, Conv3dDims d, float* __restrict__ z) {
  const long long kvol = (long long)d.kt * d.kh * d.kw, cols = d.in_ch * kvol;
  const long long total = (long long)d.batch * d.ot * d.oh * d.ow * cols;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / cols;
    int col = (int)(idx - row * cols);
    const int c = col / (int)kvol;
    col -= c * (int)kvol;
    const int kt = col / (d.kh * d.kw);
    col -= kt * d.kh * d.kw;
    const int kh = col / d.kw, kw = col - kh * d.kw;
    long long r = row;
    const int ow = (int)(r % d.ow);
    r /= d.ow;
    const int oh = (int)(r % d.oh);
    r /= d.oh;
    const int ot = (int)(r % d.ot);
    const int b = (int)(r / d.ot);
    z[idx] = x[((((size_t)b * d.in_ch + c) * d.t + ot * d.st + kt) * d.h + oh * d.sh + kh) * d.w + ow * d.sw + kw];
  }
}

// y[b][o][pos] = t[(b, pos)][o]   (pos = ot, oh, ow flattened): the reference's permute {0, 4, 1, 2, 3}
__global__ void conv3d_permute_out_kernel(const float* __restrict__ t, int batch, int positions, int out_ch,
                                          float* __restrict__ y) {
  const long long total = (long long)batch * positions * out_ch;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int pos = (int)(idx % positions);
    const long long r = idx / positions;
    const int o = (int)(r % out_ch);
    const int b = (int)(r / out_ch);
    y[idx] = t[((size_t)b * positions + pos) * out_ch + o];
  }
}

static bool conv3d_dims(const int* in_shape, const int* kernel, const int* stride, int out_ch, Conv3dDims* d) {
  d->batch = in_shape[0], d->in_ch = in_shape[1], d->t = in_shape[2], d->h = in_shape[3], d->w = in_shape[4];
  d->kt = kernel[0], d->kh = kernel[1], d->kw = kernel[2];
  d->st = stride[0], d->sh = stride[1], d->sw = stride[2];
  d->out_ch = out_ch;
  if (d->batch < 1 || d->in_ch < 1 || d->kt < 1 || d->kh < 1 || d->kw < 1 || d->st < 1 || d->sh < 1 || d->sw < 1 ||
      d->t < d->kt || d->h < d->kh || d->w < d->kw || out_ch < 1)
    return false;
  d->ot = (d->t - d->kt) / d->st + 1, d->oh = (d->h - d->kh) / d->sh + 1, d->ow = (d->w - d->kw) / d->sw + 1;
  const long long m = (long long)d->batch * d->ot * d->oh * d->ow, k = (long long)d->in_ch * d->kt * d->kh * d->kw;
  return m <= 0x7fffffff && k <= 0x7fffffff;
}

}  // namespace mllmb200

using namespace mllmb200;

extern "C" {

// in_shape = {B, C, T, H, W}, kernel = {kt, kh, kw}, stride = {st, sh, sw}.
// Outputs: M = B*T'*H'*W' rows and K = C*kt*kh*kw columns of the implied linear; workspace bytes
// (im2col matrix + row-major result + the linear's own workspace, each 256-aligned).
int mllmb200_conv3d_w4a32_plan(const int* in_shape, const int* kernel, const int* stride, int out_ch, int* M, int* K,
                               size_t* workspace_bytes) {
  if (!in_shape || !kernel || !stride) return MLLMB200_INVALID_ARG;
  Conv3dDims d;
  if (!conv3d_dims(in_shape, kernel, stride, out_ch, &d)) return MLLMB200_INVALID_ARG;
  const int m = d.batch * d.ot * d.oh * d.ow, k = d.in_ch * d.kt * d.kh * d.kw;
  if (M) *M = m;
  if (K) *K = k;
  if (workspace_bytes) {
    size_t lin = 0;
    const int st = mllmb200_w4a32_workspace_size(m, k, &lin);
    if (st != MLLMB200_OK) return st;
    *workspace_bytes = align_up((size_t)m * k * 4, 256) + align_up((size_t)m * out_ch * 4, 256) + lin;
  }
  return MLLMB200_OK;
}

// x_dev fp32 [B, C, T, H, W] contiguous; tiled_dev: the [out_ch, C*kt*kh*kw] weight (+ bias) in the
// tile layout; y_dev fp32 [B, out_ch, T', H', W'] contiguous; ws_dev from mllmb200_conv3d_w4a32_plan.
int mllmb200_conv3d_w4a32_forward(const float* x_dev, const void* tiled_dev, float* y_dev, void* ws_dev,
                                  const int* in_shape, const int* kernel, const int* stride, int out_ch, void* stream) {
  if (!x_dev || !tiled_dev || !y_dev || !ws_dev || !in_shape || !kernel || !stride) return MLLMB200_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(ws_dev) & 255u) return MLLMB200_INVALID_ARG;
  Conv3dDims d;
  if (!conv3d_dims(in_shape, kernel, stride, out_ch, &d)) return MLLMB200_INVALID_ARG;
  const int m = d.batch * d.ot * d.oh * d.ow, k = d.in_ch * d.kt * d.kh * d.kw;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(ws_dev);
  float* z = reinterpret_cast<float*>(ws);
  float* t = reinterpret_cast<float*>(ws + align_up((size_t)m * k * 4, 256));
  void* lin_ws = ws + align_up((size_t)m * k * 4, 256) + align_up((size_t)m * out_ch * 4, 256);
  const long long total = (long long)m * k;
  conv3d_im2col_kernel<<<(unsigned)std::min<long long>((total + 255) / 256, 148 * 32), 256, 0, st>>>(x_dev, d, z);
  if (cudaGetLastError() != cudaSuccess) return MLLMB200_CUDA_ERROR;
  const int rc = mllmb200_w4a32_linear_forward(z, tiled_dev, t, lin_ws, m, k, out_ch, k, out_ch, stream);
  if (rc != MLLMB200_OK) return rc;
  const long long total_o = (long long)m * out_ch;
  conv3d_permute_out_kernel<<<(unsigned)std::min<long long>((total_o + 255) / 256, 148 * 32), 256, 0, st>>>(
      t, d.batch, d.ot * d.oh * d.ow, out_ch, y_dev);
  return cudaGetLastError() == cudaSuccess ? MLLMB200_OK : MLLMB200_CUDA_ERROR;
}

}  // extern "C"
