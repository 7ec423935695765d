#include "CUDAConv3DOp.hpp"

#include <cuda_runtime.h>

#include "CUDALinearOp.hpp"
#include "CUDAW4A32Backend.hpp"
#include "mllm/Utils/Common.hpp"
#include "mllm/Utils/Log.hpp"
#include "mllmb200.h"

namespace mllm::cuda {

bool isW4A32Conv3DImplType(Conv3DOpImplType t) {
  switch (t) {
    case Conv3DOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp1x8_qsi4c32p4x8_1x4x32:
    case Conv3DOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp1x8_qsi4c32p8x8_1x8x32:
    case Conv3DOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp4x8_qsi4c32p4x8_8x4x32:
    case Conv3DOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp4x8_qsi4c32p4x8_16x4x32:
    case Conv3DOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp4x8_qsi4c32p8x8_4x8x32:
    case Conv3DOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp1x4_qsi4c32p4x4_1x4: return true;
    default: return false;
  }
}

CUDAW4A32Conv3DOp::CUDAW4A32Conv3DOp(const Conv3DOpCargo& cargo) : Conv3DOp(cargo) {}

CUDAW4A32Conv3DOp::~CUDAW4A32Conv3DOp() { releaseDevice(); }

void CUDAW4A32Conv3DOp::releaseDevice() {
  if (tiled_dev_ || workspace_dev_) {
    auto& be = registeredW4A32Backend();
    be.deviceFree(tiled_dev_);
    be.deviceFree(workspace_dev_);
  }
  tiled_dev_ = workspace_dev_ = nullptr;
  workspace_bytes_ = 0;
}

void CUDAW4A32Conv3DOp::load(const std::shared_ptr<ParameterLoader>& ploader) {
  Conv3DOp::load(ploader);  // weight_ / bias_ by name (mllm/Core/AOps/Conv3DOp.cpp:19-22)
  if (!isW4A32Conv3DImplType(cargo_.impl_type)) {
    MLLM_ERROR_EXIT(kError, "CUDAW4A32Conv3DOp {}: impl type {} is not a W4A32 type", name(), int(cargo_.impl_type));
  }
  MLLM_RT_ASSERT_EQ(cargo_.kernel_size.size(), 3);
  MLLM_RT_ASSERT_EQ(cargo_.stride.size(), 3);
  releaseDevice();
  n_ = cargo_.out_channels;
  k_ = cargo_.in_channels * cargo_.kernel_size[0] * cargo_.kernel_size[1] * cargo_.kernel_size[2];
  tiled_dev_ = uploadW4A32Weights(weight_, bias_, cargo_.bias, n_, k_, "CUDAW4A32Conv3DOp " + name());
}

void CUDAW4A32Conv3DOp::forward(const std::vector<Tensor>& inputs, std::vector<Tensor>& outputs) {
  const auto& x = inputs[0];
  auto& y = outputs[0];
  if (!tiled_dev_) { MLLM_ERROR_EXIT(kError, "CUDAW4A32Conv3DOp {}: forward before load", name()); }
  if (x.dtype() != kFp32 || x.device() != kCUDA || x.shape().size() != 5) {
    MLLM_ERROR_EXIT(kError, "CUDAW4A32Conv3DOp {}: input must be a 5-D fp32 tensor on the CUDA device", name());
  }
  const int in_shape[5] = {x.shape()[0], x.shape()[1], x.shape()[2], x.shape()[3], x.shape()[4]};
  const int kernel[3] = {cargo_.kernel_size[0], cargo_.kernel_size[1], cargo_.kernel_size[2]};
  const int stride[3] = {cargo_.stride[0], cargo_.stride[1], cargo_.stride[2]};
  size_t need = 0;
  int st = mllmb200_conv3d_w4a32_plan(in_shape, kernel, stride, n_, nullptr, nullptr, &need);
  if (st != MLLMB200_OK) { MLLM_ERROR_EXIT(kError, "CUDAW4A32Conv3DOp {}: {}", name(), mllmb200_status_str(st)); }
  if (need > workspace_bytes_) {
    auto& be = registeredW4A32Backend();
    be.deviceFree(workspace_dev_);  // stream order protects work that still reads it
    workspace_dev_ = be.deviceAlloc(need);
    workspace_bytes_ = need;
  }
  st = mllmb200_conv3d_w4a32_forward(x.ptr<float>(), tiled_dev_, y.ptr<float>(), workspace_dev_, in_shape, kernel, stride, n_,
                                     currentW4A32Stream());
  if (st != MLLMB200_OK) {
    MLLM_ERROR_EXIT(kCudaError, "CUDAW4A32Conv3DOp {}: {} (cuda error {})", name(), mllmb200_status_str(st),
                    mllmb200_last_cuda_error());
  }
}

}  // namespace mllm::cuda
