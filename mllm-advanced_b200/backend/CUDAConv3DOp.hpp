// Conv3D on the W4A32 linear (the Qwen2VL patch embedding): drop-in for ArmConv3DOp on the Kai
// W4A32 impl types (reference project: mllm/Backends/Arm/Ops/Conv3DOp.cpp:23-170).
// im2col, the quantized linear and the output permutation all run on the device through
// mllmb200_conv3d_w4a32_forward (include/mllmb200.h).
#pragma once

#include <cstddef>
#include <memory>

#include "mllm/Core/AOps/Conv3DOp.hpp"

namespace mllm::cuda {

class CUDAW4A32Conv3DOp final : public Conv3DOp {
 public:
  explicit CUDAW4A32Conv3DOp(const Conv3DOpCargo& cargo);
  ~CUDAW4A32Conv3DOp();

  // "<name>.weight": the int8 pre-pack blob of the [O, C*kt*kh*kw] matrix, or the fp32 kernel
  // [O, C, kt, kh, kw] (quantized here); "<name>.bias" when cargo.bias.
  void load(const std::shared_ptr<ParameterLoader>& ploader) override;

  // reshape is the base class's (mllm/Core/AOps/Conv3DOp.cpp:37-79): [B, O, T', H', W']
  void forward(const std::vector<Tensor>& inputs, std::vector<Tensor>& outputs) override;

 private:
  void releaseDevice();

  void* tiled_dev_ = nullptr;
  void* workspace_dev_ = nullptr;
  size_t workspace_bytes_ = 0;
  int n_ = 0, k_ = 0;
};

class CUDAConv3DOpFactory : public TypedOpFactory<OpType::kConv3D, Conv3DOpCargo> {
 public:
  std::shared_ptr<BaseOp> createOpImpl(const Conv3DOpCargo& cargo) override {
    return std::make_shared<CUDAW4A32Conv3DOp>(cargo);
  }
};

bool isW4A32Conv3DImplType(Conv3DOpImplType t);

}  // namespace mllm::cuda
