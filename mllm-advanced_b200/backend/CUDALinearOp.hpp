// The W4A32 quantized linear as an mllm op: drop-in for ArmLinearOp on the Kai W4A32 impl types
// (reference project: mllm/Backends/Arm/Ops/LinearOp.hpp:15-29, LinearOp.cpp:21-264), and on the
// W4A16 sibling types KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk (LinearOp.cpp:135-190: fp16 or fp32 input,
// fp16 output per LinearOp.cpp:246-251).  All device work goes through the C ABI in include/mllmb200.h.
#pragma once

#include <cstddef>
#include <memory>
#include <string>

#include "mllm/Core/AOps/LinearOp.hpp"

namespace mllm::cuda {

class CUDAW4A32LinearOp final : public LinearOp {
 public:
  explicit CUDAW4A32LinearOp(const LinearOpCargo& cargo);
  ~CUDAW4A32LinearOp();

  // Binds "<name>.weight" (the 1-D int8 pre-pack blob written by the quantization pass, or an
  // fp32 [N,K] tensor that is then quantized on the fly) and uploads + repacks it once.
  void load(const std::shared_ptr<ParameterLoader>& ploader) override;

  void reshape(const std::vector<Tensor>& inputs, std::vector<Tensor>& outputs) override;

  void forward(const std::vector<Tensor>& inputs, std::vector<Tensor>& outputs) override;

 private:
  void releaseDevice();
  void growWorkspace(size_t need);

  void* tiled_dev_ = nullptr;      // weights in the tile layout (from the backend's allocator)
  void* workspace_dev_ = nullptr;  // quantized activations, grown on demand, reused across calls
  size_t workspace_bytes_ = 0;
  int n_ = 0, k_ = 0;
  bool a16_ = false;  // the W4A16 sibling format
};

class CUDALinearOpFactory : public TypedOpFactory<OpType::kLinear, LinearOpCargo> {
 public:
  std::shared_ptr<BaseOp> createOpImpl(const LinearOpCargo& cargo) override {
    return std::make_shared<CUDAW4A32LinearOp>(cargo);
  }
};

// Pre-pack blob (int8 tensor) or fp32 weight of an [n, k] matrix -> device buffer in the tile layout
// (from the registered backend's allocator; the caller returns it with deviceFree).  Shared with the Conv3D op.
void* uploadW4A32Weights(Tensor& weight, Tensor& bias, bool want_bias, int n, int k, const std::string& name);

// True for the impl types this op implements (the six f32 W4 Kai tiles; the tile choice is an
// Arm micro-kernel detail and is ignored here).
bool isW4A32ImplType(LinearOpImplType t);

// The same for the W4A16 sibling format (blob layout 1), and its three impl types.
void* uploadW4A16Weights(Tensor& weight, Tensor& bias, bool want_bias, int n, int k, const std::string& name);
bool isW4A16ImplType(LinearOpImplType t);

}  // namespace mllm::cuda
