// Offline quantization pass for the B200 W4A32 linear: the counterpart of the reference's
// KaiQuantizationPass (mllm/Backends/Arm/Passes/KaiQuantizationPass.{hpp,cpp}) for Linear ops - and
// Conv3D ops run as a linear (KaiQuantizationPass.cpp:402-495) - whose configured impl type is a
// KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk tile.  It replaces the op's
// fp32 [N,K] weight by the 1-D int8 pre-pack blob of include/mllmb200.h (same tensor name) and the
// bias by a 1-byte int8 placeholder, exactly the convention the reference writes into .mllm files.
#pragma once

#include <memory>

#include "mllm/Engine/CfgFile.hpp"
#include "mllm/IR/Passes/Pass.hpp"

namespace mllm::cuda {

class CudaQuantizationPass final : public ir::Pass {
 public:
  explicit CudaQuantizationPass(const MllmModelCfg& cfg) : cfg_(cfg) {}
  ~CudaQuantizationPass() override = default;

  uint8_t run(const ir::node_ptr_t& op) override;

  // Quantizes one linalg LinearOp if the config asks for it; false when it was left untouched.
  bool quantizeLinear(const ir::op_ptr_t& op);

  // The same for a linalg Conv3DOp: the fp32 kernel [O, C, kt, kh, kw] is the [O, C*kt*kh*kw] matrix of the
  // implied linear, its rows in the (c, kt, kh, kw) order the im2col of the op produces.
  bool quantizeConv3D(const ir::op_ptr_t& op);

  [[nodiscard]] int quantizedCount() const { return quantized_; }

 private:
  void visitGraph(const ir::op_ptr_t& subgraph);

  const MllmModelCfg& cfg_;
  int quantized_ = 0;
};

inline std::shared_ptr<CudaQuantizationPass> createCudaQuantizationPass(const MllmModelCfg& cfg) {
  return std::make_shared<CudaQuantizationPass>(cfg);
}

}  // namespace mllm::cuda
