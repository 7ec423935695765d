#include "CudaQuantizationPass.hpp"

#include <string>

#include "mllm/Core/AOps/Conv3DOp.hpp"
#include "mllm/Core/AOps/LinearOp.hpp"
#include "mllm/IR/Builtin/Op.hpp"
#include "mllm/IR/Graph/Op.hpp"
#include "mllm/IR/Linalg/Op.hpp"
#include "mllm/Utils/Common.hpp"
#include "mllm/Utils/Log.hpp"
#include "mllmb200.h"

namespace mllm::cuda {

namespace {
constexpr const char* kFamily = "KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk";
// the W4A16 sibling (KQP_linear_f16_qsi8d32p_qai4c32p_mxk_nxk, KaiQuantizationPass.cpp:301-392 of the reference)
constexpr const char* kFamilyA16 = "KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk";

// "family:tile" -> family
std::string implFamily(const std::string& impl) {
  const auto pos = impl.find(':');
  return pos == std::string::npos ? impl : impl.substr(0, pos);
}
}  // namespace

bool CudaQuantizationPass::quantizeLinear(const ir::op_ptr_t& op) {
  auto* linear = (LinearOp*)(op->cast_<ir::linalg::LinearOp>()->getAOp());
  const std::string family = implFamily(cfg_.opImplType(linear->name()));
  const bool a16 = family == kFamilyA16;
  if (family != kFamily && !a16) return false;

  const Tensor weight = linear->weight();
  const Tensor bias = linear->bias();
  const int n = linear->cargo().out_channels, k = linear->cargo().in_channels;
  const bool has_bias = linear->cargo().bias;
  if (weight.dtype() != kFp32 || (has_bias && bias.dtype() != kFp32)) {
    MLLM_WARN("CudaQuantizationPass: {} needs an fp32 weight (and bias); left unquantized", linear->name());
    return false;
  }
  const auto shape = weight.shape();
  if (shape.size() != 2 || shape[0] != n || shape[1] != k) {
    MLLM_WARN("CudaQuantizationPass: {} weight must be [out_channels, in_channels]; left unquantized", linear->name());
    return false;
  }

  size_t bytes = 0;
  int st = a16 ? mllmb200_w4a16_prepack_size(n, k, has_bias ? 1 : 0, &bytes)
               : mllmb200_w4a32_prepack_size(n, k, has_bias ? 1 : 0, &bytes);
  if (st != MLLMB200_OK) {
    MLLM_WARN("CudaQuantizationPass: {}: {}", linear->name(), mllmb200_status_str(st));
    return false;
  }
  // a flat int8 buffer stands for the packed weight; it cannot be read as an ordinary tensor
  Tensor packed = Tensor::empty({(int32_t)bytes}, kInt8, kCPU).alloc();
  st = a16 ? mllmb200_w4a16_quant_prepack(weight.ptr<float>(), has_bias ? bias.ptr<float>() : nullptr, n, k,
                                          packed.ptr<uint8_t>())
           : mllmb200_w4a32_quant_prepack(weight.ptr<float>(), has_bias ? bias.ptr<float>() : nullptr, n, k,
                                          MLLMB200_SCALE_BF16_TRUNC, packed.ptr<uint8_t>());
  if (st != MLLMB200_OK) {
    MLLM_WARN("CudaQuantizationPass: {}: {}", linear->name(), mllmb200_status_str(st));
    return false;
  }
  packed.setName(weight.name());
  linear->weight() = packed;
  // the bias now lives inside the blob; a 1-byte tensor keeps its slot in the parameter file
  linear->bias() = Tensor::empty({1}, kInt8, kCPU).alloc();
  ++quantized_;
  return true;
}

bool CudaQuantizationPass::quantizeConv3D(const ir::op_ptr_t& op) {
  auto* conv = (Conv3DOp*)(op->cast_<ir::linalg::Conv3DOp>()->getAOp());
  if (implFamily(cfg_.opImplType(conv->name())) != kFamily) return false;
  const auto& cargo = conv->cargo();
  const Tensor weight = conv->weight();
  const Tensor bias = conv->bias();
  if (weight.dtype() != kFp32 || (cargo.bias && bias.dtype() != kFp32)) {
    MLLM_WARN("CudaQuantizationPass: {} needs an fp32 kernel (and bias); left unquantized", conv->name());
    return false;
  }
  if (cargo.kernel_size.size() != 3) return false;
  const int n = cargo.out_channels;
  const int k = cargo.in_channels * cargo.kernel_size[0] * cargo.kernel_size[1] * cargo.kernel_size[2];
  if ((size_t)weight.numel() != (size_t)n * (size_t)k) {
    MLLM_WARN("CudaQuantizationPass: {} kernel must be [out, in, kt, kh, kw]; left unquantized", conv->name());
    return false;
  }
  // The kernel is used as it lies: row o of the matrix is kernel[o] flattened in (c, kt, kh, kw) order, the column
  // order of the op's im2col (mllm/Backends/Arm/Kernels/conv3d.cpp:49-62 of the reference).  The reference's own
  // pattern first permutes the kernel to [out, kt, kh, kw, in] (KaiQuantizationPass.cpp:461-465), which does not
  // match that column order when in_channels > 1; the pairing kept here is the one that computes the convolution.
  size_t bytes = 0;
  int st = mllmb200_w4a32_prepack_size(n, k, cargo.bias ? 1 : 0, &bytes);
  if (st != MLLMB200_OK) return false;
  Tensor packed = Tensor::empty({(int32_t)bytes}, kInt8, kCPU).alloc();
  st = mllmb200_w4a32_quant_prepack(weight.ptr<float>(), cargo.bias ? bias.ptr<float>() : nullptr, n, k,
                                    MLLMB200_SCALE_BF16_TRUNC, packed.ptr<uint8_t>());
  if (st != MLLMB200_OK) {
    MLLM_WARN("CudaQuantizationPass: {}: {}", conv->name(), mllmb200_status_str(st));
    return false;
  }
  packed.setName(weight.name());
  conv->weight() = packed;
  conv->bias() = Tensor::empty({1}, kInt8, kCPU).alloc();
  ++quantized_;
  return true;
}

void CudaQuantizationPass::visitGraph(const ir::op_ptr_t& subgraph) {
  auto region = subgraph->cast_<ir::graph::SubGraphOp>()->getTopRegion();
  for (auto& node : region->ops()) {
    if (node->isa_<ir::graph::CallGraphOp>()) {
      auto callee = getCtx()->lookupSymbolTable(node->cast_<ir::graph::CallGraphOp>()->getSymbolAttr()->str());
      visitGraph(callee->cast_<ir::graph::SubGraphOp>());
    } else if (node->isa_<ir::linalg::LinearOp>()) {
      if (!quantizeLinear(node)) {
        MLLM_WARN("CudaQuantizationPass: linear {} not quantized (no matching impl type in the config)",
                  node->cast_<ir::linalg::LinalgIROp>()->getAOp()->name());
      }
    } else if (node->isa_<ir::linalg::Conv3DOp>()) {
      if (!quantizeConv3D(node)) {
        MLLM_WARN("CudaQuantizationPass: conv3d {} not quantized (no matching impl type in the config)",
                  node->cast_<ir::linalg::LinalgIROp>()->getAOp()->name());
      }
    }
  }
}

uint8_t CudaQuantizationPass::run(const ir::node_ptr_t& op) {
  MLLM_RT_ASSERT(op->isa_<ir::ModuleOp>());
  // entry point: the single CallGraphOp of the module
  ir::graph::CallGraphOp::self_ptr_t entry = nullptr;
  for (auto& node : op->cast_<ir::ModuleOp>()->getTopRegion()->ops()) {
    if (node->isa_<ir::graph::CallGraphOp>()) {
      MLLM_RT_ASSERT_EQ(entry, nullptr);
      entry = node->cast_<ir::graph::CallGraphOp>();
    }
  }
  if (entry == nullptr) return ir::PASS_RET_FAILURE;
  visitGraph(getCtx()->lookupSymbolTable(entry->getSymbolAttr()->str())->cast_<ir::graph::SubGraphOp>());
  return ir::PASS_RET_SUCCESS;
}

}  // namespace mllm::cuda
