// Test-only kCPU backend for the boundary test.  Every nn::Layer of the reference is born on kCPU and
// nn::Module::reg immediately asks the kCPU backend for an op (mllm/Nn/Module.hpp:75-86,
// mllm/Nn/HierarchyBase.hpp:56), and the reference's own X86 backend registers no Linear factory
// (mllm/Backends/X86/X86Backend.cpp:16-19).  This shim supplies a host allocator and a placeholder
// Linear factory (the abstract mllm::LinearOp, which only binds parameters), so that a module can be
// constructed on the host and then moved with model.to(kCUDA); likewise a placeholder Conv3D factory, and a
// host cast op for the quantizer flow.
#pragma once

#include <cstdlib>
#include <memory>

#include "half/half.hpp"
#include "mllm/Core/AOps/CastTypeOp.hpp"
#include "mllm/Core/AOps/Conv3DOp.hpp"
#include "mllm/Core/AOps/LinearOp.hpp"
#include "mllm/Engine/Allocator.hpp"
#include "mllm/Engine/BackendBase.hpp"

namespace shim {

class HostAllocator final : public mllm::Allocator {
 public:
  bool ctrlByMllmMemManager() override { return true; }
  bool alloc(const std::shared_ptr<mllm::Storage>& s) override { return generalAlloc(&s->ptr_, s->size_, alignSize()); }
  void free(const std::shared_ptr<mllm::Storage>& s) override { generalFree(s->ptr_); }
  void free(mllm::Storage* s) override { generalFree(s->ptr_); }
  bool generalAlloc(void** ptr, size_t cap, size_t align) override {
    const size_t a = align < 64 ? 64 : align;
    *ptr = std::aligned_alloc(a, (cap + a - 1) / a * a);
    return *ptr != nullptr;
  }
  void generalFree(void* ptr) override { std::free(ptr); }
  size_t allocSize(mllm::Storage* s) override { return (s->size_ + 63) / 64 * 64; }
  size_t allocSize(const std::shared_ptr<mllm::Storage>& s) override { return allocSize(s.get()); }
  [[nodiscard]] size_t alignSize() const override { return 64; }
};

class PlaceholderLinearFactory : public mllm::TypedOpFactory<mllm::OpType::kLinear, mllm::LinearOpCargo> {
 public:
  std::shared_ptr<mllm::BaseOp> createOpImpl(const mllm::LinearOpCargo& cargo) override {
    return std::make_shared<mllm::LinearOp>(cargo);
  }
};

class PlaceholderConv3DFactory : public mllm::TypedOpFactory<mllm::OpType::kConv3D, mllm::Conv3DOpCargo> {
 public:
  std::shared_ptr<mllm::BaseOp> createOpImpl(const mllm::Conv3DOpCargo& cargo) override {
    return std::make_shared<mllm::Conv3DOp>(cargo);
  }
};

// fp32 -> fp16 cast on the host, so that the reference's CommonParamQuantizePass (Tensor::to(dtype),
// mllm/IR/Passes/QuantizePass.cpp:31-50) can run in the quantizer-flow test.
class HostCastOp final : public mllm::CastTypeOp {
 public:
  explicit HostCastOp(const mllm::CastTypeOpCargo& cargo) : CastTypeOp(cargo) {}
  void forward(const std::vector<mllm::Tensor>& inputs, std::vector<mllm::Tensor>& outputs) override {
    auto& in = const_cast<mllm::Tensor&>(inputs[0]);
    auto& out = outputs[0];
    const size_t n = in.numel();
    if (in.dtype() == mllm::kFp32 && out.dtype() == mllm::kFp16) {
      auto* dst = out.ptr<half_float::half>();
      const float* src = in.ptr<float>();
      for (size_t i = 0; i < n; ++i) dst[i] = half_float::half(src[i]);
    } else if (in.dtype() == mllm::kFp16 && out.dtype() == mllm::kFp32) {
      auto* src = in.ptr<half_float::half>();
      float* dst = out.ptr<float>();
      for (size_t i = 0; i < n; ++i) dst[i] = (float)src[i];
    }
  }
};

class HostCastFactory : public mllm::TypedOpFactory<mllm::OpType::kCastType, mllm::CastTypeOpCargo> {
 public:
  std::shared_ptr<mllm::BaseOp> createOpImpl(const mllm::CastTypeOpCargo& cargo) override {
    return std::make_shared<HostCastOp>(cargo);
  }
};

class HostShimBackend final : public mllm::BackendBase {
 public:
  HostShimBackend() : BackendBase(mllm::kCPU) {
    allocator_ = std::make_shared<HostAllocator>();
    regOpFactory<PlaceholderLinearFactory>();
    regOpFactory<PlaceholderConv3DFactory>();
    regOpFactory<HostCastFactory>();
  }
};

}  // namespace shim
