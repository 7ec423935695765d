// B200 W4A32 backend for the mllm engine: a `BackendBase` for `kCUDA` that registers the
// quantized LinearOp of this library.  Written against the reference project's plugin API
// (mllm/Engine/BackendBase.hpp:20-46, mllm/Engine/Allocator.hpp:17-31); supersedes the stub
// in mllm/Backends/CUDA/CUDABackend.cpp:18-24 for this path.
#pragma once

#include <cstddef>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "mllm/Core/AOps/D2HOp.hpp"
#include "mllm/Core/Tensor.hpp"
#include "mllm/Engine/Allocator.hpp"
#include "mllm/Engine/BackendBase.hpp"

namespace mllm::cuda {

// Device allocator.  The engine's MemManager sends every request of 128 MB or more, and each new
// buddy-pool segment, straight here (mllm/Engine/MemManager.cpp:54-63,138-179).  The stub it
// replaces synchronized the whole device on every free; this one keeps freed blocks in a
// per-size cache and reuses them, so steady-state inference makes no cudaMalloc / cudaFree calls.
class CUDAW4A32Allocator final : public Allocator {
 public:
  ~CUDAW4A32Allocator();

  bool ctrlByMllmMemManager() override { return true; }
  bool alloc(const std::shared_ptr<Storage>& storage) override;
  void free(const std::shared_ptr<Storage>& storage) override;
  void free(Storage* storage) override;
  bool generalAlloc(void** ptr, size_t cap, size_t align) override;
  void generalFree(void* ptr) override;
  size_t allocSize(Storage* storage) override;
  size_t allocSize(const std::shared_ptr<Storage>& storage) override;
  [[nodiscard]] size_t alignSize() const override { return 256; }

 private:
  std::mutex mu_;
  std::map<void*, size_t> live_;                      // pointer -> rounded size
  std::multimap<size_t, void*> cache_;                // rounded size -> free block
};

class CUDAW4A32Backend final : public BackendBase {
 public:
  CUDAW4A32Backend();
  ~CUDAW4A32Backend();

  // The stream every op of this backend launches on (one per backend instance).
  [[nodiscard]] void* stream() const { return stream_; }

  // Device memory for the ops' own buffers (packed weights, activation workspaces): the backend's caching
  // allocator, so steady-state inference calls neither cudaMalloc nor cudaFree.
  void* deviceAlloc(size_t bytes);
  void deviceFree(void* ptr);

  // Kernel policy of CUDAW4A32LinearOp::forward for M >= 65 (the `kernel` argument of
  // mllmb200_w4a32_linear_forward_ex): 0 = the exact int8 tensor-core path (default: the reference's
  // arithmetic), 5 = the fastest path (fp16 tensor-core kernel for M >= 128, same 1e-3 * rms bound).
  void setLinearKernelPolicy(int policy) { linear_policy_ = policy; }
  [[nodiscard]] int linearKernelPolicy() const { return linear_policy_; }

 private:
  void* stream_ = nullptr;  // cudaStream_t
  int linear_policy_ = 0;
};

std::shared_ptr<CUDAW4A32Backend> createCUDAW4A32Backend();

// The backend registered with the engine for kCUDA (exits when none is, as every backend lookup of the engine does).
CUDAW4A32Backend& registeredW4A32Backend();

// Its stream.
void* currentW4A32Stream();

// Device -> host copy as an engine op (reference: mllm/Backends/CUDA/Ops/D2HOp.cpp:18-22; reached through
// Tensor::cpu(), mllm/Core/Tensor.cpp:120-126).  Copies on the backend's stream and waits for it: the host reads
// the result right after (mllm/Models/AutoLLM.hpp:70-85).
class CUDAW4A32D2HOp final : public D2HOp {
 public:
  explicit CUDAW4A32D2HOp(const D2HOpCargo& cargo) : D2HOp(cargo) {}
  void forward(const std::vector<Tensor>& inputs, std::vector<Tensor>& outputs) override;
};

class CUDAW4A32D2HOpFactory final : public TypedOpFactory<OpType::kD2H, D2HOpCargo> {
 public:
  std::shared_ptr<BaseOp> createOpImpl(const D2HOpCargo& cargo) override { return std::make_shared<CUDAW4A32D2HOp>(cargo); }
};

// Host -> device: a new kCUDA tensor of the same shape and dtype, allocated by the engine's memory manager and
// filled on the backend's stream.  The reference has an OpType for this direction but no op
// (mllm/Core/Tensor.cpp:128-132 "TODO Host 2 Device"), and the engine picks an op's backend from its INPUT's
// device, i.e. the host's - so this is a function of the CUDA backend, not an op of it.
Tensor toDevice(const Tensor& host);

}  // namespace mllm::cuda
