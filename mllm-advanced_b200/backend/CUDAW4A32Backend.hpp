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

  // The stream every op of this backend launches on.
  [[nodiscard]] void* stream() const { return stream_; }

 private:
  void* stream_ = nullptr;  // cudaStream_t
};

std::shared_ptr<CUDAW4A32Backend> createCUDAW4A32Backend();

// Stream of the registered backend (nullptr = default stream when none is registered yet).
void* currentW4A32Stream();

}  // namespace mllm::cuda
