#include "CUDAW4A32Backend.hpp"

#include <cuda_runtime.h>

#include "CUDAConv3DOp.hpp"
#include "CUDALinearOp.hpp"
#include "mllm/Utils/Common.hpp"
#include "mllm/Utils/Log.hpp"

#define MLLMB200_CHECK_CUDA(expr)                                                                         \
  do {                                                                                                    \
    cudaError_t err__ = (expr);                                                                           \
    if (err__ != cudaSuccess) {                                                                           \
      MLLM_ERROR_EXIT(kCudaError, "CUDA error code {}: {}", int(err__), cudaGetErrorString(err__));       \
    }                                                                                                     \
  } while (0)

namespace mllm::cuda {

namespace {
void* g_stream = nullptr;
size_t round_block(size_t cap, size_t align) {
  // power-of-two-ish size classes above 1 MiB keep the cache hit rate high for growing shapes
  size_t v = (cap + align - 1) & ~(align - 1);
  if (v > (1u << 20)) v = (v + (1u << 20) - 1) & ~size_t((1u << 20) - 1);
  return v;
}
}  // namespace

CUDAW4A32Allocator::~CUDAW4A32Allocator() {
  for (auto& kv : cache_) cudaFree(kv.second);
}

bool CUDAW4A32Allocator::generalAlloc(void** ptr, size_t cap, size_t align) {
  const size_t want = round_block(cap, align < 256 ? 256 : align);
  {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = cache_.find(want);
    if (it != cache_.end()) {
      *ptr = it->second;
      cache_.erase(it);
      live_[*ptr] = want;
      return true;
    }
  }
  MLLMB200_CHECK_CUDA(cudaMalloc(ptr, want));
  std::lock_guard<std::mutex> lk(mu_);
  live_[*ptr] = want;
  return true;
}

void CUDAW4A32Allocator::generalFree(void* ptr) {
  if (!ptr) return;
  std::lock_guard<std::mutex> lk(mu_);
  auto it = live_.find(ptr);
  if (it == live_.end()) return;
  // Work that still uses the block was enqueued on the backend's single stream before this call;
  // the next user of the cached block launches on the same stream, so stream order protects it.
  cache_.insert({it->second, ptr});
  live_.erase(it);
}

bool CUDAW4A32Allocator::alloc(const std::shared_ptr<Storage>& storage) {
  void* ptr = nullptr;
  if (!generalAlloc(&ptr, storage->size_, alignSize()) || !ptr) return false;
  storage->ptr_ = ptr;
  return true;
}

void CUDAW4A32Allocator::free(const std::shared_ptr<Storage>& storage) { generalFree(storage->ptr_); }
void CUDAW4A32Allocator::free(Storage* storage) { generalFree(storage->ptr_); }

size_t CUDAW4A32Allocator::allocSize(Storage* storage) {
  const size_t a = alignSize();
  return (storage->size_ + a - 1) & ~(a - 1);
}
size_t CUDAW4A32Allocator::allocSize(const std::shared_ptr<Storage>& storage) { return allocSize(storage.get()); }

CUDAW4A32Backend::CUDAW4A32Backend() : BackendBase(kCUDA) {
  int count = 0;
  MLLMB200_CHECK_CUDA(cudaGetDeviceCount(&count));
  if (count <= 0) { MLLM_ERROR_EXIT(kCudaError, "no CUDA device: the W4A32 backend has no CPU fallback"); }
  cudaStream_t s;
  MLLMB200_CHECK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  stream_ = s;
  g_stream = s;
  allocator_ = std::make_shared<CUDAW4A32Allocator>();
  regOpFactory<CUDALinearOpFactory>();
  regOpFactory<CUDAConv3DOpFactory>();
}

CUDAW4A32Backend::~CUDAW4A32Backend() {
  if (g_stream == stream_) g_stream = nullptr;
  if (stream_) cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
}

std::shared_ptr<CUDAW4A32Backend> createCUDAW4A32Backend() { return std::make_shared<CUDAW4A32Backend>(); }

void* currentW4A32Stream() { return g_stream; }

}  // namespace mllm::cuda
