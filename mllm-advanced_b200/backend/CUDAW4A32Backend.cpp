#include "CUDAW4A32Backend.hpp"

#include <cuda_runtime.h>

#include "CUDAConv3DOp.hpp"
#include "CUDALinearOp.hpp"
#include "mllm/Core/DataTypes.hpp"
#include "mllm/Engine/Context.hpp"
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
// BackendBase has no virtual functions, so an instance handed back by the engine cannot be dynamic_cast; every
// W4A32 backend alive is listed here instead and a lookup checks the address against the list.
std::mutex g_instances_mu;
std::vector<const CUDAW4A32Backend*> g_instances;

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
  {
    std::lock_guard<std::mutex> lk(g_instances_mu);
    g_instances.push_back(this);
  }
  allocator_ = std::make_shared<CUDAW4A32Allocator>();
  regOpFactory<CUDALinearOpFactory>();
  regOpFactory<CUDAConv3DOpFactory>();
  regOpFactory<CUDAW4A32D2HOpFactory>();
}

CUDAW4A32Backend::~CUDAW4A32Backend() {
  {
    std::lock_guard<std::mutex> lk(g_instances_mu);
    for (auto it = g_instances.begin(); it != g_instances.end(); ++it)
      if (*it == this) {
        g_instances.erase(it);
        break;
      }
  }
  if (stream_) cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
}

void* CUDAW4A32Backend::deviceAlloc(size_t bytes) {
  void* ptr = nullptr;
  if (!allocator_->generalAlloc(&ptr, bytes, 256) || !ptr) { MLLM_ERROR_EXIT(kCudaError, "out of device memory ({} bytes)", bytes); }
  return ptr;
}

void CUDAW4A32Backend::deviceFree(void* ptr) {
  if (ptr) allocator_->generalFree(ptr);  // back into the cache; later users launch on the same stream
}

std::shared_ptr<CUDAW4A32Backend> createCUDAW4A32Backend() { return std::make_shared<CUDAW4A32Backend>(); }

CUDAW4A32Backend& registeredW4A32Backend() {
  auto base = MllmEngineCtx::instance().getBackend(kCUDA);
  auto* be = static_cast<CUDAW4A32Backend*>(base.get());
  bool ours = false;
  {
    std::lock_guard<std::mutex> lk(g_instances_mu);
    for (const auto* p : g_instances) ours = ours || p == be;
  }
  if (!ours) { MLLM_ERROR_EXIT(kError, "the backend registered for kCUDA is not the W4A32 backend"); }
  return *be;
}

void* currentW4A32Stream() { return registeredW4A32Backend().stream(); }

void CUDAW4A32D2HOp::forward(const std::vector<Tensor>& inputs, std::vector<Tensor>& outputs) {
  auto stream = static_cast<cudaStream_t>(currentW4A32Stream());
  const size_t bytes = inputs[0].numel() * dataTypeSize(inputs[0].dtype());
  MLLMB200_CHECK_CUDA(cudaMemcpyAsync(outputs[0].ptr<char>(), inputs[0].ptr<char>(), bytes, cudaMemcpyDeviceToHost, stream));
  MLLMB200_CHECK_CUDA(cudaStreamSynchronize(stream));
}

Tensor toDevice(const Tensor& host) {
  if (host.device() == kCUDA) return host;
  Tensor dev = Tensor::empty(host.shape(), host.dtype(), kCUDA).alloc();
  auto stream = static_cast<cudaStream_t>(currentW4A32Stream());
  const size_t bytes = host.numel() * dataTypeSize(host.dtype());
  MLLMB200_CHECK_CUDA(cudaMemcpyAsync(dev.ptr<char>(), const_cast<Tensor&>(host).ptr<char>(), bytes, cudaMemcpyHostToDevice, stream));
  MLLMB200_CHECK_CUDA(cudaStreamSynchronize(stream));  // the host buffer may be reused by the caller right away
  return dev;
}

}  // namespace mllm::cuda
