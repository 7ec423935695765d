#include "CUDALinearOp.hpp"

#include <cuda_runtime.h>

#include <vector>

#include "CUDAW4A32Backend.hpp"
#include "mllm/Utils/Common.hpp"
#include "mllm/Utils/Log.hpp"
#include "mllmb200.h"

#define MLLMB200_CHECK_CUDA(expr)                                                                         \
  do {                                                                                                    \
    cudaError_t err__ = (expr);                                                                           \
    if (err__ != cudaSuccess) {                                                                           \
      MLLM_ERROR_EXIT(kCudaError, "CUDA error code {}: {}", int(err__), cudaGetErrorString(err__));       \
    }                                                                                                     \
  } while (0)

#define MLLMB200_CHECK(expr)                                                                              \
  do {                                                                                                    \
    int st__ = (expr);                                                                                    \
    if (st__ != MLLMB200_OK) {                                                                            \
      MLLM_ERROR_EXIT(kCudaError, "mllmb200: {} (status {}, cuda error {})", mllmb200_status_str(st__),   \
                      st__, mllmb200_last_cuda_error());                                                  \
    }                                                                                                     \
  } while (0)

namespace mllm::cuda {

bool isW4A32ImplType(LinearOpImplType t) {
  switch (t) {
    case LinearOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp1x8_qsi4c32p4x8_1x4x32:
    case LinearOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp1x8_qsi4c32p8x8_1x8x32:
    case LinearOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp4x8_qsi4c32p4x8_8x4x32:
    case LinearOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp4x8_qsi4c32p4x8_16x4x32:
    case LinearOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp4x8_qsi4c32p8x8_4x8x32:
    case LinearOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp1x4_qsi4c32p4x4_1x4: return true;
    default: return false;
  }
}

bool isW4A16ImplType(LinearOpImplType t) {
  switch (t) {
    case LinearOpImplType::KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk_qsi8d32p1x8_qai4c32p4x8_1x4:
    case LinearOpImplType::KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk_qsi8d32p4x4_qai4c32p4x4_8x4:
    case LinearOpImplType::KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk_qsi8d32p4x8_qai4c32p4x8_8x4_i8mm: return true;
    default: return false;
  }
}

CUDAW4A32LinearOp::CUDAW4A32LinearOp(const LinearOpCargo& cargo) : LinearOp(cargo) {}

CUDAW4A32LinearOp::~CUDAW4A32LinearOp() { releaseDevice(); }

void CUDAW4A32LinearOp::releaseDevice() {
  if (tiled_dev_ || workspace_dev_) {
    auto& be = registeredW4A32Backend();
    be.deviceFree(tiled_dev_);
    be.deviceFree(workspace_dev_);
  }
  tiled_dev_ = workspace_dev_ = nullptr;
  workspace_bytes_ = 0;
}

void CUDAW4A32LinearOp::growWorkspace(size_t need) {
  // the old block goes back to the backend's cache; work that still reads it was enqueued on the backend's
  // stream before this call and the next user of the block launches on the same stream
  auto& be = registeredW4A32Backend();
  be.deviceFree(workspace_dev_);
  workspace_dev_ = be.deviceAlloc(need);
  workspace_bytes_ = need;
}

void* uploadW4A32Weights(Tensor& weight, Tensor& bias, bool want_bias, int n, int k, const std::string& name) {
  std::vector<unsigned char> owned;  // holds the blob when it is produced here
  const void* blob = nullptr;
  size_t blob_bytes = 0;
  if (weight.dtype() == kInt8) {
    // the quantization pass's output: an opaque 1-D int8 tensor (KaiQuantizationPass.cpp:167-184 convention)
    blob = weight.ptr<unsigned char>();
    blob_bytes = weight.numel();
  } else if (weight.dtype() == kFp32) {
    // unquantized checkpoint: quantize at load time with the same routine the pass uses; any trailing
    // dimensions (a Conv3D kernel [O, C, kt, kh, kw]) are the row of the implied [N, K] matrix
    MLLM_RT_ASSERT_EQ((size_t)weight.numel(), (size_t)n * (size_t)k);
    const bool has_bias = want_bias && bias.dtype() == kFp32 && (int)bias.numel() == n;
    MLLMB200_CHECK(mllmb200_w4a32_prepack_size(n, k, has_bias, &blob_bytes));
    owned.resize(blob_bytes);
    MLLMB200_CHECK(mllmb200_w4a32_quant_prepack(weight.ptr<float>(), has_bias ? bias.ptr<float>() : nullptr, n, k,
                                                MLLMB200_SCALE_BF16_TRUNC, owned.data()));
    blob = owned.data();
  } else {
    MLLM_ERROR_EXIT(kError, "{}: weight dtype must be int8 (pre-packed) or fp32", name);
  }

  int bn = 0, bk = 0, scale_mode = 0, has_bias = 0;
  MLLMB200_CHECK(mllmb200_w4a32_blob_info(blob, blob_bytes, &bn, &bk, &scale_mode, &has_bias));
  if (bn != n || bk != k) { MLLM_ERROR_EXIT(kError, "{}: blob is {}x{} but the layer is {}x{}", name, bn, bk, n, k); }

  auto& be = registeredW4A32Backend();
  auto stream = static_cast<cudaStream_t>(be.stream());
  size_t tiled_bytes = 0;
  MLLMB200_CHECK(mllmb200_w4a32_tiled_size(n, k, &tiled_bytes));
  void* blob_dev = be.deviceAlloc(blob_bytes);
  void* tiled_dev = be.deviceAlloc(tiled_bytes);
  MLLMB200_CHECK_CUDA(cudaMemcpyAsync(blob_dev, blob, blob_bytes, cudaMemcpyHostToDevice, stream));
  MLLMB200_CHECK(mllmb200_w4a32_repack_device(blob_dev, n, k, scale_mode, has_bias, 0, n, tiled_dev, stream));
  MLLMB200_CHECK_CUDA(cudaStreamSynchronize(stream));  // `owned` (host) goes away below
  be.deviceFree(blob_dev);
  return tiled_dev;
}

void* uploadW4A16Weights(Tensor& weight, Tensor& bias, bool want_bias, int n, int k, const std::string& name) {
  std::vector<unsigned char> owned;
  const void* blob = nullptr;
  size_t blob_bytes = 0;
  if (weight.dtype() == kInt8) {
    blob = weight.ptr<unsigned char>();
    blob_bytes = weight.numel();
  } else if (weight.dtype() == kFp32) {
    MLLM_RT_ASSERT_EQ((size_t)weight.numel(), (size_t)n * (size_t)k);
    const bool has_bias = want_bias && bias.dtype() == kFp32 && (int)bias.numel() == n;
    MLLMB200_CHECK(mllmb200_w4a16_prepack_size(n, k, has_bias, &blob_bytes));
    owned.resize(blob_bytes);
    MLLMB200_CHECK(mllmb200_w4a16_quant_prepack(weight.ptr<float>(), has_bias ? bias.ptr<float>() : nullptr, n, k,
                                                owned.data()));
    blob = owned.data();
  } else {
    MLLM_ERROR_EXIT(kError, "{}: weight dtype must be int8 (pre-packed) or fp32", name);
  }
  int bn = 0, bk = 0, has_bias = 0;
  MLLMB200_CHECK(mllmb200_w4a16_blob_info(blob, blob_bytes, &bn, &bk, &has_bias));
  if (bn != n || bk != k) { MLLM_ERROR_EXIT(kError, "{}: blob is {}x{} but the layer is {}x{}", name, bn, bk, n, k); }

  auto& be = registeredW4A32Backend();
  auto stream = static_cast<cudaStream_t>(be.stream());
  size_t tiled_bytes = 0;
  MLLMB200_CHECK(mllmb200_w4a16_tiled_size(n, k, &tiled_bytes));
  void* blob_dev = be.deviceAlloc(blob_bytes);
  void* tiled_dev = be.deviceAlloc(tiled_bytes);
  MLLMB200_CHECK_CUDA(cudaMemcpyAsync(blob_dev, blob, blob_bytes, cudaMemcpyHostToDevice, stream));
  MLLMB200_CHECK(mllmb200_w4a16_repack_device(blob_dev, n, k, has_bias, 0, n, tiled_dev, stream));
  MLLMB200_CHECK_CUDA(cudaStreamSynchronize(stream));  // `owned` (host) goes away below
  be.deviceFree(blob_dev);
  return tiled_dev;
}

void CUDAW4A32LinearOp::load(const std::shared_ptr<ParameterLoader>& ploader) {
  LinearOp::load(ploader);  // weight_ / bias_ by name (mllm/Core/AOps/LinearOp.cpp:60-63)
  a16_ = isW4A16ImplType(cargo_.impl_type_);
  if (!a16_ && !isW4A32ImplType(cargo_.impl_type_)) {
    MLLM_ERROR_EXIT(kError, "CUDAW4A32LinearOp {}: impl type {} is neither a W4A32 nor a W4A16 Kai type; this backend "
                    "implements only those", name(), int(cargo_.impl_type_));
  }
  releaseDevice();
  k_ = cargo_.in_channels;
  n_ = cargo_.out_channels;
  if (weight_.dtype() == kFp32) {
    auto shape = weight_.shape();
    MLLM_RT_ASSERT_EQ(shape.size(), 2);
    MLLM_RT_ASSERT_EQ(shape[0], n_);
    MLLM_RT_ASSERT_EQ(shape[1], k_);
  }
  tiled_dev_ = a16_ ? uploadW4A16Weights(weight_, bias_, cargo_.bias, n_, k_, "CUDAW4A32LinearOp " + name())
                    : uploadW4A32Weights(weight_, bias_, cargo_.bias, n_, k_, "CUDAW4A32LinearOp " + name());
}

void CUDAW4A32LinearOp::reshape(const std::vector<Tensor>& inputs, std::vector<Tensor>& outputs) {
  const auto& i = inputs[0];
  auto o_shape = i.shape();
  MLLM_RT_ASSERT_EQ(o_shape[o_shape.size() - 1], cargo_.in_channels);
  o_shape[o_shape.size() - 1] = cargo_.out_channels;
  // W4A32: fp32 out whatever the tile; W4A16: fp16 out (ArmLinearOp::reshape, LinearOp.cpp:246-259).
  // reshape can run before load: decide from the cargo, not from a16_
  outputs.emplace_back(Tensor::empty(o_shape, isW4A16ImplType(cargo_.impl_type_) ? kFp16 : kFp32, i.device()));
}

void CUDAW4A32LinearOp::forward(const std::vector<Tensor>& inputs, std::vector<Tensor>& outputs) {
  const auto& x = inputs[0];
  auto& y = outputs[0];
  if (!tiled_dev_) { MLLM_ERROR_EXIT(kError, "CUDAW4A32LinearOp {}: forward before load", name()); }
  if (a16_) {
    // fp16 activations (the reference's model configs) or fp32 (its second matmul overload, kai_linear.cpp:853-901)
    if ((x.dtype() != kFp16 && x.dtype() != kFp32) || x.device() != kCUDA || y.dtype() != kFp16) {
      MLLM_ERROR_EXIT(kError, "CUDAW4A32LinearOp {}: W4A16 needs an fp16 or fp32 input on the CUDA device and an fp16 output",
                      name());
    }
    const int m = (int)(x.numel() / (size_t)k_);
    size_t need = 0;
    MLLMB200_CHECK(mllmb200_w4a16_workspace_size(m, k_, n_, &need));
    if (need > workspace_bytes_) growWorkspace(need);
    MLLMB200_CHECK(mllmb200_w4a16_linear_forward(x.ptr<unsigned char>(), x.dtype() == kFp16 ? MLLMB200_DTYPE_F16 : MLLMB200_DTYPE_F32,
                                                 tiled_dev_, y.ptr<unsigned char>(), workspace_dev_, m, k_, n_, k_, n_,
                                                 currentW4A32Stream()));
    return;
  }
  if (x.dtype() != kFp32 || x.device() != kCUDA) {
    MLLM_ERROR_EXIT(kError, "CUDAW4A32LinearOp {}: input must be fp32 on the CUDA device", name());
  }
  // every leading dimension is a row of the matrix product (the Arm kai path takes shape[-2] only,
  // LinearOp.cpp:34, which silently drops batches; here a [B,S,K] input is B*S rows)
  const int m = (int)(x.numel() / (size_t)k_);
  size_t need = 0;
  MLLMB200_CHECK(mllmb200_w4a32_workspace_size(m, k_, &need));
  // grow once and keep: the reference allocates a workspace tensor on every call (LinearOp.cpp:41-43)
  if (need > workspace_bytes_) growWorkspace(need);
  auto& be = registeredW4A32Backend();
  MLLMB200_CHECK(mllmb200_w4a32_linear_forward_ex(x.ptr<float>(), tiled_dev_, y.ptr<float>(), workspace_dev_, m, k_, n_, k_,
                                                  n_, be.linearKernelPolicy(), be.stream()));
}

}  // namespace mllm::cuda
