// Boundary test: the B200 W4A32 linear driven through the reference's OWN plugin API
// (MllmEngineCtx / BackendBase / nn::Module / nn::Linear / ParameterLoader / ir::PassManager),
// compiled against the reference's real classes.  Follows the shape of the reference's
// op-through-plugin test (tests/Arm/SingleConv3DTest.cpp:88-120): build a one-layer module, hand it
// a ParameterLoader, call it, compare with a scalar reference - here the CPU oracle.  The quantized
// parameters also make the trip through a .mllm file written and read by the reference's own code.
//
//   1. CudaQuantizationPass on a flat IR module (as tools/Quantizer/FlatModuleBuilder.cpp builds it):
//      the int8 blob's nibble and scale sections must equal the oracle's quantizer bit for bit.
//   2. model.load(blob) -> model.to(kCUDA) -> y = model(x): outputs within 1e-3 * rms of the oracle,
//      for M = 1 (GEMV), a [2,3,K] batch (M = 6) and M = 64 (tcgen05 path).
//   3. The same two steps for the W4A16 sibling format (impl type
//      KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk:qsi8d32p4x8_qai4c32p4x8_8x4_i8mm): blob sections equal
//      oracle/w4a16_oracle.c bit for bit, fp16 activations in, fp16 out.
//   4. Conv3D as a linear (the Qwen2VL patch embedding, K = 3*2*14*14 = 1176): the pass's Conv3D pattern on a
//      linalg Conv3DOp, then nn::Conv3D on the CUDA backend against im2col + the oracle's linear.
//   5. The quantizer tool's flow (tools/Quantizer/main.cpp:103-135 with the CUDA pass in the slot its x86 branch
//      leaves empty): a generated 28-layer parameter file and quantization config -> tools::createFlatModule ->
//      CudaQuantizationPass + the reference's CommonParamQuantizePass -> mllm::write -> mllm::load.
// Host <-> device moves go through the backend: cuda::toDevice(x) and Tensor::cpu() (the D2H op of the backend).
// Exit code 0 = all passed.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "CUDALinearOp.hpp"
#include "CUDAW4A32Backend.hpp"
#include "CudaQuantizationPass.hpp"
#include "HostShimBackend.hpp"
#include "mllm/Engine/Context.hpp"
#include "mllm/Engine/ParameterReader.hpp"
#include "mllm/IR/Builtin/Op.hpp"
#include "mllm/IR/Graph/Op.hpp"
#include "mllm/IR/Linalg/Op.hpp"
#include "mllm/IR/Passes/PassManager.hpp"
#include "mllm/IR/Passes/QuantizePass.hpp"
#include "mllm/IR/Tensor/Op.hpp"
#include "mllm/Nn/HierarchyBase.hpp"
#include "mllm/Nn/Layers/Conv3D.hpp"
#include "mllm/Nn/Layers/Linear.hpp"
#include "tools/Quantizer/FlatModuleBuilder.hpp"
#include "mllm/Nn/Module.hpp"
#include "mllmb200.h"

extern "C" {  // oracle/w4a32_oracle.c
void oracle_quant_nxk_qs4c32_f32(size_t n, size_t k, size_t bl, const float* rhs, uint8_t* q, uint16_t* s, int mode);
void oracle_linear_w4a32(size_t m, size_t n, size_t k, const float* x, const uint8_t* q, const uint16_t* s, int mode,
                         const float* bias, float* y, void* workspace);
// oracle/w4a16_oracle.c
void oracle_w4a16_quant_nxk_qai4c32_f32(size_t n, size_t k, size_t bl, const float* rhs, uint8_t* q, float* zeros,
                                        float* scales, int32_t* zp);
void oracle_linear_w4a16(size_t m, size_t n, size_t k, const float* x, const uint8_t* q, const float* scales,
                         const float* zeros, const float* bias, uint16_t* y_f16, void* ws);
uint16_t oracle_cast_f16_f32(float f);
float oracle_cast_f32_f16(uint16_t h);
}

using namespace mllm;

namespace {

constexpr auto kImpl = LinearOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp4x8_qsi4c32p4x8_8x4x32;
constexpr auto kImplA16 = LinearOpImplType::KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk_qsi8d32p4x8_qai4c32p4x8_8x4_i8mm;

class SingleLinear final : public nn::Module {
 public:
  nn::Linear fc_;
  SingleLinear() = default;
  SingleLinear(const std::string& name, int k, int n, bool bias, LinearOpImplType impl = kImpl) {
    selfAssignName(name);
    fc_ = reg<nn::Linear>("fc", k, n, bias, false, impl);
  }
  std::vector<Tensor> forward(const std::vector<Tensor>& inputs) override { return {fc_(inputs[0])}; }
};

uint32_t g_rng = 12345u;
float frand() {  // uniform in [-1, 1)
  g_rng = g_rng * 1664525u + 1013904223u;
  return (float)((g_rng >> 8) & 0xFFFFFF) / 8388608.0f - 1.0f;
}

// Flat IR module holding one linalg LinearOp, the way the quantizer tool builds it.
std::shared_ptr<ir::IRContext> flatModule(const std::shared_ptr<BaseOp>& op) {
  auto ir_ctx = std::make_shared<ir::IRContext>();
  ir_ctx->createAndSetModuleOp<ir::ModuleOp>(ir_ctx->create<ir::SymbolAttr>("main"));
  ir_ctx->create<ir::graph::CallGraphOp>(ir_ctx->create<ir::SymbolAttr>("flat"));
  std::shared_ptr<ir::graph::SubGraphOp> graph = nullptr;
  {
    auto guard = ir::IRWriterGuard(ir_ctx, ir_ctx->topLevelOp()->cast_<ir::ModuleOp>()->getTopRegion());
    graph = ir_ctx->create<ir::graph::SubGraphOp>(ir_ctx->create<ir::SymbolAttr>("flat"),
                                                  std::make_shared<HierarchyBase>(HierarchyTypes::kModule));
  }
  graph->setDevice(kCPU);
  {
    auto guard = ir::IRWriterGuard(ir_ctx, graph->getTopRegion());
    ir_ctx->create<ir::linalg::LinearOp>(op, std::vector<ir::tensor::TensorValue::self_ptr_t>{},
                                         std::vector<ir::tensor::TensorValue::self_ptr_t>{});
  }
  return ir_ctx;
}

int g_failures = 0;
bool g_host_only = false;  // --host-only: quantization pass only (no CUDA device needed)
void check(bool ok, const char* what) {
  std::printf("[%s] %s\n", ok ? " ok " : "FAIL", what);
  if (!ok) ++g_failures;
}

void runCase(const std::string& model, int k, int n, bool with_bias, const std::vector<std::vector<int32_t>>& x_shapes) {
  const std::string layer = model + ".fc";
  auto& ctx = MllmEngineCtx::instance();
  char label[256];

  // ---- fp32 parameters
  Tensor w = Tensor::empty({n, k}, kFp32, kCPU).alloc();
  Tensor b = Tensor::empty({n}, kFp32, kCPU).alloc();
  for (int i = 0; i < n * k; ++i) w.ptr<float>()[i] = frand() * 0.05f;
  for (int i = 0; i < n; ++i) b.ptr<float>()[i] = frand() * 0.1f;
  w.setName(layer + ".weight");
  b.setName(layer + ".bias");

  // ---- 1. the quantization pass, through the reference's PassManager
  auto host_op = ctx.getBackend(kCPU)->createOp(
      OpType::kLinear, LinearOpCargo{.in_channels = k, .out_channels = n, .bias = with_bias, .transpose = false});
  host_op->setName(layer);
  auto* host_linear = (LinearOp*)host_op.get();
  host_linear->weight() = w;
  if (with_bias) host_linear->bias() = b;
  MllmModelCfg cfg;
  cfg.rawJson()["Ops"][layer] = {{"type", "Linear"},
                                 {"implType", "KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk:qai8dxp4x8_qsi4c32p4x8_8x4x32"}};
  auto ir_ctx = flatModule(host_op);
  auto pass = cuda::createCudaQuantizationPass(cfg);
  ir::PassManager pm(ir_ctx);
  pm.reg(pass);
  const bool pm_ok = pm.run();
  std::snprintf(label, sizeof(label), "K=%d N=%d bias=%d: pass ran and quantized one linear", k, n, (int)with_bias);
  check(pm_ok && pass->quantizedCount() == 1, label);
  Tensor blob = host_linear->weight();
  check(blob.dtype() == kInt8 && blob.shape().size() == 1 && blob.name() == layer + ".weight",
        "  weight replaced by a 1-D int8 tensor of the same name");
  check(host_linear->bias().dtype() == kInt8 && host_linear->bias().numel() == 1, "  bias replaced by the 1-byte placeholder");

  // blob sections vs the oracle's quantizer, bit for bit
  const size_t ns = (size_t)(k + 1) / 2, nb = (size_t)(k + 31) / 32;
  std::vector<uint8_t> q_ref(n * ns);
  std::vector<uint16_t> s_ref(n * nb);
  oracle_quant_nxk_qs4c32_f32(n, k, 32, w.ptr<float>(), q_ref.data(), s_ref.data(), 0);
  size_t off_q = 0, off_s = 0, off_b = 0;
  mllmb200_w4a32_blob_offsets(n, k, with_bias, &off_q, &off_s, &off_b);
  const uint8_t* blob_bytes = blob.ptr<uint8_t>();
  check(std::memcmp(blob_bytes + off_q, q_ref.data(), q_ref.size()) == 0, "  nibbles bit-identical to the oracle");
  check(std::memcmp(blob_bytes + off_s, s_ref.data(), s_ref.size() * 2) == 0, "  scales bit-identical to the oracle");
  if (with_bias) check(std::memcmp(blob_bytes + off_b, b.ptr<float>(), n * 4) == 0, "  bias carried inside the blob");

  // ---- 1b. the .mllm parameter file: what mllm-quantizer writes after its pass
  // (tools/Quantizer/main.cpp -> mllm::write) and what a model loads (mllm::load): the blob must
  // come back byte for byte under the same name and dtype, through the reference's own writer/reader
  Tensor bias_placeholder = host_linear->bias();
  const std::string file = "/tmp/mllmb200_boundary_" + model + ".mllm";
  {
    std::unordered_map<std::string, Tensor> params;
    params.insert({layer + ".weight", blob});
    if (with_bias) params.insert({layer + ".bias", bias_placeholder});
    mllm::write(file, params, model);
  }
  auto ploader = mllm::load(file);
  {
    auto back = ploader->params().find(layer + ".weight");
    bool ok = back != ploader->params().end();
    if (ok) {
      Tensor t(back->second);
      ok = t.dtype() == kInt8 && (size_t)t.numel() == (size_t)blob.numel() &&
           std::memcmp(t.ptr<uint8_t>(), blob.ptr<uint8_t>(), blob.numel()) == 0;
    }
    check(ok, "  .mllm round trip (reference ParameterWriter -> ParameterLoader): blob byte-identical");
    if (with_bias) check(ploader->params().count(layer + ".bias") == 1, "  .mllm round trip: bias placeholder present");
  }

  if (g_host_only) {
    std::remove(file.c_str());
    return;
  }
  // ---- 2. one-layer module: load from the parameter file, move to the GPU, run
  auto net = SingleLinear(model, k, n, with_bias);
  net.load(ploader);
  net.to(kCUDA);
  auto stream = static_cast<cudaStream_t>(cuda::currentW4A32Stream());

  for (const auto& shape : x_shapes) {
    size_t numel = 1;
    for (auto d : shape) numel *= (size_t)d;
    const int m = (int)(numel / (size_t)k);
    std::vector<float> x_host(numel), y_host((size_t)m * n), y_ref((size_t)m * n);
    for (auto& v : x_host) v = frand() * 2.0f;
    // host tensor -> the backend's toDevice -> the module -> Tensor::cpu() (the backend's D2H op)
    Tensor x_cpu = Tensor::empty(shape, kFp32, kCPU).alloc();
    std::memcpy(x_cpu.ptr<float>(), x_host.data(), numel * 4);
    Tensor x = cuda::toDevice(x_cpu);
    Tensor y = net(x)[0];
    Tensor y_cpu = y.cpu();
    std::memcpy(y_host.data(), y_cpu.ptr<float>(), y_host.size() * 4);
    const cudaError_t e = cudaStreamSynchronize(stream);
    const int dev_status = mllmb200_check_device_status(stream);
    std::vector<uint8_t> ws((size_t)m * (k + 8));
    oracle_linear_w4a32(m, n, k, x_host.data(), q_ref.data(), s_ref.data(), 0, with_bias ? b.ptr<float>() : nullptr,
                        y_ref.data(), ws.data());
    double sq = 0, err = 0;
    for (size_t i = 0; i < y_ref.size(); ++i) {
      sq += (double)y_ref[i] * y_ref[i];
      err = std::fmax(err, std::fabs((double)y_host[i] - y_ref[i]));
    }
    const double rms = std::sqrt(sq / y_ref.size());
    auto y_shape = y.shape();
    bool shape_ok = y_shape.size() == shape.size() && y_shape.back() == n && y.dtype() == kFp32 && y.device() == kCUDA;
    for (size_t d = 0; d + 1 < shape.size(); ++d) shape_ok = shape_ok && y_shape[d] == shape[d];
    std::snprintf(label, sizeof(label), "  forward M=%d: max|diff| %.3e <= 1e-3 * rms %.3e, shape/dtype/device ok", m, err, rms);
    check(e == cudaSuccess && dev_status == 0 && shape_ok && err <= 1e-3 * rms, label);
  }
}

// The W4A16 sibling format through the same plugin API: impl type 11, fp16 activations in, fp16 out.
void runCaseA16(const std::string& model, int k, int n, bool with_bias, const std::vector<std::vector<int32_t>>& x_shapes) {
  const std::string layer = model + ".fc";
  auto& ctx = MllmEngineCtx::instance();
  char label[256];
  Tensor w = Tensor::empty({n, k}, kFp32, kCPU).alloc();
  Tensor b = Tensor::empty({n}, kFp32, kCPU).alloc();
  for (int i = 0; i < n * k; ++i) w.ptr<float>()[i] = frand() * 0.05f;
  for (int i = 0; i < n; ++i) b.ptr<float>()[i] = frand() * 0.1f;
  w.setName(layer + ".weight");
  b.setName(layer + ".bias");

  auto host_op = ctx.getBackend(kCPU)->createOp(
      OpType::kLinear, LinearOpCargo{.in_channels = k, .out_channels = n, .bias = with_bias, .transpose = false});
  host_op->setName(layer);
  auto* host_linear = (LinearOp*)host_op.get();
  host_linear->weight() = w;
  if (with_bias) host_linear->bias() = b;
  MllmModelCfg cfg;
  cfg.rawJson()["Ops"][layer] = {{"type", "Linear"},
                                 {"implType", "KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk:qsi8d32p4x8_qai4c32p4x8_8x4_i8mm"}};
  auto ir_ctx = flatModule(host_op);
  auto pass = cuda::createCudaQuantizationPass(cfg);
  ir::PassManager pm(ir_ctx);
  pm.reg(pass);
  const bool pm_ok = pm.run();
  std::snprintf(label, sizeof(label), "W4A16 K=%d N=%d bias=%d: pass ran and quantized one linear", k, n, (int)with_bias);
  check(pm_ok && pass->quantizedCount() == 1, label);
  Tensor blob = host_linear->weight();
  check(blob.dtype() == kInt8 && blob.shape().size() == 1 && blob.name() == layer + ".weight",
        "  weight replaced by a 1-D int8 tensor of the same name");

  const size_t ns = (size_t)(k + 1) / 2, nb = (size_t)(k + 31) / 32;
  std::vector<uint8_t> q_ref(n * ns);
  std::vector<float> s_ref(n * nb), z_ref(n * nb);
  oracle_w4a16_quant_nxk_qai4c32_f32(n, k, 32, w.ptr<float>(), q_ref.data(), z_ref.data(), s_ref.data(), nullptr);
  size_t off_q = 0, off_s = 0, off_z = 0, off_b = 0;
  mllmb200_w4a16_blob_offsets(n, k, with_bias, &off_q, &off_s, &off_z, &off_b);
  const uint8_t* blob_bytes = blob.ptr<uint8_t>();
  check(std::memcmp(blob_bytes + off_q, q_ref.data(), q_ref.size()) == 0, "  nibbles bit-identical to the oracle");
  check(std::memcmp(blob_bytes + off_s, s_ref.data(), s_ref.size() * 4) == 0, "  scales bit-identical to the oracle");
  check(std::memcmp(blob_bytes + off_z, z_ref.data(), z_ref.size() * 4) == 0, "  zero terms bit-identical to the oracle");
  if (with_bias) check(std::memcmp(blob_bytes + off_b, b.ptr<float>(), n * 4) == 0, "  bias carried inside the blob");

  const std::string file = "/tmp/mllmb200_boundary_" + model + ".mllm";
  {
    std::unordered_map<std::string, Tensor> params;
    params.insert({layer + ".weight", blob});
    if (with_bias) params.insert({layer + ".bias", host_linear->bias()});
    mllm::write(file, params, model);
  }
  auto ploader = mllm::load(file);
  {
    auto back = ploader->params().find(layer + ".weight");
    bool ok = back != ploader->params().end();
    if (ok) {
      Tensor t(back->second);
      ok = t.dtype() == kInt8 && (size_t)t.numel() == (size_t)blob.numel() &&
           std::memcmp(t.ptr<uint8_t>(), blob.ptr<uint8_t>(), blob.numel()) == 0;
    }
    check(ok, "  .mllm round trip (reference ParameterWriter -> ParameterLoader): blob byte-identical");
  }
  if (g_host_only) {
    std::remove(file.c_str());
    return;
  }
  auto net = SingleLinear(model, k, n, with_bias, kImplA16);
  net.load(ploader);
  net.to(kCUDA);
  auto stream = static_cast<cudaStream_t>(cuda::currentW4A32Stream());
  for (const auto& shape : x_shapes) {
    size_t numel = 1;
    for (auto d : shape) numel *= (size_t)d;
    const int m = (int)(numel / (size_t)k);
    std::vector<uint16_t> x_half(numel), y_half((size_t)m * n), y_ref((size_t)m * n);
    std::vector<float> x_wide(numel);
    for (size_t i = 0; i < numel; ++i) {
      x_half[i] = oracle_cast_f16_f32(frand() * 2.0f);
      x_wide[i] = oracle_cast_f32_f16(x_half[i]);
    }
    Tensor x = Tensor::empty(shape, kFp16, kCUDA).alloc();
    cudaMemcpyAsync(x.ptr<uint8_t>(), x_half.data(), numel * 2, cudaMemcpyHostToDevice, stream);
    Tensor y = net(x)[0];
    cudaMemcpyAsync(y_half.data(), y.ptr<uint8_t>(), y_half.size() * 2, cudaMemcpyDeviceToHost, stream);
    const cudaError_t e = cudaStreamSynchronize(stream);
    const int dev_status = mllmb200_check_device_status(stream);
    std::vector<uint8_t> ws((size_t)m * nb * 36);
    oracle_linear_w4a16(m, n, k, x_wide.data(), q_ref.data(), s_ref.data(), z_ref.data(),
                        with_bias ? b.ptr<float>() : nullptr, y_ref.data(), ws.data());
    double sq = 0;
    for (size_t i = 0; i < y_ref.size(); ++i) sq += (double)oracle_cast_f32_f16(y_ref[i]) * oracle_cast_f32_f16(y_ref[i]);
    const double rms = std::sqrt(sq / y_ref.size());
    // dp4a kernels: 1e-3 * rms; tensor-core kernel (M >= 128, operands rounded to fp16): 4e-3 * rms; + 2 fp16 ulps
    const double bar = m >= 128 ? 4e-3 : 1e-3;
    double worst = 0;
    bool within = true;
    for (size_t i = 0; i < y_ref.size(); ++i) {
      const double r = oracle_cast_f32_f16(y_ref[i]), g = oracle_cast_f32_f16(y_half[i]);
      const double d = std::fabs(g - r);
      worst = std::fmax(worst, d);
      within = within && d <= bar * rms + 2.0 * std::fabs(r) / 1024.0;
    }
    auto y_shape = y.shape();
    bool shape_ok = y_shape.size() == shape.size() && y_shape.back() == n && y.dtype() == kFp16 && y.device() == kCUDA;
    for (size_t d = 0; d + 1 < shape.size(); ++d) shape_ok = shape_ok && y_shape[d] == shape[d];
    std::snprintf(label, sizeof(label), "  W4A16 forward M=%d: max|diff| %.3e (rms %.3e), fp16 out, shape/device ok", m, worst, rms);
    check(e == cudaSuccess && dev_status == 0 && shape_ok && within, label);
  }
}

constexpr auto kImplConv = Conv3DOpImplType::kKaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk_qai8dxp4x8_qsi4c32p4x8_8x4x32;

class SingleConv3D final : public nn::Module {
 public:
  nn::Conv3D conv_;
  SingleConv3D() = default;
  SingleConv3D(const std::string& name, int c, int o, const std::vector<int32_t>& kernel, const std::vector<int32_t>& stride,
               bool bias) {
    selfAssignName(name);
    conv_ = reg<nn::Conv3D>("proj", c, o, kernel, stride, bias, kImplConv);
  }
  std::vector<Tensor> forward(const std::vector<Tensor>& inputs) override { return {conv_(inputs[0])}; }
};

// Conv3D as a W4A32 linear through the plugin API: the pass's Conv3D pattern, a .mllm round trip, nn::Conv3D on
// the CUDA backend.  Reference flow: mllm/Backends/Arm/Ops/Conv3DOp.cpp:31-170 (im2col -> matmul -> permute).
void runConv3D(const std::string& model, int c, int o, const std::vector<int32_t>& kernel, const std::vector<int32_t>& stride,
               bool with_bias, const std::vector<int32_t>& in_shape /* B, C, T, H, W */) {
  const std::string layer = model + ".proj";
  auto& ctx = MllmEngineCtx::instance();
  char label[256];
  const int k = c * kernel[0] * kernel[1] * kernel[2];
  Tensor w = Tensor::empty({o, c, kernel[0], kernel[1], kernel[2]}, kFp32, kCPU).alloc();
  Tensor b = Tensor::empty({o}, kFp32, kCPU).alloc();
  for (int i = 0; i < o * k; ++i) w.ptr<float>()[i] = frand() * 0.05f;
  for (int i = 0; i < o; ++i) b.ptr<float>()[i] = frand() * 0.1f;
  w.setName(layer + ".weight");
  b.setName(layer + ".bias");

  // ---- the pass on a linalg Conv3DOp
  auto host_op = ctx.getBackend(kCPU)->createOp(
      OpType::kConv3D, Conv3DOpCargo{.in_channels = c, .out_channels = o, .kernel_size = kernel, .stride = stride,
                                     .bias = with_bias, .impl_type = kImplConv});
  host_op->setName(layer);
  auto* host_conv = (Conv3DOp*)host_op.get();
  host_conv->weight() = w;
  if (with_bias) host_conv->bias() = b;
  MllmModelCfg cfg;
  cfg.rawJson()["Ops"][layer] = {{"type", "Conv3D"},
                                 {"implType", "KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk:qai8dxp4x8_qsi4c32p4x8_8x4x32"}};
  auto ir_ctx = std::make_shared<ir::IRContext>();
  ir_ctx->createAndSetModuleOp<ir::ModuleOp>(ir_ctx->create<ir::SymbolAttr>("main"));
  ir_ctx->create<ir::graph::CallGraphOp>(ir_ctx->create<ir::SymbolAttr>("flat"));
  std::shared_ptr<ir::graph::SubGraphOp> graph = nullptr;
  {
    auto guard = ir::IRWriterGuard(ir_ctx, ir_ctx->topLevelOp()->cast_<ir::ModuleOp>()->getTopRegion());
    graph = ir_ctx->create<ir::graph::SubGraphOp>(ir_ctx->create<ir::SymbolAttr>("flat"),
                                                  std::make_shared<HierarchyBase>(HierarchyTypes::kModule));
  }
  graph->setDevice(kCPU);
  {
    auto guard = ir::IRWriterGuard(ir_ctx, graph->getTopRegion());
    ir_ctx->create<ir::linalg::Conv3DOp>(host_op, std::vector<ir::tensor::TensorValue::self_ptr_t>{},
                                         std::vector<ir::tensor::TensorValue::self_ptr_t>{});
  }
  auto pass = cuda::createCudaQuantizationPass(cfg);
  ir::PassManager pm(ir_ctx);
  pm.reg(pass);
  const bool pm_ok = pm.run();
  std::snprintf(label, sizeof(label), "Conv3D C=%d O=%d K=%d bias=%d: pass ran and quantized one conv3d", c, o, k, (int)with_bias);
  check(pm_ok && pass->quantizedCount() == 1, label);
  Tensor blob = host_conv->weight();
  check(blob.dtype() == kInt8 && blob.shape().size() == 1 && blob.name() == layer + ".weight",
        "  kernel replaced by a 1-D int8 tensor of the same name");
  const size_t ns = (size_t)(k + 1) / 2, nb = (size_t)(k + 31) / 32;
  std::vector<uint8_t> q_ref(o * ns);
  std::vector<uint16_t> s_ref(o * nb);
  oracle_quant_nxk_qs4c32_f32(o, k, 32, w.ptr<float>(), q_ref.data(), s_ref.data(), 0);
  size_t off_q = 0, off_s = 0, off_b = 0;
  mllmb200_w4a32_blob_offsets(o, k, with_bias, &off_q, &off_s, &off_b);
  check(std::memcmp(blob.ptr<uint8_t>() + off_q, q_ref.data(), q_ref.size()) == 0 &&
            std::memcmp(blob.ptr<uint8_t>() + off_s, s_ref.data(), s_ref.size() * 2) == 0,
        "  nibbles and scales of the [O, C*kt*kh*kw] matrix bit-identical to the oracle");

  const std::string file = "/tmp/mllmb200_boundary_" + model + ".mllm";
  {
    std::unordered_map<std::string, Tensor> params;
    params.insert({layer + ".weight", blob});
    if (with_bias) params.insert({layer + ".bias", host_conv->bias()});
    mllm::write(file, params, model);
  }
  auto ploader = mllm::load(file);
  if (g_host_only) {
    std::remove(file.c_str());
    return;
  }
  // ---- nn::Conv3D on the CUDA backend
  auto net = SingleConv3D(model, c, o, kernel, stride, with_bias);
  net.load(ploader);
  net.to(kCUDA);
  auto stream = static_cast<cudaStream_t>(cuda::currentW4A32Stream());
  const int B = in_shape[0], T = in_shape[2], H = in_shape[3], W = in_shape[4];
  const int To = (T - kernel[0]) / stride[0] + 1, Ho = (H - kernel[1]) / stride[1] + 1, Wo = (W - kernel[2]) / stride[2] + 1;
  const int m = B * To * Ho * Wo;
  Tensor x_cpu = Tensor::empty(in_shape, kFp32, kCPU).alloc();
  const size_t numel = (size_t)B * c * T * H * W;
  for (size_t i = 0; i < numel; ++i) x_cpu.ptr<float>()[i] = frand() * 2.0f;
  Tensor y = net(cuda::toDevice(x_cpu))[0];
  Tensor y_cpu = y.cpu();
  const cudaError_t e = cudaStreamSynchronize(stream);
  const int dev_status = mllmb200_check_device_status(stream);
  // im2col in the op's order: rows (b, t', h', w'), columns (c, kt, kh, kw); then the oracle's linear
  std::vector<float> cols((size_t)m * k), y_lin((size_t)m * o);
  const float* xp = x_cpu.ptr<float>();
  for (int bi = 0; bi < B; ++bi)
    for (int t = 0; t < To; ++t)
      for (int h = 0; h < Ho; ++h)
        for (int wv = 0; wv < Wo; ++wv) {
          float* row = cols.data() + (size_t)(((bi * To + t) * Ho + h) * Wo + wv) * k;
          for (int ci = 0; ci < c; ++ci)
            for (int kt = 0; kt < kernel[0]; ++kt)
              for (int kh = 0; kh < kernel[1]; ++kh)
                for (int kw = 0; kw < kernel[2]; ++kw)
                  *row++ = xp[((((size_t)bi * c + ci) * T + t * stride[0] + kt) * H + h * stride[1] + kh) * W + wv * stride[2] + kw];
        }
  std::vector<uint8_t> ws((size_t)m * (k + 8));
  oracle_linear_w4a32(m, o, k, cols.data(), q_ref.data(), s_ref.data(), 0, with_bias ? b.ptr<float>() : nullptr, y_lin.data(),
                      ws.data());
  // the op's output is [B, O, T', H', W']
  double sq = 0, err = 0;
  const float* yp = y_cpu.ptr<float>();
  for (int bi = 0; bi < B; ++bi)
    for (int oc = 0; oc < o; ++oc)
      for (int t = 0; t < To; ++t)
        for (int h = 0; h < Ho; ++h)
          for (int wv = 0; wv < Wo; ++wv) {
            const double ref = y_lin[(size_t)(((bi * To + t) * Ho + h) * Wo + wv) * o + oc];
            const double got = yp[((((size_t)bi * o + oc) * To + t) * Ho + h) * Wo + wv];
            sq += ref * ref;
            err = std::fmax(err, std::fabs(got - ref));
          }
  const double rms = std::sqrt(sq / ((double)m * o));
  auto ys = y.shape();
  const bool shape_ok = ys.size() == 5 && ys[0] == B && ys[1] == o && ys[2] == To && ys[3] == Ho && ys[4] == Wo && y.dtype() == kFp32;
  std::snprintf(label, sizeof(label), "  nn::Conv3D forward, %d patches: max|diff| %.3e <= 1e-3 * rms %.3e, [B,O,T',H',W'] ok", m, err, rms);
  check(e == cudaSuccess && dev_status == 0 && shape_ok && err <= 1e-3 * rms, label);
}

// The quantizer tool's flow on a generated model: 28 layers with the parameter names of the 1.5B checkpoint
// (reduced widths so that the fp32 file stays small), a config that lists every quantized linear of every layer
// (the shipped one lists layer 0 only and misspells one key, scripts/QuantCfg/ds_qwen2/1.5B-W4A32-KAI.json:12) and
// casts norms and lm_head to fp16.  Host only.
void runQuantizerFlow() {
  char label[256];
  const int layers = 28, H = 64, QD = 64, KD = 32, I = 160, V = 96;
  const char* lin_names[7] = {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                              "mlp.gate_proj",    "mlp.up_proj",      "mlp.down_proj"};
  const int lin_n[7] = {QD, KD, KD, H, I, I, H}, lin_k[7] = {H, H, H, QD, H, H, I};
  const bool lin_bias[7] = {true, true, true, false, false, false, false};
  std::unordered_map<std::string, Tensor> params;
  std::unordered_map<std::string, std::vector<float>> keep;  // fp32 copies for the oracle
  auto add = [&](const std::string& name, const std::vector<int32_t>& shape, float scale) {
    Tensor t = Tensor::empty(shape, kFp32, kCPU).alloc();
    size_t n = 1;
    for (auto d : shape) n *= (size_t)d;
    auto& copy = keep[name];
    copy.resize(n);
    for (size_t i = 0; i < n; ++i) copy[i] = t.ptr<float>()[i] = frand() * scale;
    t.setName(name);
    params.insert({name, t});
  };
  MllmModelCfg cfg;
  cfg.rawJson()["ModelName"] = "generated-qwen2-28-layers";
  add("model.embed_tokens.weight", {V, H}, 1.0f);
  add("model.norm.weight", {H}, 1.0f);
  add("lm_head.weight", {V, H}, 0.05f);
  for (int l = 0; l < layers; ++l) {
    const std::string base = "model.layers." + std::to_string(l) + ".";
    add(base + "input_layernorm.weight", {H}, 1.0f);
    add(base + "post_attention_layernorm.weight", {H}, 1.0f);
    for (int i = 0; i < 7; ++i) {
      add(base + lin_names[i] + ".weight", {lin_n[i], lin_k[i]}, 0.05f);
      if (lin_bias[i]) add(base + lin_names[i] + ".bias", {lin_n[i]}, 0.1f);
      cfg.rawJson()["Ops"][base + lin_names[i]] = {{"type", "Linear"},
                                                   {"implType", "KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk:qai8dxp4x8_qsi4c32p4x8_8x4x32"}};
    }
  }
  cfg.rawJson()["Params"]["^model\\.layers\\.\\d+\\.post_attention_layernorm\\.weight$"] = {{"dtype", "Fp16"}};
  cfg.rawJson()["Params"]["^model\\.layers\\.\\d+\\.input_layernorm\\.weight$"] = {{"dtype", "Fp16"}};
  cfg.rawJson()["Params"]["^model.norm.weight$"] = {{"dtype", "Fp16"}};
  cfg.rawJson()["Params"]["^lm_head.weight$"] = {{"dtype", "Fp16"}};
  const std::string in_file = "/tmp/mllmb200_quantflow_fp32.mllm", out_file = "/tmp/mllmb200_quantflow_w4a32.mllm";
  mllm::write(in_file, params, "generated-qwen2-28-layers");
  params.clear();

  // ---- tools/Quantizer/main.cpp:103-135, with the CUDA pass registered where the x86 branch registers none
  auto loader = mllm::load(in_file);
  std::vector<std::shared_ptr<BaseOp>> quantized_ops;
  auto ir_ctx = tools::createFlatModule(quantized_ops, loader, cfg);
  for (auto& op : quantized_ops) op->load(loader);
  ir::PassManager pm(ir_ctx);
  auto pass = cuda::createCudaQuantizationPass(cfg);
  pm.reg(pass);
  pm.reg(ir::createCommonParamQuantizePass(cfg));
  const bool pm_ok = pm.run();
  std::snprintf(label, sizeof(label), "quantizer flow: createFlatModule found %zu linears, the pass quantized %d", quantized_ops.size(),
                pass->quantizedCount());
  check(pm_ok && (int)quantized_ops.size() == layers * 7 && pass->quantizedCount() == layers * 7, label);
  for (auto& op : quantized_ops)
    for (auto& kv : op->params()) loader->params()[kv.first] = kv.second.impl();
  {
    auto init_params_graph = ir_ctx->lookupSymbolTable("init_params")->cast_<ir::graph::SubGraphOp>();
    auto r = ir::IRWriter(ir_ctx, init_params_graph->getTopRegion());
    r.walk<ir::tensor::AllocGlobalOp>([&](ir::IRWriter&, const ir::tensor::AllocGlobalOp::self_ptr_t& op) -> ir::IRWriter::WalkResult {
      auto pt = (op->outputs().front())->cast_<ir::tensor::TensorValue>();
      loader->params()[pt->getSymbolAttr()->str()] = pt->tensor_.impl();
      return ir::IRWriter::WalkResult::WALK_CONTINUE;
    });
  }
  mllm::write(out_file, loader->params(), cfg.modelName());

  // ---- read it back: every linear is a blob whose sections equal the oracle's quantizer; norms and lm_head are fp16
  auto back = mllm::load(out_file);
  bool blobs_ok = true, dtypes_ok = true;
  int checked = 0;
  for (int l = 0; l < layers; ++l) {
    const std::string base = "model.layers." + std::to_string(l) + ".";
    for (int i = 0; i < 7; ++i) {
      const std::string name = base + lin_names[i] + ".weight";
      auto it = back->params().find(name);
      if (it == back->params().end()) {
        blobs_ok = false;
        continue;
      }
      Tensor t(it->second);
      int bn = 0, bk = 0, mode = -1, hb = -1;
      if (t.dtype() != kInt8 || mllmb200_w4a32_blob_info(t.ptr<uint8_t>(), t.numel(), &bn, &bk, &mode, &hb) != MLLMB200_OK ||
          bn != lin_n[i] || bk != lin_k[i] || hb != (lin_bias[i] ? 1 : 0)) {
        blobs_ok = false;
        continue;
      }
      const size_t ns = (size_t)(bk + 1) / 2, nb = (size_t)(bk + 31) / 32;
      std::vector<uint8_t> q_ref(bn * ns);
      std::vector<uint16_t> s_ref(bn * nb);
      oracle_quant_nxk_qs4c32_f32(bn, bk, 32, keep[name].data(), q_ref.data(), s_ref.data(), 0);
      size_t off_q = 0, off_s = 0, off_b = 0;
      mllmb200_w4a32_blob_offsets(bn, bk, hb, &off_q, &off_s, &off_b);
      blobs_ok = blobs_ok && std::memcmp(t.ptr<uint8_t>() + off_q, q_ref.data(), q_ref.size()) == 0 &&
                 std::memcmp(t.ptr<uint8_t>() + off_s, s_ref.data(), s_ref.size() * 2) == 0;
      if (lin_bias[i]) {
        blobs_ok = blobs_ok && std::memcmp(t.ptr<uint8_t>() + off_b, keep[base + lin_names[i] + ".bias"].data(), (size_t)bn * 4) == 0;
        auto bit = back->params().find(base + lin_names[i] + ".bias");
        blobs_ok = blobs_ok && bit != back->params().end() && Tensor(bit->second).dtype() == kInt8;
      }
      ++checked;
    }
    for (const char* norm : {"input_layernorm.weight", "post_attention_layernorm.weight"}) {
      auto it = back->params().find(base + norm);
      dtypes_ok = dtypes_ok && it != back->params().end() && Tensor(it->second).dtype() == kFp16;
    }
  }
  for (const char* name : {"model.norm.weight", "lm_head.weight"}) {
    auto it = back->params().find(name);
    dtypes_ok = dtypes_ok && it != back->params().end() && Tensor(it->second).dtype() == kFp16;
  }
  {
    auto it = back->params().find("model.embed_tokens.weight");
    dtypes_ok = dtypes_ok && it != back->params().end() && Tensor(it->second).dtype() == kFp32;
  }
  std::snprintf(label, sizeof(label), "  written file read back: %d linear blobs bit-identical to the oracle's quantizer", checked);
  check(blobs_ok && checked == layers * 7, label);
  check(dtypes_ok, "  norms and lm_head cast to fp16 by the reference's CommonParamQuantizePass, embedding left fp32");
  std::remove(in_file.c_str());
  std::remove(out_file.c_str());
}

}  // namespace

int main(int argc, char** argv) {
  g_host_only = argc > 1 && std::strcmp(argv[1], "--host-only") == 0;
  std::setvbuf(stdout, nullptr, _IOLBF, 0);
  auto& ctx = MllmEngineCtx::instance();
  ctx.registerBackend(std::make_shared<shim::HostShimBackend>());
  ctx.mem()->initBuddyCtx(kCPU);
  ctx.mem()->initOC(kCPU);
  if (!g_host_only) {
    ctx.registerBackend(cuda::createCUDAW4A32Backend());
    ctx.mem()->initBuddyCtx(kCUDA);
    ctx.mem()->initOC(kCUDA);
  }

  runCase("model", 1536, 256, true, {{1, 1, 1536}, {2, 3, 1536}, {1, 64, 1536}});
  runCase("vit", 1176, 160, false, {{1, 1176}, {40, 1176}});  // K not a multiple of 32 (Qwen2VL patch embed width)
  runCaseA16("a16", 1536, 256, true, {{1, 1, 1536}, {2, 3, 1536}, {1, 64, 1536}, {2, 80, 1536}});
  runCaseA16("a16vit", 1176, 160, false, {{1, 1176}, {40, 1176}});
  // the linears of the Qwen2VL vision tower (mllm/Models/qwen2vl/modeling_qwen2vl.hpp:129-130,163-164 of the
  // reference): qkv 1280 -> 3840, proj 1280 -> 1280, fc1 1280 -> 5120, fc2 5120 -> 1280; one patch row and a 40-patch image
  runCase("vit_qkv", 1280, 3840, true, {{1, 1280}, {40, 1280}});
  runCase("vit_proj", 1280, 1280, true, {{1, 1280}, {40, 1280}});
  runCase("vit_fc1", 1280, 5120, true, {{1, 1280}, {40, 1280}});
  runCase("vit_fc2", 5120, 1280, true, {{1, 5120}, {40, 5120}});
  // the Qwen2VL patch embedding: Conv3D 3 -> 1280, kernel = stride = {2, 14, 14}; one patch, and a 2 x 3 grid of patches
  runConv3D("patch1", 3, 1280, {2, 14, 14}, {2, 14, 14}, false, {1, 3, 2, 14, 14});
  runConv3D("patch6", 3, 1280, {2, 14, 14}, {2, 14, 14}, true, {1, 3, 2, 28, 42});
  runConv3D("conv_overlap", 2, 96, {2, 3, 3}, {1, 2, 2}, true, {2, 2, 3, 9, 11});  // overlapping windows, batch 2
  runQuantizerFlow();

  std::printf("%s (%d failures)\n", g_failures == 0 ? "BOUNDARY TEST PASSED" : "BOUNDARY TEST FAILED", g_failures);
  std::fflush(stdout);
  // leave without running the engine's static destructors after the CUDA context may be gone
  std::_Exit(g_failures == 0 ? 0 : 1);
}
