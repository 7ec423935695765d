// Device side of the C ABI (include/mllmb200.h): argument checks, kernel selection, launches.
#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/mllmb200.h"
#include "device_common.cuh"

namespace mllmb200 {
// repack.cu
__global__ void repack_cells_kernel(const uint8_t*, const uint16_t*, int, int, int, int, int, uint8_t*);
__global__ void repack_rowdata_kernel(const uint8_t*, const float*, int, int, int, int, uint32_t, float*, float*,
                                      unsigned int*);
__global__ void unpack_cells_kernel(const uint8_t*, int, int, int, int, uint8_t*, uint16_t*);
__global__ void unpack_bias_kernel(const float*, int, float*);
// act_quant.cu
__global__ void act_quant_reflayout_kernel(const float*, int, int, uint8_t*);
cudaError_t launch_act_quant_records(const float*, int, int, int, uint8_t*, float2*, int, int, cudaStream_t);
int w4a32_gemm_tc_m_pad(int m);
// gemv.cu / gemm_simt.cu / gemm_tc.cu
bool w4a32_gemv_supported(int m, int k, int n);
// gemv_stream.cu: the single-launch GEMV (quantizes x itself; up to 8 matrices, each with its own activations)
bool w4a32_gemv_stream_supported(int m, int count, const int* k, const int* n);
cudaError_t launch_w4a32_gemv_stream(int count, const float* const* x, const int* ldx, const uint8_t* const* a_rec,
                                     const float2* const* a_hdr, int m, const int* k, const void* const* tiled,
                                     float* const* y, const int* n, const int* ldy, int use_pdl, cudaStream_t stream,
                                     int num_peers = 0, float* const* y_peers = nullptr);
int w4a32_gemv_stream_plan_check(int, int, const int*, const int*, int*, int*, int*, int*, size_t*);
cudaError_t w4a32_gemv_stream_set_trace(unsigned long long*, int);
cudaError_t launch_w4a32_gemv_grouped(const uint8_t*, const float2*, int, int, int, const void* const*, float* const*,
                                      const int*, const int*, int, cudaStream_t);
cudaError_t launch_w4a32_gemm_simt(const uint8_t*, const float2*, const void*, float*, int, int, int, int, cudaStream_t);
cudaError_t launch_w4a32_gemm_tc(const uint8_t*, const float2*, const void*, float*, int, int, int, int, cudaStream_t);
bool w4a32_gemm_tc_supported(int m, int k, int n);
// gemm_tcf16.cu (+ its activation layout in act_quant.cu)
bool w4a32_gemm_tcf16_supported(int m, int k, int n);
bool w4a32_gemm_tcf16_preferred(int m, int k, int n);
int w4a32_gemm_tcf16_m_pad(int m, int n);
int w4a32_gemm_tcf16_m_pad_max(int m);
cudaError_t launch_w4a32_gemm_tcf16(const uint8_t*, const float2*, const void*, float*, int, int, int, int, cudaStream_t, int use_pdl,
                                    int* split_sync, int split_sync_ints);
cudaError_t launch_act_quant_blocks_f16(const float*, int, int, int, int, uint8_t*, float2*, cudaStream_t, int use_pdl = 0,
                                        int* clear_ints = nullptr, int clear_count = 0);
int w4a32_gemm_tcf16_tile_grouped(int m, int count, const int* n);
cudaError_t launch_w4a32_gemm_tcf16_grouped(const uint8_t*, const float2*, int, int, int, const void* const*, float* const*,
                                            const int*, const int*, cudaStream_t, int num_peers = 0,
                                            float* const* y_peers = nullptr, int use_pdl = 0, int* split_sync = nullptr,
                                            int split_sync_ints = 0);
constexpr int kSplitSyncInts = 1024;  // K-split counters of the fp16 tile GEMM at the end of the workspace (two per output tile)

bool w4a32_gemm_stream_supported(int m, int k, int count, const int* n);
size_t w4a32_gemm_stream_act_bytes(int m, int k);
cudaError_t launch_act_quant_mma(const float*, int, int, int, uint8_t*, float2*, int, cudaStream_t);
cudaError_t launch_w4a32_gemm_stream(const uint8_t*, const float2*, int, int, int, const void* const*, float* const*,
                                     const int*, const int*, int, cudaStream_t);
constexpr int kStreamGemmMinM = 5, kStreamGemmMaxM = 64;  // batch sizes the streaming tensor-core GEMM takes by default

static thread_local int t_last_cuda_error = 0;
static int cuda_fail(cudaError_t e) {
  t_last_cuda_error = (int)e;
  return MLLMB200_CUDA_ERROR;
}
int record_cuda_failure(cudaError_t e) { return cuda_fail(e); }  // for the other C-ABI translation units
// workspace = [quantized activations][row headers: M * 8 bytes], each 256-aligned.  The first part
// holds either 48-byte records (GEMV, SIMT GEMM) or 256-byte operand blocks over rows padded to
// the tcgen05 tile (tcgen05 GEMM); it is sized for the larger of the two.
static inline size_t ws_rec_bytes(int m, int k) {
  const size_t rec = (size_t)m * blob_num_blocks(k) * kActRecordBytes;
  // operand blocks are only written when the tcgen05 path can be chosen for this M
  const size_t blk = w4a32_gemm_tc_supported(m, k, 1) ? (size_t)w4a32_gemm_tc_m_pad(m) * blob_num_blocks(k) * 32 : 0;
  // fp16 operand blocks of the fp16 tensor-core path (64 bytes per row and K-group, rows padded to its widest tile)
  const size_t blk16 = w4a32_gemm_tcf16_supported(m, k, 1) ? (size_t)w4a32_gemm_tcf16_m_pad_max(m) * blob_num_blocks(k) * 64 : 0;
  // activation blocks of the streaming small-batch GEMM (36 bytes per row and K-group, rows padded to 8)
  const size_t mma = m <= kStreamGemmMaxM ? w4a32_gemm_stream_act_bytes(m, k) : 0;
  size_t big = rec > blk ? rec : blk;
  big = big > mma ? big : mma;
  return align_up(big > blk16 ? big : blk16, 256);
}
size_t w4a32_ws_rec_bytes(int m, int k) { return ws_rec_bytes(m, k); }  // for tp.cu
// the K-split counters of the fp16 tile GEMM: behind the row headers of a workspace of workspace_size(m, k) bytes
int* w4a32_ws_split_sync(void* ws_dev, int m, int k) {
  return reinterpret_cast<int*>(static_cast<uint8_t*>(ws_dev) + ws_rec_bytes(m, k) + align_up((size_t)m * sizeof(float2), 256));
}
int w4a32_ws_split_sync_ints() { return kSplitSyncInts; }
}  // namespace mllmb200

using namespace mllmb200;

// Self-test of the bounded waits: one CTA arms an mbarrier for 16 bytes that nobody ever copies and waits for
// them with the given tick limit.  The wait gives up, raises the timeout bit of the status word and the kernel
// returns normally - nothing faults, nothing spins without bound.
__global__ void selftest_wait_timeout_kernel(long long limit_ticks, int* gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    mbar_arrive_expect_tx(&bar, 16);  // the phase now needs 16 bytes that are never sent
    const bool landed = mbar_wait_bounded(&bar, 0, limit_ticks);
    if (gave_up) *gave_up = landed ? 0 : 1;
  }
}

extern "C" {

int mllmb200_last_cuda_error(void) { return t_last_cuda_error; }

int mllmb200_w4a32_tiled_size(int N_rows, int K, size_t* bytes) {
  if (!bytes || N_rows <= 0 || K <= 0) return MLLMB200_INVALID_ARG;
  *bytes = make_tiled_header(N_rows, K, 0, 0).total_bytes;
  return MLLMB200_OK;
}

int mllmb200_w4a32_repack_device(const void* blob_dev, int N, int K, int scale_mode, int has_bias, int row_begin,
                                 int row_count, void* tiled_dev, void* stream) {
  if (!blob_dev || !tiled_dev || N <= 0 || K <= 0 || row_count <= 0 || row_begin < 0 || row_begin + row_count > N)
    return MLLMB200_INVALID_ARG;
  if (scale_mode < 0 || scale_mode > 2) return MLLMB200_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(blob_dev) & 15u) || (reinterpret_cast<uintptr_t>(tiled_dev) & 15u))
    return MLLMB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const BlobHeader bh = make_blob_header(N, K, scale_mode, has_bias);
  const TiledHeader th = make_tiled_header(row_count, K, scale_mode, has_bias);
  const uint8_t* blob = static_cast<const uint8_t*>(blob_dev);
  uint8_t* tiled = static_cast<uint8_t*>(tiled_dev);
  cudaError_t e = cudaMemcpyAsync(tiled, &th, sizeof(th), cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) return cuda_fail(e);
  const long long items = (long long)th.num_panels * th.num_groups * kPanelRows;
  const int blocks = (int)std::min<long long>((items + 255) / 256, 148 * 16);
  repack_cells_kernel<<<blocks, 256, 0, st>>>(blob + bh.nibbles_off,
                                              reinterpret_cast<const uint16_t*>(blob + bh.scales_off), K, row_begin,
                                              row_count, (int)th.num_groups, (int)th.num_panels, tiled + th.cells_off);
  if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail(e);
  const int rows_pad = (int)th.num_panels * kPanelRows;
  const int blocks2 = std::min((rows_pad + 7) / 8, 148 * 8);
  repack_rowdata_kernel<<<blocks2, 256, 0, st>>>(
      tiled + th.cells_off, has_bias ? reinterpret_cast<const float*>(blob + bh.bias_off) : nullptr, row_begin,
      row_count, (int)th.num_groups, (int)th.num_panels, (uint32_t)scale_mode,
      reinterpret_cast<float*>(tiled + th.zsum_off), reinterpret_cast<float*>(tiled + th.bias_off),
      reinterpret_cast<unsigned int*>(tiled + offsetof(TiledHeader, max_scale_bits)));
  if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail(e);
  return MLLMB200_OK;
}

int mllmb200_w4a32_unpack_device(const void* tiled_dev, int row_count, int K, void* out_blob_dev, void* stream) {
  if (!tiled_dev || !out_blob_dev || row_count <= 0 || K <= 0) return MLLMB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the header is small: read it back to learn scale_mode / has_bias (synchronizes the stream)
  TiledHeader th;
  cudaError_t e = cudaMemcpyAsync(&th, tiled_dev, sizeof(th), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return cuda_fail(e);
  if ((e = cudaStreamSynchronize(st)) != cudaSuccess) return cuda_fail(e);
  if (th.magic != kTiledMagic || th.n != (uint32_t)row_count || th.k != (uint32_t)K) return MLLMB200_BAD_BLOB;
  const BlobHeader bh = make_blob_header(row_count, K, (int)th.scale_mode, (int)th.has_bias);
  uint8_t* out = static_cast<uint8_t*>(out_blob_dev);
  const uint8_t* tiled = static_cast<const uint8_t*>(tiled_dev);
  if ((e = cudaMemsetAsync(out, 0, bh.total_bytes, st)) != cudaSuccess) return cuda_fail(e);
  if ((e = cudaMemcpyAsync(out, &bh, sizeof(bh), cudaMemcpyHostToDevice, st)) != cudaSuccess) return cuda_fail(e);
  const long long items = (long long)th.num_panels * th.num_groups * kPanelRows;
  const int blocks = (int)std::min<long long>((items + 255) / 256, 148 * 16);
  unpack_cells_kernel<<<blocks, 256, 0, st>>>(tiled + th.cells_off, K, row_count, (int)th.num_groups,
                                              (int)th.num_panels, out + bh.nibbles_off,
                                              reinterpret_cast<uint16_t*>(out + bh.scales_off));
  if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail(e);
  if (th.has_bias) {
    unpack_bias_kernel<<<std::min((row_count + 255) / 256, 1024), 256, 0, st>>>(
        reinterpret_cast<const float*>(tiled + th.bias_off), row_count, reinterpret_cast<float*>(out + bh.bias_off));
    if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail(e);
  }
  // the header copy above read from a stack variable: wait before it goes out of scope
  if ((e = cudaStreamSynchronize(st)) != cudaSuccess) return cuda_fail(e);
  return MLLMB200_OK;
}

int mllmb200_w4a32_workspace_size(int M, int K, size_t* bytes) {
  if (!bytes || M <= 0 || K <= 0) return MLLMB200_INVALID_ARG;
  *bytes = ws_rec_bytes(M, K) + align_up((size_t)M * sizeof(float2), 256);
  if (w4a32_gemm_tcf16_supported(M, K, 1)) *bytes += kSplitSyncInts * sizeof(int);
  return MLLMB200_OK;
}

int mllmb200_w4a32_quant_activations(const float* x_dev, int M, int K, int ldx, void* out_dev, void* stream) {
  if (!x_dev || !out_dev || M <= 0 || K <= 0 || ldx < K) return MLLMB200_INVALID_ARG;
  act_quant_reflayout_kernel<<<M, 256, 0, static_cast<cudaStream_t>(stream)>>>(x_dev, K, ldx,
                                                                              static_cast<uint8_t*>(out_dev));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
}

int mllmb200_w4a32_select_kernel(int M, int K, int N) {
  if (M > 0 && K > 0 && N > 0 && w4a32_gemv_stream_supported(M, 1, &K, &N)) return 1;
  if (M >= kStreamGemmMinM && M <= kStreamGemmMaxM && K > 0 && N > 0 && w4a32_gemm_stream_supported(M, K, 1, &N)) return 7;
  if (w4a32_gemm_tc_supported(M, K, N)) return 3;
  return 2;
}

// Shared front half of every forward: validate, quantize the activations into the workspace.
static int quantize_into_ws(const float* x_dev, void* ws_dev, int M, int K, int ldx, int use_pdl, cudaStream_t st,
                            uint8_t** a_rec, float2** a_hdr, bool tc_blocks = false) {
  if (!ws_dev || (reinterpret_cast<uintptr_t>(ws_dev) & 255u)) return MLLMB200_INVALID_ARG;
  *a_rec = static_cast<uint8_t*>(ws_dev);
  *a_hdr = reinterpret_cast<float2*>(static_cast<uint8_t*>(ws_dev) + ws_rec_bytes(M, K));
  const cudaError_t e =
      launch_act_quant_records(x_dev, M, K, ldx, *a_rec, *a_hdr, use_pdl, tc_blocks ? w4a32_gemm_tc_m_pad(M) / 8 : 0, st);
  return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
}

int mllmb200_w4a32_linear_forward_ex(const float* x_dev, const void* tiled_dev, float* y_dev, void* ws_dev, int M,
                                     int K, int N, int ldx, int ldy, int kernel, void* stream) {
  if (!x_dev || !tiled_dev || !y_dev || M <= 0 || K <= 0 || N <= 0 || ldx < K || ldy < N) return MLLMB200_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(tiled_dev) & 15u) || (reinterpret_cast<uintptr_t>(x_dev) & 3u) ||
      (reinterpret_cast<uintptr_t>(y_dev) & 3u))
    return MLLMB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int use_pdl = (kernel >> 8) & 1;
  kernel &= 0xFF;
  if (kernel < 0 || kernel > 7) return MLLMB200_INVALID_ARG;
  if (kernel == 5) kernel = w4a32_gemm_tcf16_preferred(M, K, N) ? 4 : 0;  // "fastest": fp16 path where it wins
  if (kernel == 0) kernel = mllmb200_w4a32_select_kernel(M, K, N);
  if (kernel == 1) {  // single launch: x is quantized inside the GEMV, no workspace
    if (!w4a32_gemv_stream_supported(M, 1, &K, &N)) return MLLMB200_UNSUPPORTED;
    const cudaError_t e1 =
        launch_w4a32_gemv_stream(1, &x_dev, &ldx, nullptr, nullptr, M, &K, &tiled_dev, &y_dev, &N, &ldy, use_pdl, st);
    return e1 == cudaSuccess ? MLLMB200_OK : cuda_fail(e1);
  }
  if (kernel == 7) {  // streaming tensor-core GEMM for small batches: its own activation layout
    if (!w4a32_gemm_stream_supported(M, K, 1, &N)) return MLLMB200_UNSUPPORTED;
    if (!ws_dev || (reinterpret_cast<uintptr_t>(ws_dev) & 255u)) return MLLMB200_INVALID_ARG;
    uint8_t* acts = static_cast<uint8_t*>(ws_dev);
    float2* hdr7 = reinterpret_cast<float2*>(acts + ws_rec_bytes(M, K));
    cudaError_t e7 = launch_act_quant_mma(x_dev, M, K, ldx, acts, hdr7, use_pdl, st);
    if (e7 == cudaSuccess) e7 = launch_w4a32_gemm_stream(acts, hdr7, M, K, 1, &tiled_dev, &y_dev, &N, &ldy, use_pdl, st);
    return e7 == cudaSuccess ? MLLMB200_OK : cuda_fail(e7);
  }
  if (kernel == 6 && !w4a32_gemv_supported(M, K, N)) return MLLMB200_UNSUPPORTED;
  if (kernel == 3 && !w4a32_gemm_tc_supported(M, K, N)) return MLLMB200_UNSUPPORTED;
  if (kernel == 4) {  // fp16 tensor-core path: its own activation layout
    if (!w4a32_gemm_tcf16_supported(M, K, N)) return MLLMB200_UNSUPPORTED;
    if (!ws_dev || (reinterpret_cast<uintptr_t>(ws_dev) & 255u)) return MLLMB200_INVALID_ARG;
    uint8_t* blocks = static_cast<uint8_t*>(ws_dev);
    float2* hdr16 = reinterpret_cast<float2*>(blocks + ws_rec_bytes(M, K));
    int* sync16 = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(hdr16) + align_up((size_t)M * sizeof(float2), 256));
    cudaError_t e16 = launch_act_quant_blocks_f16(x_dev, M, w4a32_gemm_tcf16_m_pad(M, N), K, ldx, blocks, hdr16, st, use_pdl,
                                                  sync16, kSplitSyncInts);
    if (e16 == cudaSuccess)
      e16 = launch_w4a32_gemm_tcf16(blocks, hdr16, tiled_dev, y_dev, M, K, N, ldy, st, use_pdl, sync16, kSplitSyncInts);
    return e16 == cudaSuccess ? MLLMB200_OK : cuda_fail(e16);
  }
  uint8_t* a_rec;
  float2* a_hdr;
  if (int s = quantize_into_ws(x_dev, ws_dev, M, K, ldx, use_pdl & 1, st, &a_rec, &a_hdr, kernel == 3)) return s;
  cudaError_t e;
  if (kernel == 6) e = launch_w4a32_gemv_grouped(a_rec, a_hdr, M, K, 1, &tiled_dev, &y_dev, &N, &ldy, use_pdl, st);
  else if (kernel == 3) e = launch_w4a32_gemm_tc(a_rec, a_hdr, tiled_dev, y_dev, M, K, N, ldy, st);
  else e = launch_w4a32_gemm_simt(a_rec, a_hdr, tiled_dev, y_dev, M, K, N, ldy, st);
  return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
}

int mllmb200_w4a32_linear_forward(const float* x_dev, const void* tiled_dev, float* y_dev, void* ws_dev, int M, int K,
                                  int N, int ldx, int ldy, void* stream) {
  return mllmb200_w4a32_linear_forward_ex(x_dev, tiled_dev, y_dev, ws_dev, M, K, N, ldx, ldy, 0, stream);
}

int mllmb200_w4a32_linear_forward_grouped(const float* x_dev, int M, int K, int ldx, int count,
                                          const void* const* tiled_dev, float* const* y_dev, const int* N,
                                          const int* ldy, void* ws_dev, int flags, void* stream) {
  if (!x_dev || !tiled_dev || !y_dev || !N || !ldy || count < 1 || count > 4 || M <= 0 || K <= 0 || ldx < K)
    return MLLMB200_INVALID_ARG;
  const float* xs[4];
  int ldxs[4], ks[4];
  for (int i = 0; i < count; ++i) {
    if (!tiled_dev[i] || !y_dev[i] || N[i] <= 0 || ldy[i] < N[i]) return MLLMB200_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(tiled_dev[i]) & 15u) || (reinterpret_cast<uintptr_t>(y_dev[i]) & 3u))
      return MLLMB200_INVALID_ARG;
    xs[i] = x_dev;
    ldxs[i] = ldx;
    ks[i] = K;
  }
  if ((flags & 0xFF) != 6 && w4a32_gemv_stream_supported(M, count, ks, N)) {
    const cudaError_t e = launch_w4a32_gemv_stream(count, xs, ldxs, nullptr, nullptr, M, ks, tiled_dev, y_dev, N, ldy,
                                                   (flags >> 8) & 1, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
  }
  int n_group = 0;
  for (int i = 0; i < count; ++i) n_group += N[i];
  // ("fastest" at 64 <= M: wide groups with a short K go to the fp16 tile GEMM further down)
  const bool tile16_first = (flags & 0xFF) == 5 && count > 1 && w4a32_gemm_tcf16_preferred(M, K, n_group);
  if (((flags & 0xFF) == 0 || (flags & 0xFF) == 5) && !tile16_first && M >= kStreamGemmMinM && M <= kStreamGemmMaxM &&
      w4a32_gemm_stream_supported(M, K, count, N)) {  // small batch: one quantization, ONE streaming tensor-core launch
    if (!ws_dev || (reinterpret_cast<uintptr_t>(ws_dev) & 255u)) return MLLMB200_INVALID_ARG;
    cudaStream_t st7 = static_cast<cudaStream_t>(stream);
    uint8_t* acts = static_cast<uint8_t*>(ws_dev);
    float2* hdr7 = reinterpret_cast<float2*>(acts + ws_rec_bytes(M, K));
    const int pdl7 = (flags >> 8) & 1;
    cudaError_t e7 = launch_act_quant_mma(x_dev, M, K, ldx, acts, hdr7, pdl7, st7);
    if (e7 == cudaSuccess) e7 = launch_w4a32_gemm_stream(acts, hdr7, M, K, count, tiled_dev, y_dev, N, ldy, pdl7, st7);
    return e7 == cudaSuccess ? MLLMB200_OK : cuda_fail(e7);
  }
  bool gemv = (flags & 0xFF) == 6;  // the two-launch path (quantization kernel + one-shot GEMV), kept for comparison
  for (int i = 0; i < count && gemv; ++i) gemv = w4a32_gemv_supported(M, K, N[i]);
  if ((flags & 0xFF) == 6 && !gemv) return MLLMB200_UNSUPPORTED;
  if (gemv) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* a_rec;
    float2* a_hdr;
    if (int s = quantize_into_ws(x_dev, ws_dev, M, K, ldx, (flags >> 8) & 1, st, &a_rec, &a_hdr)) return s;
    cudaError_t e = launch_w4a32_gemv_grouped(a_rec, a_hdr, M, K, count, tiled_dev, y_dev, N, ldy, (flags >> 8) & 1, st);
    return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
  }
  // Larger M: the matrices share ONE quantization of x.  With the "fastest" policy (5) and M >= 128 they
  // also share ONE launch of the fp16 tensor-core kernel (their tiles side by side in the grid: q, k, v
  // alone fill 16 + 2 + 2 tiles); with the default policy, or when the fp16 path does not apply, they
  // run as separate int8 tensor-core launches behind one quantization, or as ordinary forwards.
  const int policy = flags & 0xFF;  // 0 auto, 5 fastest (as the kernel argument of linear_forward_ex)
  if (policy != 0 && policy != 5) return MLLMB200_INVALID_ARG;
  cudaStream_t st_grp = static_cast<cudaStream_t>(stream);
  if (count > 1 && policy == 5 && M >= 64) {
    bool all16 = true;
    int n_sum = 0;
    for (int i = 0; i < count; ++i) {
      all16 = all16 && w4a32_gemm_tcf16_supported(M, K, N[i]);
      n_sum += N[i];
    }
    all16 = all16 && w4a32_gemm_tcf16_preferred(M, K, n_sum);  // (the group's weight tiles ride in one grid)
    if (all16) {
      if (!ws_dev || (reinterpret_cast<uintptr_t>(ws_dev) & 255u)) return MLLMB200_INVALID_ARG;
      uint8_t* blocks = static_cast<uint8_t*>(ws_dev);
      float2* hdr = reinterpret_cast<float2*>(blocks + ws_rec_bytes(M, K));
      const int nt = w4a32_gemm_tcf16_tile_grouped(M, count, N);
      const int pdl = (flags >> 8) & 1;
      int* sync = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(hdr) + align_up((size_t)M * sizeof(float2), 256));
      cudaError_t e = launch_act_quant_blocks_f16(x_dev, M, (M + nt - 1) / nt * nt, K, ldx, blocks, hdr, st_grp, pdl, sync, kSplitSyncInts);
      if (e == cudaSuccess)
        e = launch_w4a32_gemm_tcf16_grouped(blocks, hdr, M, K, count, tiled_dev, y_dev, N, ldy, st_grp, 0, nullptr, pdl, sync,
                                            kSplitSyncInts);
      return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
    }
  }
  bool all8 = count > 1;
  for (int i = 0; i < count; ++i) all8 = all8 && mllmb200_w4a32_select_kernel(M, K, N[i]) == 3;
  if (all8) {
    if (!ws_dev || (reinterpret_cast<uintptr_t>(ws_dev) & 255u)) return MLLMB200_INVALID_ARG;
    uint8_t* blocks = static_cast<uint8_t*>(ws_dev);
    float2* hdr = reinterpret_cast<float2*>(blocks + ws_rec_bytes(M, K));
    cudaError_t e = launch_act_quant_records(x_dev, M, K, ldx, blocks, hdr, 0, w4a32_gemm_tc_m_pad(M) / 8, st_grp);
    for (int i = 0; i < count && e == cudaSuccess; ++i)
      e = launch_w4a32_gemm_tc(blocks, hdr, tiled_dev[i], y_dev[i], M, K, N[i], ldy[i], st_grp);
    return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
  }
  for (int i = 0; i < count; ++i) {
    const int st = mllmb200_w4a32_linear_forward_ex(x_dev, tiled_dev[i], y_dev[i], ws_dev, M, K, N[i], ldx, ldy[i],
                                                    (flags & 0x100) | policy, stream);
    if (st != MLLMB200_OK) return st;
  }
  return MLLMB200_OK;
}

int mllmb200_w4a32_linear_forward_multi(int count, const float* const* x_dev, const int* ldx, const int* K,
                                        const void* const* tiled_dev, float* const* y_dev, const int* N, const int* ldy,
                                        int M, int flags, void* stream) {
  if (!x_dev || !ldx || !K || !tiled_dev || !y_dev || !N || !ldy || count < 1 || M <= 0) return MLLMB200_INVALID_ARG;
  if (count > 8 || M > 4) return MLLMB200_UNSUPPORTED;
  for (int i = 0; i < count; ++i) {
    if (!x_dev[i] || !tiled_dev[i] || !y_dev[i] || K[i] <= 0 || N[i] <= 0 || ldx[i] < K[i] || ldy[i] < N[i])
      return MLLMB200_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(tiled_dev[i]) & 15u) || (reinterpret_cast<uintptr_t>(x_dev[i]) & 3u) ||
        (reinterpret_cast<uintptr_t>(y_dev[i]) & 3u))
      return MLLMB200_INVALID_ARG;
  }
  if (!w4a32_gemv_stream_supported(M, count, K, N)) return MLLMB200_UNSUPPORTED;
  const cudaError_t e = launch_w4a32_gemv_stream(count, x_dev, ldx, nullptr, nullptr, M, K, tiled_dev, y_dev, N, ldy,
                                                 (flags >> 8) & 1, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
}

int mllmb200_w4a32_gemv_plan_check(int M, int count, const int* K, const int* N, int* clusters, int* cluster_size,
                                   int* cells_per_stage, int* stages, size_t* smem_bytes) {
  if (!N || !K || count < 1 || count > 8 || M <= 0) return MLLMB200_INVALID_ARG;
  for (int i = 0; i < count; ++i)
    if (N[i] <= 0 || K[i] <= 0) return MLLMB200_INVALID_ARG;
  const int r = w4a32_gemv_stream_plan_check(M, count, K, N, clusters, cluster_size, cells_per_stage, stages, smem_bytes);
  if (r < 0) return MLLMB200_UNSUPPORTED;
  return r == 0 ? MLLMB200_OK : 100 + r;
}

int mllmb200_w4a32_gemv_trace(void* dev_buf, int capacity_launches) {
  if (dev_buf && (capacity_launches <= 0 || (reinterpret_cast<uintptr_t>(dev_buf) & 7u))) return MLLMB200_INVALID_ARG;
  const cudaError_t e = w4a32_gemv_stream_set_trace(static_cast<unsigned long long*>(dev_buf), dev_buf ? capacity_launches : 0);
  return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
}

int mllmb200_selftest_wait_timeout(long long limit_ticks, int* gave_up_dev, void* stream) {
  if (limit_ticks < 1 || limit_ticks > (1ll << 31)) return MLLMB200_INVALID_ARG;
  selftest_wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ticks, gave_up_dev);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MLLMB200_OK : cuda_fail(e);
}

int mllmb200_check_device_status(void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(e);
  unsigned int word = 0;
  if ((e = cudaMemcpyFromSymbol(&word, g_device_status, sizeof(word))) != cudaSuccess) return cuda_fail(e);
  if (word != 0) {
    const unsigned int zero = 0;
    if ((e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero))) != cudaSuccess) return cuda_fail(e);
  }
  if (word & kDevStatusTimeout) return MLLMB200_TIMEOUT;
  if (word & kDevStatusBadHeader) return MLLMB200_BAD_BLOB;
  return MLLMB200_OK;
}

}  // extern "C"
