/*
 * mllmb200.h - C ABI of the B200 (sm_100a) W4A32 quantized-linear library.
 *
 * This is the whole boundary between host code (the mllm CUDA backend in
 * mllm-advanced_b200/backend/, or any FFI binding) and the CUDA kernels: plain pointers and
 * sizes, no C++ or framework types.  Every function returns an mllmb200_status (0 = ok) unless
 * stated otherwise and never calls exit().  Pointers named *_dev are device pointers on the
 * current CUDA device; all others are host pointers.  `stream` is a cudaStream_t passed as
 * void* (NULL = the legacy default stream).  Device work is enqueued asynchronously on
 * `stream`; nothing here synchronizes unless its comment says so.
 *
 * Each entry point names the interface of the reference project (mllm-advanced, paths relative
 * to its root) that it stands in for.
 */
#ifndef MLLMB200_H_
#define MLLMB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define MLLMB200_API
#else
#define MLLMB200_API __attribute__((visibility("default")))
#endif

typedef enum mllmb200_status {
  MLLMB200_OK = 0,
  MLLMB200_INVALID_ARG = 1,   /* null pointer, non-positive size, bad stride, misaligned pointer */
  MLLMB200_UNSUPPORTED = 2,   /* a shape or mode this build has no kernel for */
  MLLMB200_CUDA_ERROR = 3,    /* a CUDA runtime call failed; see mllmb200_last_cuda_error() */
  MLLMB200_TIMEOUT = 4,       /* a bounded device-side wait ran out (reported by mllmb200_check_device_status) */
  MLLMB200_BAD_BLOB = 5,      /* pre-pack blob header does not match (magic, version, sizes) */
  MLLMB200_TOO_LARGE = 6      /* request exceeds a fixed capacity (static scratch entry point) */
} mllmb200_status;

/* How the 2-byte per-group scale is encoded.
 * BF16_TRUNC is what the reference does (tests/Arm/KaiLinearTest.hpp:133-143 without
 * __ARM_FEATURE_BF16; call site mllm/Backends/Arm/Kernels/kai_linear.cpp:258). */
typedef enum mllmb200_scale_mode {
  MLLMB200_SCALE_BF16_TRUNC = 0,
  MLLMB200_SCALE_BF16_RNE = 1,
  MLLMB200_SCALE_FP16 = 2
} mllmb200_scale_mode;

/* Text for a status code.  Replaces the reference's MLLM_ERROR_EXIT messages
 * (mllm/Utils/Log.hpp:59-64): the library reports, the caller decides whether to exit. */
MLLMB200_API const char* mllmb200_status_str(int status);

/* cudaError_t (as int) of the last failed CUDA call made by this library on this thread. */
MLLMB200_API int mllmb200_last_cuda_error(void);

MLLMB200_API int mllmb200_version(void);

/* ------------------------------------------------------------------------------------------
 * Offline side (host): quantize + pre-pack.  Stands in for
 *   KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk::quant_pack_rhs_size     (mllm/Backends/Arm/Kernels/kai_linear.cpp:302-309)
 *   KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk::quant_pack_rhs_offline  (mllm/Backends/Arm/Kernels/kai_linear.cpp:311-348)
 * The blob is what the quantization pass stores as the 1-D int8 weight tensor
 * (mllm/Backends/Arm/Passes/KaiQuantizationPass.cpp:104-187).  Layout:
 *   64-byte header {magic 'MB2W', version, N, K, group=32, scale_mode, has_bias, layout=0, ...}
 *   nibbles  u8  [N][ceil(K/2)]   q+8, even k in the low half-byte        (kai_linear.cpp:276-287)
 *   scales   u16 [N][ceil(K/32)]                                          (kai_linear.cpp:254-258)
 *   bias     f32 [N]              only when has_bias
 * each section starting on a 16-byte boundary.  The nibble and scale sections are bit-identical
 * to what the reference's quant_nxk_qs4c32_f32 (kai_linear.cpp:220-291) produces.
 * ------------------------------------------------------------------------------------------ */
MLLMB200_API int mllmb200_w4a32_prepack_size(int N, int K, int has_bias, size_t* bytes);

/* W: fp32 [N,K] row-major; bias: fp32 [N] or NULL; blob: prepack_size bytes (host). */
MLLMB200_API int mllmb200_w4a32_quant_prepack(const float* W, const float* bias, int N, int K,
                                              int scale_mode, void* blob);

/* Same blob from already-quantized data (nibbles [N][ceil(K/2)], scales [N][ceil(K/32)]),
 * for checkpoints that ship int4 + scales. */
MLLMB200_API int mllmb200_w4a32_prepack_from_quantized(const uint8_t* nibbles, const uint16_t* scales,
                                                       const float* bias, int N, int K, int scale_mode,
                                                       void* blob);

/* Reads a blob header (host memory). Any out pointer may be NULL. */
MLLMB200_API int mllmb200_w4a32_blob_info(const void* blob, size_t blob_bytes, int* N, int* K,
                                          int* scale_mode, int* has_bias);

/* Byte offsets of the sections inside a blob of the given shape. */
MLLMB200_API int mllmb200_w4a32_blob_offsets(int N, int K, int has_bias, size_t* nibbles_off,
                                             size_t* scales_off, size_t* bias_off);

/* ------------------------------------------------------------------------------------------
 * Load side (device): repack rows [row_begin, row_begin+row_count) of a blob that was copied to
 * device memory into the tile layout the kernels stream.  Stands in for the KleidiAI packing
 * step kai_run_rhs_pack_nxk_qsi4c32p_qsu4c32s1s0 (call site kai_linear.cpp:335-344), which in
 * the reference runs offline on the CPU; here it runs once in LinearOp::load on the GPU.
 * A row range gives a tensor-parallel rank its output-channel shard.
 * blob_dev and tiled_dev must be 16-byte aligned (256 for tiled_dev recommended).
 * ------------------------------------------------------------------------------------------ */
MLLMB200_API int mllmb200_w4a32_tiled_size(int N_rows, int K, size_t* bytes);

MLLMB200_API int mllmb200_w4a32_repack_device(const void* blob_dev, int N, int K, int scale_mode,
                                              int has_bias, int row_begin, int row_count,
                                              void* tiled_dev, void* stream);

/* Inverse of the repack (tile layout -> nibbles/scales/bias sections of a blob of row_count rows),
 * used to prove the repack loses nothing. out_blob_dev must hold prepack_size(row_count,K,has_bias). */
MLLMB200_API int mllmb200_w4a32_unpack_device(const void* tiled_dev, int row_count, int K,
                                              void* out_blob_dev, void* stream);

/* ------------------------------------------------------------------------------------------
 * Forward.  Stands in for
 *   KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk::workspace_size  (kai_linear.cpp:293-300)
 *   KaiLinear_f32_qai8dxp_qsi4c32p_mxk_nxk::matmul          (kai_linear.cpp:350-398)
 * as called by ArmLinearOp::forward (mllm/Backends/Arm/Ops/LinearOp.cpp:32-133).
 *   y[m,n] = lhs_scale[m] * sum_b( (float)( sum_{k in b} (a_q[m,k]+a_off[m]) * (u[n,k]-8) ) * s[n,b] ) + bias[n]
 * with the per-row dynamic int8 activation quantization of kai_run_lhs_quant_pack_qai8dxp_f32
 * (call site kai_linear.cpp:358-362) done on the device inside the call.
 * x_dev: fp32 [M, ldx] (ldx >= K, elements); y_dev: fp32 [M, ldy] (ldy >= N).
 * ws_dev: workspace_size(M,K) bytes, 256-byte aligned; may be NULL when that size is 0.
 * N must equal the row_count the tiled buffer was repacked with.
 * ------------------------------------------------------------------------------------------ */
MLLMB200_API int mllmb200_w4a32_workspace_size(int M, int K, size_t* bytes);

MLLMB200_API int mllmb200_w4a32_linear_forward(const float* x_dev, const void* tiled_dev, float* y_dev,
                                               void* ws_dev, int M, int K, int N, int ldx, int ldy,
                                               void* stream);

/* Same, with the kernel family forced (tests and benchmarks):
 * 0 auto, 1 streaming GEMV (M <= 4: ONE launch, x quantized inside it, ws_dev unused), 2 SIMT dp4a GEMM,
 * 3 tcgen05 kind::i8 GEMM (exact int32 group sums, as the reference), 4 tcgen05 fp16 GEMM (M >= 64: group
 * scales folded into an fp16 weight operand - exact for bf16-encoded scales, rounded to fp16's 11 bits
 * (relative error <= 2^-11 per weight) for MLLMB200_SCALE_FP16 - fp32 accumulation over all of K in
 * tensor memory; same 1e-3*rms bound; auto never picks it; launches that would fill less than half of the SMs
 * split K between two CTAs per output tile, and y holds one half's partial sums for a moment during the
 * call - deterministic, but y is scratch until the call's work on the stream has finished), 5 fastest: kernel 4
 * for M >= 128 and, at 64 <= M < 128, for matrices (or groups) of at least 8192 rows with K <= 4096; else auto,
 * 6 the two-launch GEMV (activation-quantization kernel + one-shot GEMV), kept for comparison,
 * 7 streaming tensor-core GEMM for small batches (M <= 64; what auto picks for 5 <= M <= 64): the weight cells are
 * spread over all SMs as in the GEMV, the per-group integer products run as mma.sync u8 x s8 (exact int32 group
 * sums, as the reference), clusters split K where the quantized activations of a whole row do not fit one CTA.
 * OR 0x100 into `kernel` to allow programmatic dependent launch (kernels 1, 4, 5, 6, 7): the kernel then
 * requests its (constant) weights while the previous kernel of the stream still runs and reads x only
 * after that kernel has completed. */
MLLMB200_API int mllmb200_w4a32_linear_forward_ex(const float* x_dev, const void* tiled_dev, float* y_dev,
                                                  void* ws_dev, int M, int K, int N, int ldx, int ldy,
                                                  int kernel, void* stream);

/* Several linears that read the SAME activations (q/k/v, gate/up of a decoder layer,
 * mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:47-54,106-112 of the reference) in one call: count in
 * [1,4], all with the same K.  For M <= 4 this is a single kernel launch that quantizes x once per
 * CTA and streams all the weight matrices; for larger M the matrices share one quantization of x
 * when they take the same tensor-core path, else it is `count` ordinary forwards.
 * flags: bit 8 = allow programmatic dependent launch; low byte = kernel policy: 0 auto, 5 fastest
 * (as linear_forward_ex's kernel argument), 6 the two-launch GEMV (M <= 4 only). */
MLLMB200_API int mllmb200_w4a32_linear_forward_grouped(const float* x_dev, int M, int K, int ldx, int count,
                                                       const void* const* tiled_dev, float* const* y_dev,
                                                       const int* N, const int* ldy, void* ws_dev, int flags,
                                                       void* stream);

/* Which kernel family `kernel = 0` picks for a shape (1, 2 or 3 as above). */
MLLMB200_API int mllmb200_w4a32_select_kernel(int M, int K, int N);

/* Several INDEPENDENT linears in one launch: count in [1,8] matrices [N[i], K[i]], each with its own
 * activations x_dev[i] [M, ldx[i]] (pointers may repeat) and output y_dev[i] [M, ldy[i]], M <= 4.  The
 * seven linears of one decoder layer at decode (BASELINE config 1) are such a set.  Every matrix gets a
 * share of the grid in proportion to its size; each CTA quantizes the activations of its own matrix.
 * (No counterpart in the reference, which dispatches one op at a time: mllm/Engine/Context.cpp:65-122.)
 * MLLMB200_UNSUPPORTED when M > 4, count > 8 or the set has no GEMV plan: call the linears one by one.
 * flags: bit 8 = allow programmatic dependent launch. */
MLLMB200_API int mllmb200_w4a32_linear_forward_multi(int count, const float* const* x_dev, const int* ldx,
                                                     const int* K, const void* const* tiled_dev,
                                                     float* const* y_dev, const int* N, const int* ldy, int M,
                                                     int flags, void* stream);

/* Host-only (no GPU needed): the streaming GEMV's work decomposition for a call of `count` matrices
 * [N[i], K[i]] with activations [M, K[i]] - clusters, CTAs per cluster, shared-memory ring shape - and
 * a replay of it with the kernel's own integer arithmetic that verifies every weight cell is
 * requested and consumed exactly once, every consumed cell's activation group is quantized by its
 * CTA, and every 32-row panel is finished exactly once.  (The reference has no counterpart:
 * KleidiAI's ukernel takes m/n steps from a table, kai_linear.cpp:123-218.)
 * MLLMB200_OK, MLLMB200_UNSUPPORTED when the call has no GEMV plan, 100 + c when check c fails.
 * Output pointers may be NULL. */
MLLMB200_API int mllmb200_w4a32_gemv_plan_check(int M, int count, const int* K, const int* N, int* clusters,
                                                int* cluster_size, int* cells_per_stage, int* stages,
                                                size_t* smem_bytes);

/* Profiling aid for the streaming GEMV (no counterpart in the reference): while dev_buf is set, the
 * next capacity_launches GEMV launches of this process each record 20 words (8 bytes each) at
 * dev_buf[1 + 20 * launch_index ...]: for thread 0 of the first CTA, then of the last CTA, eight
 * global-timer values (ns) - kernel entry, prologue done (first weight copies requested), previous
 * kernel complete (programmatic dependent launch), activations quantized, main loop done, partial
 * sums visible, cluster peers started, outputs stored - then the clock cycles that thread spent
 * waiting for weights to land, then one unused word.  dev_buf must hold 1 + 20 * capacity_launches
 * words and stay alive.  A launch replayed from a CUDA graph overwrites the slot it was captured
 * with.  dev_buf = NULL switches the trace off.  Calls cudaMemcpyToSymbol: not during stream capture. */
MLLMB200_API int mllmb200_w4a32_gemv_trace(void* dev_buf, int capacity_launches);

/* Activation quantization alone (rows -> int8 + {recip scale, -zero point} headers in the
 * reference's row layout of k + 8 bytes, tests/Arm/KaiLinearTest.hpp:163-230), for parity tests.
 * out_dev: M * (K + 8) bytes. */
MLLMB200_API int mllmb200_w4a32_quant_activations(const float* x_dev, int M, int K, int ldx,
                                                  void* out_dev, void* stream);

/* Forward that allocates nothing.  (No counterpart in the reference project: its linear op
 * allocates a workspace tensor on every call, mllm/Backends/Arm/Ops/LinearOp.cpp:41-43.)
 * For callers that cannot obtain device memory at call time - a host that owns all device memory
 * through its own pool, a fixed-budget serving loop, a step that must not trigger cudaMalloc's
 * device synchronization.  The activation workspace lives in a 1 MiB array inside the library's
 * device image (held by every GPU that loads the library until exit); a call needing more
 * (see mllmb200_w4a32_workspace_size) returns MLLMB200_TOO_LARGE.  All calls on a device share that
 * array: calls that overlap on the GPU race, so keep them on one stream or order them.  The first
 * call on each device resolves the array's address (cudaGetSymbolAddress) - make it before any
 * stream capture.  Same arguments and results as mllmb200_w4a32_linear_forward, minus ws_dev. */
MLLMB200_API int mllmb200_w4a32_linear_forward_static(const float* x_dev, const void* tiled_dev, float* y_dev,
                                                      int M, int K, int N, int ldx, int ldy, void* stream);

/* Capacity of that array in bytes. */
MLLMB200_API int mllmb200_w4a32_static_scratch_bytes(size_t* bytes);

/* ------------------------------------------------------------------------------------------
 * Conv3D as a W4A32 linear (the Qwen2VL patch embedding): im2col, the quantized linear on
 * [B*T'*H'*W', C*kt*kh*kw], permutation to [B, O, T', H', W'] - the flow of
 * mllm/Backends/Arm/Ops/Conv3DOp.cpp:31-170 (no padding, dilation 1; column order c, kt, kh, kw as
 * mllm/Backends/Arm/Kernels/conv3d.cpp:15-79).  in_shape = {B, C, T, H, W}, kernel = {kt, kh, kw},
 * stride = {st, sh, sw}.  plan: the implied linear's M and K and the workspace bytes (outputs may be
 * NULL).  forward: x_dev / y_dev contiguous fp32; tiled_dev = the [out_ch, K] weight (+ bias) in the
 * tile layout (prepack + repack as for any linear); ws_dev 256-byte aligned.
 * ------------------------------------------------------------------------------------------ */
MLLMB200_API int mllmb200_conv3d_w4a32_plan(const int* in_shape, const int* kernel, const int* stride, int out_ch,
                                            int* M, int* K, size_t* workspace_bytes);
MLLMB200_API int mllmb200_conv3d_w4a32_forward(const float* x_dev, const void* tiled_dev, float* y_dev, void* ws_dev,
                                               const int* in_shape, const int* kernel, const int* stride, int out_ch,
                                               void* stream);

/* ------------------------------------------------------------------------------------------
 * W4A16 sibling path.  Stands in for KaiLinear_f16_qsi8d32p_qai4c32p_mxk_nxk
 * (mllm/Backends/Arm/Kernels/kai_linear.cpp:680-951; op dispatch mllm/Backends/Arm/Ops/LinearOp.cpp:135-190,
 * output dtype fp16 per LinearOp.cpp:246-251; impl types 9-11 of mllm/Core/AOps/LinearOp.hpp:28-30):
 * asymmetric int4 weights in groups of 32 along K with an fp32 scale and an fp32 zero term per group,
 * activations (fp32 or fp16) quantized inside the call to symmetric int8 per 32-element block with an
 * fp32 scale, fp16 output clamped to +-65504:
 *   y[m,n] = fp16( sum_b a_s[m,b] * ( s[n,b] * float(sum_{k in b} a_q[m,k] (u[n,k]-8))
 *                                   + z[n,b] * float(sum_{k in b} a_q[m,k]) ) + bias[n] )
 *
 *   prepack_size / quant_prepack (host)  quant_pack_rhs_size / quant_pack_rhs_offline + quant_nxk_qai4c32_f32
 *                                        (kai_linear.cpp:700-851).  Blob: the 64-byte header of the W4A32
 *                                        blob with layout = 1, then nibbles u8 [N][ceil(K/2)] (q+8, EVEN k in
 *                                        the HIGH half-byte, kai_linear.cpp:807-816), scales f32 [N][ceil(K/32)],
 *                                        zeros f32 [N][ceil(K/32)] (= -zero_point*scale, kai_linear.cpp:797-805),
 *                                        bias f32 [N] when present; sections 16-byte aligned, bit-identical to
 *                                        what quant_nxk_qai4c32_f32 produces.
 *   tiled_size / repack_device           the KleidiAI packing step kai_run_rhs_pack_nxk_qai4c32p_qau4c32s0s1_
 *                                        f32_f32_f32_neon (call site kai_linear.cpp:845-847), on the GPU at
 *                                        load time; a row range gives a tensor-parallel shard.
 *   workspace_size / linear_forward      workspace_size + matmul (kai_linear.cpp:680-698, 853-951), both the
 *                                        fp32 and the fp16 activation overloads (x_dtype).
 * x_dev: [M, ldx] of x_dtype; y_dev: fp16 [M, ldy]; ws_dev: workspace_size bytes, 256-byte aligned.
 * ------------------------------------------------------------------------------------------ */
#define MLLMB200_DTYPE_F32 0
#define MLLMB200_DTYPE_F16 1

MLLMB200_API int mllmb200_w4a16_prepack_size(int N, int K, int has_bias, size_t* bytes);
MLLMB200_API int mllmb200_w4a16_quant_prepack(const float* W, const float* bias, int N, int K, void* blob);
MLLMB200_API int mllmb200_w4a16_blob_info(const void* blob, size_t blob_bytes, int* N, int* K, int* has_bias);
MLLMB200_API int mllmb200_w4a16_blob_offsets(int N, int K, int has_bias, size_t* nibbles_off, size_t* scales_off,
                                             size_t* zeros_off, size_t* bias_off);
MLLMB200_API int mllmb200_w4a16_tiled_size(int N_rows, int K, size_t* bytes);
MLLMB200_API int mllmb200_w4a16_repack_device(const void* blob_dev, int N, int K, int has_bias, int row_begin,
                                              int row_count, void* tiled_dev, void* stream);
MLLMB200_API int mllmb200_w4a16_workspace_size(int M, int K, int N, size_t* bytes);
MLLMB200_API int mllmb200_w4a16_linear_forward(const void* x_dev, int x_dtype, const void* tiled_dev, void* y_dev,
                                               void* ws_dev, int M, int K, int N, int ldx, int ldy, void* stream);
/* Same with the kernel family forced: 0 auto (the tensor-core kernel for M >= 128, and for M >= 32 when
 * N >= 8192; else the dp4a kernel), 2 dp4a kernel (exact int32 block sums, fp32 combination as written above), 4 tcgen05 fp16 kernel (M >= 8):
 * weight operand fp16(((u-8)*s + z) * 2^E) and activation operand fp16(a_q * a_s), one rounding each, fp32
 * accumulation over all of K in tensor memory - it differs from the formula above by those roundings
 * (about 3e-4 of the row's rms, the size of the fp16 output's own rounding).
 * Its activation operand is fp16: fp32 activations beyond the fp16 range (|x| > 65504) overflow there - force
 * kernel 2 for such inputs (fp16 activations cannot exceed it).
 * OR 0x100 into `kernel` to launch the single-launch kernel (M <= 4) with programmatic dependent launch: it
 * then fetches its first weights while the previous kernel of the stream drains, and reads x only after
 * that kernel has completed.  Use it only when x and y are not written by anything else on the stream that
 * could still be running (the usual chain of linears on one stream is fine). */
MLLMB200_API int mllmb200_w4a16_linear_forward_ex(const void* x_dev, int x_dtype, const void* tiled_dev, void* y_dev,
                                                  void* ws_dev, int M, int K, int N, int ldx, int ldy, int kernel,
                                                  void* stream);
/* Several W4A16 linears that read the SAME activations (q/k/v, gate/up of a decoder layer,
 * mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:47-54,106-112) in one call: count in [1,4], all with the same K.
 * For M <= 4 on small matrices this is ONE kernel launch (their row panels side by side in the grid); where the
 * tensor-core kernel applies (M >= 128, or M >= 32 with sum(N) >= 8192) one quantization and ONE launch; otherwise
 * one forward per matrix.  ws_dev must hold the largest workspace_size(M, K, N[i]).  flags: 0 or 0x100 (programmatic
 * dependent launch, as above). */
MLLMB200_API int mllmb200_w4a16_linear_forward_grouped(const void* x_dev, int x_dtype, int M, int K, int ldx, int count,
                                                       const void* const* tiled_dev, void* const* y_dev, const int* N,
                                                       const int* ldy, void* ws_dev, int flags, void* stream);

/* ------------------------------------------------------------------------------------------
 * Decoder: the Qwen2-architecture language model whose linears are the W4A32 op above
 * (reference project: mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:47-54,106-155,175-215, greedy loop
 * mllm/Models/AutoLLM.hpp:39-105).  Batch 1 (the batched form follows below), fp32 activations and KV cache,
 * fp16 lm_head, greedy sampling on the device.  A decode step is one CUDA graph replay; the position and the current
 * token live in device memory.  All calls are asynchronous on the decoder's own stream except
 * set_* (which synchronize it) and read.
 * ------------------------------------------------------------------------------------------ */
typedef struct mllmb200_qwen2_config {
  int layers, hidden, q_heads, kv_heads, head_dim, inter, vocab, max_ctx;
  float eps, rope_theta;
} mllmb200_qwen2_config;

MLLMB200_API int mllmb200_qwen2_create(const mllmb200_qwen2_config* cfg, void** handle);
MLLMB200_API void mllmb200_qwen2_destroy(void* handle);
/* which: 0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down; blob_dev: pre-pack blob in device memory
 * (repacked into the decoder's own tiled buffer; the blob may be freed afterwards). */
MLLMB200_API int mllmb200_qwen2_set_linear(void* handle, int layer, int which, const void* blob_dev, int N, int K,
                                           int scale_mode, int has_bias);
/* Same, adopting a buffer already in the tile layout (repack_device output for the whole [N, K]
 * matrix of that projection); borrowed - keep it alive.  The shape is taken from the config. */
MLLMB200_API int mllmb200_qwen2_set_linear_tiled(void* handle, int layer, int which, const void* tiled_dev);
/* kind: 0 input norm, 1 post-attention norm (of `layer`), 2 final norm; src_dev fp32 [hidden], copied. */
MLLMB200_API int mllmb200_qwen2_set_norm(void* handle, int kind, int layer, const float* src_dev);
/* Borrowed: embedding fp32 [vocab, hidden], lm_head fp16 [vocab, hidden]; keep them alive. */
MLLMB200_API int mllmb200_qwen2_set_tables(void* handle, const float* embedding_dev, const void* lm_head_f16_dev);
/* Prompt of n tokens (int32 on the device) from an empty cache; samples the next token. */
MLLMB200_API int mllmb200_qwen2_prefill(void* handle, const int* tokens_dev, int n);
/* `steps` greedy decode steps, each feeding the previously sampled token (needs a prefill first;
 * position + steps must fit max_ctx).  mode 0 (default) or 1 = one CUDA graph replay per step (one
 * launch per operator), 2 = the persistent kernel: all steps in one cooperative launch of one CTA
 * per SM that streams each CTA's share of the weights through a shared-memory ring
 * (MLLMB200_UNSUPPORTED when the device or the shape does not allow it).  decode == decode_ex(.., 0). */
MLLMB200_API int mllmb200_qwen2_decode(void* handle, int steps);
MLLMB200_API int mllmb200_qwen2_decode_ex(void* handle, int steps, int mode);
/* Host-only: builds the persistent kernel's static work plan for this shape and CTA count and
 * verifies that every weight cell is streamed exactly once (no GPU needed).  Outputs may be NULL. */
MLLMB200_API int mllmb200_qwen2_plan_check(const mllmb200_qwen2_config* cfg, int nctas, int* max_chunks,
                                           int* max_slots, int* total_chunks);
/* Synchronizes; copies to HOST memory history[first, first+count) (entry p = the token sampled after
 * position p), the number of tokens in the cache, and the last logits [vocab]; NULLs are skipped. */
MLLMB200_API int mllmb200_qwen2_read(void* handle, int first, int count, int* tokens_out, int* pos_out,
                                     float* logits_out);
/* Per-phase cycle counters of the persistent kernel on/off (off by default; they cost a few percent). */
MLLMB200_API int mllmb200_qwen2_set_profiling(void* handle, int on);
/* Profiling of the persistent kernel: clock cycles that thread 0 of every CTA spent in each phase
 * (work and barrier waits separately) during the last launch, out[nctas][stamps]; out may be NULL
 * to query the two sizes.  Synchronizes the stream. */
MLLMB200_API int mllmb200_qwen2_phase_cycles(void* handle, long long* out, int capacity, int* nctas, int* stamps);
/* The decoder's CUDA stream (cudaStream_t), for event timing. */
MLLMB200_API void* mllmb200_qwen2_stream(void* handle);

/* Batched greedy decode: `batch` sequences, each with its own fp32 KV cache and position, advance one token per
 * step together, so every quantized linear of a step runs at M = batch.  No counterpart in the reference, whose
 * KV cache asserts a batch of one (mllm/Backends/Arm/Ops/KVCacheOp.cpp:107,156): the contract is that sequence b
 * yields the tokens the batch-1 decoder yields on sequence b alone (its forward: modeling_ds_qwen2.hpp:106-155,
 * cache append KVCacheOp.cpp:15-72, greedy loop AutoLLM.hpp:39-105).  The batch object borrows weights, norms,
 * tables, context length and stream of `decoder` (a handle of mllmb200_qwen2_create with everything set; keep it
 * alive, and do not run it while batch calls are in flight: prefill shares its activation buffers).
 * Device memory: 2 * layers * batch * kv_heads * max_ctx * head_dim * 4 bytes of cache plus activations. */
MLLMB200_API int mllmb200_qwen2_batch_create(void* decoder, int batch, void** handle);
MLLMB200_API void mllmb200_qwen2_batch_destroy(void* handle);
/* Kernel policy of the M = batch linears: 0 (default) exact int32 group sums, 4 / 5 as in linear_forward_ex. */
MLLMB200_API int mllmb200_qwen2_batch_set_policy(void* handle, int policy);
/* Prefills sequence `seq` from an empty cache and samples its first token.  Exactly one of tokens_dev (int32 [n])
 * and embeds_dev (fp32 [n, hidden]: rows that already are embeddings, e.g. vision-patch embeddings mixed with
 * looked-up text tokens) is non-NULL.  Prompts of different sequences may differ in length. */
MLLMB200_API int mllmb200_qwen2_batch_prefill(void* handle, int seq, const int* tokens_dev, const float* embeds_dev, int n);
/* `steps` greedy steps for all sequences together: one CUDA graph replay per step.  Every sequence needs a
 * prefill first and position + steps <= max_ctx. */
MLLMB200_API int mllmb200_qwen2_batch_decode(void* handle, int steps);
/* As mllmb200_qwen2_read, for sequence `seq`. */
MLLMB200_API int mllmb200_qwen2_batch_read(void* handle, int seq, int first, int count, int* tokens_out, int* pos_out,
                                           float* logits_out);

/* ------------------------------------------------------------------------------------------
 * Tensor parallelism over the GPUs of one node, one process per GPU (no counterpart in the reference, whose
 * engine is single-device: mllm/Engine/Context.cpp:56-59).  Output channels are sharded: rank r holds rows
 * [r N/g, (r+1) N/g) of W in the tile layout (mllmb200_w4a32_repack_device with that row range), x is
 * replicated, and every rank ends up with the full fp32 y [M, N] in an output buffer that the library
 * allocates and maps into the other ranks' processes (CUDA IPC).
 *   tp_init          nranks in [1,8]; nccl_comm = an ncclComm_t (as void*) over exactly these ranks, or NULL.
 *                    The library calls NCCL through the copy the process has already loaded (dlopen).
 *   tp_alloc_output  collective: allocates this rank's y buffer (bytes must cover the largest M * N * 4 to be
 *                    used) and a flag array, exchanges their IPC handles over the communicator and maps the peers'.
 *                    Needs the communicator.  Synchronizes `stream`.
 *   tp_ipc_export /  the same in two steps for hosts that move the 128-byte blobs themselves: export allocates and
 *   tp_ipc_import    writes this rank's blob; import takes all ranks' blobs (nranks * 128 bytes, in rank order).
 *   linear_forward_tp  y[:, r N/g : (r+1) N/g] = x W_r^T + b_r on this rank, delivered to all ranks:
 *                    gather_mode 2 = the kernels' epilogues store every finished element into every rank's buffer
 *                    (plain stores over NVLink while other tiles are still computed: the single-launch GEMV for
 *                    M <= 4, the fp16 tensor-core GEMM for kernel policies 4 / 5 at M >= 128; other kernels
 *                    compute the block and push it with strided device copies), then each rank flags every peer
 *                    and waits - bounded, MLLMB200_TIMEOUT through mllmb200_check_device_status - for theirs;
 *                    1 = NCCL baseline (ncclAllGather of the blocks + a re-assembly kernel; needs the
 *                    communicator); 0 = no gather (own columns only).  `kernel` as in linear_forward_ex.
 *                    N must be a multiple of 32 * nranks.  All ranks must make the same sequence of calls.
 *                    Not capturable in a CUDA graph (a call counter is baked into the launches).
 *   tp_output        the buffer again (device pointer, bytes).
 * ------------------------------------------------------------------------------------------ */
MLLMB200_API int mllmb200_w4a32_tp_init(int nranks, int rank, void* nccl_comm, void** handle);
MLLMB200_API int mllmb200_w4a32_tp_alloc_output(void* handle, size_t y_bytes, float** y_dev, void* stream);
MLLMB200_API int mllmb200_w4a32_tp_ipc_export(void* handle, size_t y_bytes, float** y_dev, void* blob_out);
MLLMB200_API int mllmb200_w4a32_tp_ipc_import(void* handle, const void* all_blobs);
MLLMB200_API int mllmb200_w4a32_linear_forward_tp(void* handle, const float* x_dev, const void* tiled_shard_dev,
                                                  void* ws_dev, int M, int K, int N_total, int ldx, int kernel,
                                                  int gather_mode, void* stream);
MLLMB200_API int mllmb200_w4a32_tp_output(void* handle, float** y_dev, size_t* bytes);
MLLMB200_API void mllmb200_w4a32_tp_destroy(void* handle);

/* Self-test of the bounded device-side waits (no counterpart in the reference).  Every wait on an
 * mbarrier in this library has a tick limit; when it runs out the kernel raises the timeout bit of the
 * status word and returns instead of hanging the GPU.  This launches one warp that waits, with the
 * given limit (1 .. 2^31 clock ticks), for 16 bytes that are never sent: afterwards
 * mllmb200_check_device_status reports MLLMB200_TIMEOUT once, and *gave_up_dev (device int, may be
 * NULL) is 1.  The kernel returns normally; nothing faults. */
MLLMB200_API int mllmb200_selftest_wait_timeout(long long limit_ticks, int* gave_up_dev, void* stream);

/* Device-side status word (bounded waits that ran out, bad tile headers).  Synchronizes `stream`,
 * reads and clears the word.  0 = clean. */
MLLMB200_API int mllmb200_check_device_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MLLMB200_H_ */
