// Qwen2-architecture decoder (DeepSeek-Distill-Qwen-1.5B, Qwen2VL-2B language tower) on top of the
// W4A32 linears: host-side orchestration behind a C ABI (include/mllmb200.h, "decoder" section).
// Mirrors the forward of the reference project's model, mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:
// 106-155 (attention), :47-54 (MLP), :175-183 (decoder layer), :202-215 (model), and its greedy
// loop mllm/Models/AutoLLM.hpp:39-65.  Batch 1, fp32 activations and KV cache, fp16 lm_head.
//
// Decode runs as ONE CUDA graph per token, replayed: the position and the current token live in
// device memory, so nothing changes between replays.  In decode every op that feeds a quantized
// linear also writes that linear's int8 activation records, so a layer is 9 launches:
//   add+rmsnorm+quant, gemv(q,k,v), attention over context splits (rotates, appends K/V),
//   merge of the splits + quant, gemv(o), add+rmsnorm+quant,
//   gemv(gate,up), silu*up+quant, gemv(down)      (the residual add of `down` is fused into the next norm)
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <vector>

#include "../../include/mllmb200.h"
#include "decoder_state.h"
#include "device_common.cuh"

namespace mllmb200 {
// persistent decode kernel (decoder_persistent.cu)
void persistent_prepare(Decoder* d);
bool persistent_usable(Decoder* d);
cudaError_t persistent_decode(Decoder* d, int steps);
void persistent_destroy(Decoder* d);
int persistent_phase_cycles(Decoder* d, long long* out, int capacity, int* nctas, int* stamps);
// kernels defined in the other translation units
__global__ void add_rmsnorm_quant_kernel(const float*, const float*, const float*, float, int, float*, float*, uint8_t*,
                                         float2*, int);
__global__ void silu_mul_quant_kernel(const float*, const float*, int, float*, uint8_t*, float2*, int);
__global__ void embedding_kernel(const int*, const float*, int, float*);
__global__ void rope_tables_kernel(float*, float*, int, int, float);
__global__ void rope_kv_append_kernel(const float*, const float*, int, const float*, const float*, const int*, int,
                                      float*, float*);
template <int D>
__global__ void attn_decode_partial_kernel(const float*, const float*, const float*, const float*, const float*, const int*,
                                           int, int, int, float*, float*, float*, float*, int, int);
__global__ void attn_combine_quant_kernel(const float*, const float*, const int*, int, int, int, int, int, float*, uint8_t*,
                                          float2*, int);
template <int D>
__global__ void attention_prefill_kernel(const float*, int, int, const float*, const float*, const int*, int, int, const float*,
                                         const float*, float*, int);
size_t attention_prefill_smem_bytes(int head_dim);
int attention_prefill_rows();
int attention_prefill_threads();
__global__ void lm_head_f16_kernel(const float*, const __half*, int, int, float*, float2*);
__global__ void sample_advance_kernel(const float2*, int, int*, int*, int*, int*, int);
__global__ void act_quant_records_kernel(const float*, int, int, int, uint8_t*, float2*, int, int);
cudaError_t launch_w4a32_gemv_grouped(const uint8_t*, const float2*, int, int, int, const void* const*, float* const*,
                                      const int*, const int*, int, cudaStream_t);
cudaError_t launch_act_quant_records(const float*, int, int, int, uint8_t*, float2*, int, int, cudaStream_t);

__global__ void set_int_kernel(int* dst, int v) { *dst = v; }

namespace {

// launch with the programmatic-dependent-launch attribute (the kernels call griddepcontrol themselves)
template <class... KArgs, class... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define DEC_CHECK(expr)                     \
  do {                                      \
    cudaError_t e__ = (expr);               \
    if (e__ != cudaSuccess) {               \
      d->last_error = (int)e__;             \
      return MLLMB200_CUDA_ERROR;           \
    }                                       \
  } while (0)
#define DEC_ST(expr)                        \
  do {                                      \
    int s__ = (expr);                       \
    if (s__ != MLLMB200_OK) return s__;     \
  } while (0)

int gemv_group(Decoder* d, const uint8_t* rec, const float2* hdr, int k, int count, const int* which, float* const* outs,
               const Layer& L) {
  const void* tiled[4];
  int n[4], ldy[4];
  const auto& c = d->cfg;
  for (int i = 0; i < count; ++i) {
    tiled[i] = L.w[which[i]];
    switch (which[i]) {
      case kQ: case kO: n[i] = (which[i] == kQ) ? c.q_heads * c.head_dim : c.hidden; break;
      case kK: case kV: n[i] = c.kv_heads * c.head_dim; break;
      case kGate: case kUp: n[i] = c.inter; break;
      default: n[i] = c.hidden; break;
    }
    ldy[i] = n[i];
  }
  DEC_CHECK(launch_w4a32_gemv_grouped(rec, hdr, 1, k, count, tiled, outs, n, ldy, 1, d->stream));
  return MLLMB200_OK;
}

// One decode step at the position / token held in device memory.
int enqueue_decode_step(Decoder* d) {
  const auto& c = d->cfg;
  cudaStream_t s = d->stream;
  const int H = c.hidden, QD = c.q_heads * c.head_dim, I = c.inter;
  embedding_kernel<<<1, 256, 0, s>>>(d->token, d->embedding, H, d->h);
  for (int l = 0; l < c.layers; ++l) {
    const Layer& L = d->layers[l];
    DEC_CHECK(launch_pdl(add_rmsnorm_quant_kernel, dim3(1), dim3(256), 0, s, d->h, l == 0 ? nullptr : d->down, L.ln1,
                         c.eps, H, d->h, nullptr, d->rec_a, d->hdr_a, 1));
    {
      const int which[3] = {kQ, kK, kV};
      float* outs[3] = {d->q, d->k, d->v};
      DEC_ST(gemv_group(d, d->rec_a, d->hdr_a, H, 3, which, outs, L));
    }
    {
      const dim3 grid(d->attn_splits, c.kv_heads);
      const int group = c.q_heads / c.kv_heads;
      if (c.head_dim == 128)
        DEC_CHECK(launch_pdl(attn_decode_partial_kernel<128>, grid, dim3(256), 0, s, d->q, d->k, d->v, d->sin_t, d->cos_t,
                             d->pos, c.max_ctx, d->attn_chunk, group, L.cache_k, L.cache_v, d->part_o, d->part_ml,
                             d->attn_splits, 1));
      else
        DEC_CHECK(launch_pdl(attn_decode_partial_kernel<64>, grid, dim3(256), 0, s, d->q, d->k, d->v, d->sin_t, d->cos_t,
                             d->pos, c.max_ctx, d->attn_chunk, group, L.cache_k, L.cache_v, d->part_o, d->part_ml,
                             d->attn_splits, 1));
      DEC_CHECK(launch_pdl(attn_combine_quant_kernel, dim3(1), dim3(512), (size_t)c.q_heads * d->attn_splits * sizeof(float),
                           s, d->part_o, d->part_ml, d->pos, c.max_ctx, d->attn_chunk, d->attn_splits, c.q_heads, c.head_dim,
                           nullptr, d->rec_a, d->hdr_a, 1));
    }
    {
      const int which[1] = {kO};
      float* outs[1] = {d->o};
      DEC_ST(gemv_group(d, d->rec_a, d->hdr_a, QD, 1, which, outs, L));
    }
    DEC_CHECK(launch_pdl(add_rmsnorm_quant_kernel, dim3(1), dim3(256), 0, s, d->h, d->o, L.ln2, c.eps, H, d->h, nullptr,
                         d->rec_a, d->hdr_a, 1));
    {
      const int which[2] = {kGate, kUp};
      float* outs[2] = {d->gate, d->up};
      DEC_ST(gemv_group(d, d->rec_a, d->hdr_a, H, 2, which, outs, L));
    }
    DEC_CHECK(launch_pdl(silu_mul_quant_kernel, dim3(1), dim3(512), (size_t)I * sizeof(float), s, d->gate, d->up, I,
                         nullptr, d->rec_b, d->hdr_b, 1));
    {
      const int which[1] = {kDown};
      float* outs[1] = {d->down};
      DEC_ST(gemv_group(d, d->rec_b, d->hdr_b, I, 1, which, outs, L));
    }
  }
  DEC_CHECK(launch_pdl(add_rmsnorm_quant_kernel, dim3(1), dim3(256), 0, s, d->h, d->down, d->final_norm, c.eps, H, d->h,
                       d->xn, nullptr, nullptr, 1));
  lm_head_f16_kernel<<<kHeadCtas, 256, H * sizeof(float), s>>>(d->xn, d->lm_head, H, c.vocab, d->logits, d->best);
  sample_advance_kernel<<<1, 32, 0, s>>>(d->best, kHeadCtas, d->pos, d->token, d->next, d->history, c.max_ctx);
  DEC_CHECK(cudaGetLastError());
  return MLLMB200_OK;
}

}  // namespace

int check_ready(Decoder* d) {
  if (!d->embedding || !d->lm_head) return MLLMB200_INVALID_ARG;
  for (auto& L : d->layers)
    for (int i = 0; i < kNumLinears; ++i)
      if (!L.w[i]) return MLLMB200_INVALID_ARG;
  return MLLMB200_OK;
}

// The prompt pass of the batch-1 decoder, writing keys / values into the given per-layer caches
// ([kv_heads][max_ctx][D] each) and the sampled token and position into the given words: the decoder's own for
// mllmb200_qwen2_prefill, a sequence's for the batched decoder (decoder_batch.cu).  Exactly one of tokens_dev
// (int32 [n]) and embeds_dev (fp32 [n, hidden], rows that are already embeddings) is given.
int prefill_into(Decoder* d, const int* tokens_dev, const float* embeds_dev, int n, float* const* cache_k,
                 float* const* cache_v, int* pos, int* token, int* next, int* history) {
  if (!d || (tokens_dev == nullptr) == (embeds_dev == nullptr) || n <= 0 || n >= d->cfg.max_ctx) return MLLMB200_INVALID_ARG;
  DEC_ST(check_ready(d));
  const auto& c = d->cfg;
  cudaStream_t s = d->stream;
  const int H = c.hidden, QD = c.q_heads * c.head_dim, KD = c.kv_heads * c.head_dim, I = c.inter;
  if (tokens_dev)
    embedding_kernel<<<n, 256, 0, s>>>(tokens_dev, d->embedding, H, d->h);
  else
    DEC_CHECK(cudaMemcpyAsync(d->h, embeds_dev, (size_t)n * H * sizeof(float), cudaMemcpyDeviceToDevice, s));
  for (int l = 0; l < c.layers; ++l) {
    const Layer& L = d->layers[l];
    add_rmsnorm_quant_kernel<<<n, 256, 0, s>>>(d->h, l == 0 ? nullptr : d->down, L.ln1, c.eps, H, d->h, d->xn, nullptr,
                                               nullptr, 0);
    {  // q, k, v share one quantization of the normalized rows
      const void* tw[3] = {L.w[kQ], L.w[kK], L.w[kV]};
      float* ty[3] = {d->q, d->k, d->v};
      const int tn[3] = {QD, KD, KD};
      DEC_ST(mllmb200_w4a32_linear_forward_grouped(d->xn, n, H, H, 3, tw, ty, tn, tn, d->ws, 5, s));
    }
    rope_kv_append_kernel<<<dim3(c.kv_heads, n), c.head_dim, 0, s>>>(d->k, d->v, KD, d->sin_t, d->cos_t, d->zero, c.max_ctx,
                                                                    cache_k[l], cache_v[l]);
    {
      const int rows = attention_prefill_rows();  // query rows per CTA, one warp each
      const dim3 grid((n + rows - 1) / rows, c.kv_heads);
      const size_t smem = attention_prefill_smem_bytes(c.head_dim);
      if (c.head_dim == 128)
        attention_prefill_kernel<128><<<grid, attention_prefill_threads(), smem, s>>>(d->q, QD, n, d->sin_t, d->cos_t, d->zero, c.max_ctx,
                                                               c.q_heads / c.kv_heads, cache_k[l], cache_v[l], d->attn, QD);
      else
        attention_prefill_kernel<64><<<grid, attention_prefill_threads(), smem, s>>>(d->q, QD, n, d->sin_t, d->cos_t, d->zero, c.max_ctx,
                                                              c.q_heads / c.kv_heads, cache_k[l], cache_v[l], d->attn, QD);
    }
    DEC_ST(mllmb200_w4a32_linear_forward_ex(d->attn, L.w[kO], d->o, d->ws, n, QD, H, QD, H, 5, s));
    add_rmsnorm_quant_kernel<<<n, 256, 0, s>>>(d->h, d->o, L.ln2, c.eps, H, d->h, d->xn, nullptr, nullptr, 0);
    {  // gate and up likewise
      const void* tw[2] = {L.w[kGate], L.w[kUp]};
      float* ty[2] = {d->gate, d->up};
      const int tn[2] = {I, I};
      DEC_ST(mllmb200_w4a32_linear_forward_grouped(d->xn, n, H, H, 2, tw, ty, tn, tn, d->ws, 5, s));
    }
    silu_mul_quant_kernel<<<n, 512, (size_t)I * sizeof(float), s>>>(d->gate, d->up, I, d->act, nullptr, nullptr, 0);
    DEC_ST(mllmb200_w4a32_linear_forward_ex(d->act, L.w[kDown], d->down, d->ws, n, I, H, I, H, 5, s));
  }
  // only the last position feeds the sampler (the reference computes all rows and reads the last)
  const size_t last = (size_t)(n - 1) * H;
  add_rmsnorm_quant_kernel<<<1, 256, 0, s>>>(d->h + last, d->down + last, d->final_norm, c.eps, H, nullptr, d->xn, nullptr,
                                             nullptr, 0);
  lm_head_f16_kernel<<<kHeadCtas, 256, H * sizeof(float), s>>>(d->xn, d->lm_head, H, c.vocab, d->logits, d->best);
  set_int_kernel<<<1, 1, 0, s>>>(pos, n - 1);
  sample_advance_kernel<<<1, 32, 0, s>>>(d->best, kHeadCtas, pos, token, next, history, c.max_ctx);
  DEC_CHECK(cudaGetLastError());
  return MLLMB200_OK;
}

}  // namespace mllmb200

#include "decoder_api.inc"
