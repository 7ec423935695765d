// Batched greedy decode on top of the batch-1 decoder: B sequences, each with its own KV cache and position,
// advance one token per step together, so that every quantized linear of the step runs at M = B.
//
// The reference project has no such mode - its KV cache asserts a batch of one
// (mllm/Backends/Arm/Ops/KVCacheOp.cpp:107,156) - so the semantics are those of B independent runs of its
// batch-1 forward (mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:106-155, cache append KVCacheOp.cpp:15-72, greedy
// loop mllm/Models/AutoLLM.hpp:39-105): sequence b of the batch must produce the tokens a batch-1 decoder
// produces on sequence b alone.  The tests check exactly that.
//
// A batch object borrows weights, norms, tables and the stream of a batch-1 decoder (mllmb200_qwen2_create ...)
// and adds per-sequence state: KV caches [layer][sequence][kv head][max_ctx][D] in fp32, positions, current
// tokens, histories.  Sequences are prefilled one at a time through the batch-1 prefill (from token ids, or from
// ready embedding rows for inputs that mix text with vision-patch embeddings) into their own caches; prompts may
// differ in length.  A decode step is then:
//   embedding rows -> per layer { add + RMSNorm (one CTA per row) -> q,k,v = W4A32 linears at M = B (one grouped
//   call) -> attention over (context split, kv head, sequence) CTAs, which also rotate and append the new K/V ->
//   merge of the splits (one CTA per sequence) -> o linear -> add + RMSNorm -> gate,up linears -> silu * up -> down }
//   -> final norm -> lm_head for all rows -> per-sequence argmax and bookkeeping,
// captured once as a CUDA graph and replayed (positions and tokens live in device memory).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <vector>

#include "../../include/mllmb200.h"
#include "decoder_attn_body.cuh"
#include "decoder_state.h"
#include "device_common.cuh"

namespace mllmb200 {

__global__ void add_rmsnorm_quant_kernel(const float*, const float*, const float*, float, int, float*, float*, uint8_t*,
                                         float2*, int);
__global__ void silu_mul_quant_kernel(const float*, const float*, int, float*, uint8_t*, float2*, int);
__global__ void embedding_kernel(const int*, const float*, int, float*);

// Decode-step attention for a batch: grid (splits, kv_heads, sequences), 256 threads; the work of a CTA is
// attn_partial_body on the sequence's own cache and position.
// q: [B][ldq], k_new / v_new: [B][ldkv]; caches [B][kv_heads][max_ctx][D]; part_o [B][q_heads][splits][D],
// part_ml [B][q_heads][splits][2].
template <int D>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_partial_batched_kernel(
    const float* __restrict__ q, int ldq, const float* __restrict__ k_new, const float* __restrict__ v_new, int ldkv,
    const float* __restrict__ sin_t, const float* __restrict__ cos_t, const int* __restrict__ pos_ptr, int max_ctx, int chunk,
    int group, int q_heads, float* __restrict__ cache_k, float* __restrict__ cache_v, size_t cache_seq_stride,
    float* __restrict__ part_o, float* __restrict__ part_ml, int splits) {
  __shared__ AttnSmem<D> sm;
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int pos = min(pos_ptr[seq], max_ctx - 1);
  if (split * chunk > pos) return;
  const size_t head0 = (size_t)seq * q_heads + (size_t)kvh * group;
  attn_partial_body<D>(sm, threadIdx.x, [] { __syncthreads(); }, q + (size_t)seq * ldq + (size_t)kvh * group * D,
                       k_new + (size_t)seq * ldkv + kvh * D, v_new + (size_t)seq * ldkv + kvh * D,
                       sin_t + (size_t)pos * (D / 2), cos_t + (size_t)pos * (D / 2), pos, split * chunk,
                       min((split + 1) * chunk, pos + 1), group,
                       cache_k + (size_t)seq * cache_seq_stride + (size_t)kvh * max_ctx * D,
                       cache_v + (size_t)seq * cache_seq_stride + (size_t)kvh * max_ctx * D, part_o + head0 * splits * D,
                       part_ml + head0 * splits * 2, splits, split);
}

// Merge of the context splits of one sequence per CTA (the arithmetic of attn_combine_quant_kernel, fp32 output):
//   w[h][s] = exp(m[h][s] - max_s m) / sum_s(l[h][s] * exp(m[h][s] - max_s m));  out[h][d] = sum_s w[h][s] * o[h][s][d]
// Dynamic shared memory: q_heads * splits floats.
constexpr int kBatchCombineThreads = 512;
__global__ void __launch_bounds__(kBatchCombineThreads) attn_combine_batched_kernel(
    const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ pos_ptr, int max_ctx,
    int chunk, int splits, int q_heads, int head_dim, float* __restrict__ attn_out) {
  extern __shared__ float s_w[];  // [q_heads][splits]
  const int seq = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos = min(pos_ptr[seq], max_ctx - 1);
  const int nact = min(splits, pos / chunk + 1);
  part_o += (size_t)seq * q_heads * splits * head_dim;
  part_ml += (size_t)seq * q_heads * splits * 2;
  for (int h = warp; h < q_heads; h += kBatchCombineThreads / 32) {
    const float* ml = part_ml + (size_t)h * splits * 2;
    float mx = -3.402823466e+38f;
    for (int sidx = lane; sidx < nact; sidx += 32) mx = fmaxf(mx, ml[sidx * 2]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float tot = 0.0f;
    for (int sidx = lane; sidx < nact; sidx += 32) {
      const float e = expf(ml[sidx * 2] - mx);
      s_w[h * splits + sidx] = e;
      tot += ml[sidx * 2 + 1] * e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const float inv = 1.0f / tot;
    for (int sidx = lane; sidx < nact; sidx += 32) s_w[h * splits + sidx] *= inv;  // same lane wrote it
  }
  __syncthreads();
  const int width = q_heads * head_dim;
  for (int idx = tid; idx < width; idx += kBatchCombineThreads) {
    const int h = idx / head_dim, d = idx - h * head_dim;
    const float* po = part_o + (size_t)h * splits * head_dim + d;
    float acc = 0.0f;
    for (int s0 = 0; s0 < nact; s0 += 8) {  // eight partial rows requested together; summed in split order
      float pv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) pv[j] = po[(size_t)min(s0 + j, nact - 1) * head_dim];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(s0 + j < nact ? s_w[h * splits + s0 + j] : 0.0f, pv[j], acc);
    }
    attn_out[(size_t)seq * width + idx] = acc;
  }
}

// logits[b][v] = sum_k x[b][k] * W[v][k] for a tile of kLmRows activation rows (blockIdx.y) and the vocabulary rows
// v = 4 * (blockIdx.x * 8 + warp) + {0..3}, stepping by 4 * 8 * gridDim.x: W fp16 [V, hidden], x fp32, fp32
// accumulation.  A warp holds the 16-byte chunks of FOUR vocabulary rows in registers and runs every activation
// row of the tile (fp32 in shared memory) past them, so a weight row is fetched once per tile of 16 activation
// rows.  Per (b, v) the lane-to-chunk assignment, the order of the FMAs and the shuffle tree are those of
// lm_head_f16_kernel: the logits are bit-identical to the batch-1 kernel's.  Each CTA also leaves, per activation
// row, its largest logit and the index (lowest index on ties) in best[b][blockIdx.x].
constexpr int kLmRows = 16;   // activation rows per CTA tile
constexpr int kLmVocab = 4;   // vocabulary rows a warp keeps in registers
__global__ void __launch_bounds__(256) lm_head_f16_batched_kernel(const float* __restrict__ x, int batch,
                                                                  const __half* __restrict__ w, int hidden, int vocab,
                                                                  float* __restrict__ logits, float2* __restrict__ best) {
  extern __shared__ float s_x[];  // [kLmRows][hidden]
  __shared__ float s_bv[kLmRows][8];
  __shared__ int s_bi[kLmRows][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b0 = blockIdx.y * kLmRows;
  const int nb = min(kLmRows, batch - b0);
  for (int i = threadIdx.x; i < kLmRows * hidden; i += blockDim.x) {
    const int r = i / hidden;
    s_x[i] = r < nb ? x[(size_t)(b0 + r) * hidden + (i - r * hidden)] : 0.0f;
  }
  __syncthreads();
  float bv[kLmRows];
  int bi[kLmRows];
#pragma unroll
  for (int r = 0; r < kLmRows; ++r) bv[r] = -3.402823466e+38f, bi[r] = 0x7fffffff;
  const int chunks = hidden >> 3;
  for (int v0 = kLmVocab * (blockIdx.x * 8 + warp); v0 < vocab; v0 += kLmVocab * 8 * gridDim.x) {
    float acc[kLmVocab][kLmRows];
#pragma unroll
    for (int j = 0; j < kLmVocab; ++j)
#pragma unroll
      for (int r = 0; r < kLmRows; ++r) acc[j][r] = 0.0f;
    for (int c = lane; c < chunks; c += 32) {
      uint4 pk[kLmVocab];
#pragma unroll
      for (int j = 0; j < kLmVocab; ++j)
        pk[j] = v0 + j < vocab ? reinterpret_cast<const uint4*>(w + (size_t)(v0 + j) * hidden)[c] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int r = 0; r < kLmRows; ++r) {
        const float4 xa = *reinterpret_cast<const float4*>(s_x + (size_t)r * hidden + c * 8);
        const float4 xb = *reinterpret_cast<const float4*>(s_x + (size_t)r * hidden + c * 8 + 4);
        const float xs[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int j = 0; j < kLmVocab; ++j) {
          const __half2* h2 = reinterpret_cast<const __half2*>(&pk[j]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h2[e]);
            acc[j][r] = fmaf(f.x, xs[2 * e], acc[j][r]);
            acc[j][r] = fmaf(f.y, xs[2 * e + 1], acc[j][r]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kLmVocab; ++j) {
#pragma unroll
      for (int r = 0; r < kLmRows; ++r) {
        float a = acc[j][r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        const int v = v0 + j;
        if (v < vocab && r < nb) {
          if (lane == 0 && logits) logits[(size_t)(b0 + r) * vocab + v] = a;
          if (a > bv[r]) {  // rows come in increasing order within a warp: a strict test keeps the lowest index
            bv[r] = a;
            bi[r] = v;
          }
        }
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < kLmRows; ++r) {
      s_bv[r][warp] = bv[r];
      s_bi[r][warp] = bi[r];
    }
  }
  __syncthreads();
  if (threadIdx.x < nb) {
    const int r = threadIdx.x;
    float v = s_bv[r][0];
    int i = s_bi[r][0];
    for (int k = 1; k < 8; ++k)
      if (s_bv[r][k] > v || (s_bv[r][k] == v && s_bi[r][k] < i)) {
        v = s_bv[r][k];
        i = s_bi[r][k];
      }
    best[(size_t)(b0 + r) * gridDim.x + blockIdx.x] = make_float2(v, __int_as_float(i));
  }
}

// Greedy sampling and bookkeeping of a step for every sequence (one warp each): sample_advance_kernel per row.
__global__ void sample_advance_batched_kernel(const float2* __restrict__ best, int count, int* __restrict__ pos,
                                              int* __restrict__ token, int* __restrict__ history, int max_hist) {
  const int seq = blockIdx.x;
  best += (size_t)seq * count;
  float bv = -3.402823466e+38f;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < count; i += 32) {
    const float2 c = best[i];
    const int ci = __float_as_int(c.y);
    if (c.x > bv || (c.x == bv && ci < bi)) {
      bv = c.x;
      bi = ci;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if (threadIdx.x == 0) {
    const int p = pos[seq];
    token[seq] = bi;
    if (p < max_hist) history[(size_t)seq * max_hist + p] = bi;
    pos[seq] = p + 1;
  }
}

namespace {

constexpr int kLmCtas = 148;  // vocabulary CTAs of the batched lm_head (x ceil(B / 16) activation tiles)

struct BatchDecoder {
  Decoder* base = nullptr;
  int batch = 0;
  std::vector<float*> cache_k, cache_v;  // per layer: [batch][kv_heads][max_ctx][D]
  size_t cache_seq_stride = 0;
  float *h = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *o = nullptr;
  float *gate = nullptr, *up = nullptr, *act = nullptr, *down = nullptr, *logits = nullptr;
  float *part_o = nullptr, *part_ml = nullptr;
  float2* best = nullptr;
  int *pos = nullptr, *token = nullptr, *history = nullptr, *scratch_next = nullptr;
  void* ws = nullptr;
  std::vector<int> host_pos;  // tokens in each sequence's cache (0 = not prefilled)
  cudaGraphExec_t graph = nullptr;
  int policy = 0;
  std::vector<void*> owned;
  int last_error = 0;
};

template <class T>
bool balloc(BatchDecoder* b, T** p, size_t count) {
  void* q = nullptr;
  if (cudaMalloc(&q, count * sizeof(T)) != cudaSuccess) return false;
  b->owned.push_back(q);
  *p = static_cast<T*>(q);
  return true;
}

#define BD_CHECK(expr)                      \
  do {                                      \
    cudaError_t e__ = (expr);               \
    if (e__ != cudaSuccess) {               \
      b->last_error = (int)e__;             \
      return MLLMB200_CUDA_ERROR;           \
    }                                       \
  } while (0)
#define BD_ST(expr)                         \
  do {                                      \
    int s__ = (expr);                       \
    if (s__ != MLLMB200_OK) return s__;     \
  } while (0)

int enqueue_batched_step(BatchDecoder* b) {
  Decoder* d = b->base;
  const auto& c = d->cfg;
  cudaStream_t s = d->stream;
  const int B = b->batch, H = c.hidden, QD = c.q_heads * c.head_dim, KD = c.kv_heads * c.head_dim, I = c.inter;
  const int group = c.q_heads / c.kv_heads;
  embedding_kernel<<<B, 256, 0, s>>>(b->token, d->embedding, H, b->h);
  for (int l = 0; l < c.layers; ++l) {
    const Layer& L = d->layers[l];
    add_rmsnorm_quant_kernel<<<B, 256, 0, s>>>(b->h, l == 0 ? nullptr : b->down, L.ln1, c.eps, H, b->h, b->xn, nullptr,
                                               nullptr, 0);
    {
      const void* tw[3] = {L.w[kQ], L.w[kK], L.w[kV]};
      float* ty[3] = {b->q, b->k, b->v};
      const int tn[3] = {QD, KD, KD};
      BD_ST(mllmb200_w4a32_linear_forward_grouped(b->xn, B, H, H, 3, tw, ty, tn, tn, b->ws, b->policy, s));
    }
    {
      const dim3 grid(d->attn_splits, c.kv_heads, B);
      if (c.head_dim == 128)
        attn_decode_partial_batched_kernel<128><<<grid, kAttnThreads, 0, s>>>(
            b->q, QD, b->k, b->v, KD, d->sin_t, d->cos_t, b->pos, c.max_ctx, d->attn_chunk, group, c.q_heads, b->cache_k[l],
            b->cache_v[l], b->cache_seq_stride, b->part_o, b->part_ml, d->attn_splits);
      else
        attn_decode_partial_batched_kernel<64><<<grid, kAttnThreads, 0, s>>>(
            b->q, QD, b->k, b->v, KD, d->sin_t, d->cos_t, b->pos, c.max_ctx, d->attn_chunk, group, c.q_heads, b->cache_k[l],
            b->cache_v[l], b->cache_seq_stride, b->part_o, b->part_ml, d->attn_splits);
      attn_combine_batched_kernel<<<B, kBatchCombineThreads, (size_t)c.q_heads * d->attn_splits * sizeof(float), s>>>(
          b->part_o, b->part_ml, b->pos, c.max_ctx, d->attn_chunk, d->attn_splits, c.q_heads, c.head_dim, b->attn);
    }
    BD_ST(mllmb200_w4a32_linear_forward_ex(b->attn, L.w[kO], b->o, b->ws, B, QD, H, QD, H, b->policy, s));
    add_rmsnorm_quant_kernel<<<B, 256, 0, s>>>(b->h, b->o, L.ln2, c.eps, H, b->h, b->xn, nullptr, nullptr, 0);
    {
      const void* tw[2] = {L.w[kGate], L.w[kUp]};
      float* ty[2] = {b->gate, b->up};
      const int tn[2] = {I, I};
      BD_ST(mllmb200_w4a32_linear_forward_grouped(b->xn, B, H, H, 2, tw, ty, tn, tn, b->ws, b->policy, s));
    }
    silu_mul_quant_kernel<<<B, 512, (size_t)I * sizeof(float), s>>>(b->gate, b->up, I, b->act, nullptr, nullptr, 0);
    BD_ST(mllmb200_w4a32_linear_forward_ex(b->act, L.w[kDown], b->down, b->ws, B, I, H, I, H, b->policy, s));
  }
  add_rmsnorm_quant_kernel<<<B, 256, 0, s>>>(b->h, b->down, d->final_norm, c.eps, H, nullptr, b->xn, nullptr, nullptr, 0);
  {
    const dim3 grid(kLmCtas, (B + kLmRows - 1) / kLmRows);
    lm_head_f16_batched_kernel<<<grid, 256, (size_t)kLmRows * H * sizeof(float), s>>>(b->xn, B, d->lm_head, H, c.vocab,
                                                                                      b->logits, b->best);
  }
  sample_advance_batched_kernel<<<B, 32, 0, s>>>(b->best, kLmCtas, b->pos, b->token, b->history, c.max_ctx);
  BD_CHECK(cudaGetLastError());
  return MLLMB200_OK;
}

}  // namespace

// decoder.cu: the batch-1 prefill writing into the given caches and bookkeeping words.
int prefill_into(Decoder* d, const int* tokens_dev, const float* embeds_dev, int n, float* const* cache_k,
                 float* const* cache_v, int* pos, int* token, int* next, int* history);

}  // namespace mllmb200

using namespace mllmb200;

extern "C" {

int mllmb200_qwen2_batch_create(void* decoder, int batch, void** handle) {
  auto* d = static_cast<Decoder*>(decoder);
  if (!d || !handle || batch < 1 || batch > 1024) return MLLMB200_INVALID_ARG;
  const auto& c = d->cfg;
  auto* b = new BatchDecoder();
  b->base = d;
  b->batch = batch;
  b->host_pos.assign(batch, 0);
  const size_t B = (size_t)batch;
  const int QD = c.q_heads * c.head_dim, KD = c.kv_heads * c.head_dim;
  b->cache_seq_stride = (size_t)c.kv_heads * c.max_ctx * c.head_dim;
  bool ok = balloc(b, &b->h, B * c.hidden) && balloc(b, &b->xn, B * c.hidden) && balloc(b, &b->q, B * QD) &&
            balloc(b, &b->k, B * KD) && balloc(b, &b->v, B * KD) && balloc(b, &b->attn, B * QD) && balloc(b, &b->o, B * c.hidden) &&
            balloc(b, &b->gate, B * c.inter) && balloc(b, &b->up, B * c.inter) && balloc(b, &b->act, B * c.inter) &&
            balloc(b, &b->down, B * c.hidden) && balloc(b, &b->logits, B * c.vocab) &&
            balloc(b, &b->part_o, B * c.q_heads * d->attn_splits * c.head_dim) &&
            balloc(b, &b->part_ml, B * c.q_heads * d->attn_splits * 2) && balloc(b, &b->best, B * kLmCtas) &&
            balloc(b, &b->pos, B) && balloc(b, &b->token, B) && balloc(b, &b->scratch_next, 1) &&
            balloc(b, &b->history, B * c.max_ctx);
  size_t wsb = 0;
  const int max_k = std::max(std::max(c.inter, c.hidden), QD);
  ok = ok && mllmb200_w4a32_workspace_size(batch, max_k, &wsb) == MLLMB200_OK;
  if (ok) {
    uint8_t* w = nullptr;
    ok = balloc(b, &w, wsb);
    b->ws = w;
  }
  b->cache_k.resize(c.layers);
  b->cache_v.resize(c.layers);
  for (int l = 0; ok && l < c.layers; ++l)
    ok = balloc(b, &b->cache_k[l], B * b->cache_seq_stride) && balloc(b, &b->cache_v[l], B * b->cache_seq_stride);
  if (ok)
    ok = cudaFuncSetAttribute(lm_head_f16_batched_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)((size_t)kLmRows * c.hidden * sizeof(float))) == cudaSuccess &&
         cudaMemsetAsync(b->pos, 0, B * sizeof(int), d->stream) == cudaSuccess &&
         cudaMemsetAsync(b->token, 0, B * sizeof(int), d->stream) == cudaSuccess &&
         cudaStreamSynchronize(d->stream) == cudaSuccess;
  if (!ok) {
    for (void* p : b->owned) cudaFree(p);
    delete b;
    return MLLMB200_CUDA_ERROR;
  }
  *handle = b;
  return MLLMB200_OK;
}

void mllmb200_qwen2_batch_destroy(void* handle) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b) return;
  cudaStreamSynchronize(b->base->stream);
  if (b->graph) cudaGraphExecDestroy(b->graph);
  for (void* p : b->owned) cudaFree(p);
  delete b;
}

// Kernel policy of the M = batch linears (0 auto: exact int32 group sums; 4 / 5: fp16 tensor cores where they apply).
int mllmb200_qwen2_batch_set_policy(void* handle, int policy) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b || (policy != 0 && policy != 4 && policy != 5)) return MLLMB200_INVALID_ARG;
  if (policy != b->policy && b->graph) {
    cudaGraphExecDestroy(b->graph);
    b->graph = nullptr;
  }
  b->policy = policy;
  return MLLMB200_OK;
}

// Prefills sequence `seq` from an empty cache and samples its first token.  Exactly one of tokens_dev (int32 [n])
// and embeds_dev (fp32 [n, hidden]: rows that are already embeddings, e.g. vision-patch embeddings mixed with
// looked-up text tokens) is given.  Asynchronous on the decoder's stream.
int mllmb200_qwen2_batch_prefill(void* handle, int seq, const int* tokens_dev, const float* embeds_dev, int n) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b || seq < 0 || seq >= b->batch || (tokens_dev == nullptr) == (embeds_dev == nullptr) || n <= 0 ||
      n >= b->base->cfg.max_ctx)
    return MLLMB200_INVALID_ARG;
  Decoder* d = b->base;
  const int layers = d->cfg.layers;
  std::vector<float*> ck(layers), cv(layers);
  for (int l = 0; l < layers; ++l) {
    ck[l] = b->cache_k[l] + (size_t)seq * b->cache_seq_stride;
    cv[l] = b->cache_v[l] + (size_t)seq * b->cache_seq_stride;
  }
  BD_ST(prefill_into(d, tokens_dev, embeds_dev, n, ck.data(), cv.data(), b->pos + seq, b->token + seq, b->scratch_next,
                     b->history + (size_t)seq * d->cfg.max_ctx));
  b->host_pos[seq] = n;
  return MLLMB200_OK;
}

// `steps` greedy steps for all sequences together (every sequence needs a prefill first and room in its cache).
int mllmb200_qwen2_batch_decode(void* handle, int steps) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b || steps < 0) return MLLMB200_INVALID_ARG;
  Decoder* d = b->base;
  for (int p : b->host_pos)
    if (p < 1 || p + steps > d->cfg.max_ctx) return MLLMB200_INVALID_ARG;
  if (steps == 0) return MLLMB200_OK;
  auto advance = [&] {
    for (int& p : b->host_pos) ++p;
  };
  if (!b->graph) {
    BD_ST(enqueue_batched_step(b));  // plain run first: kernel attributes get configured outside capture
    advance();
    BD_CHECK(cudaStreamSynchronize(d->stream));
    --steps;
    if (steps == 0) return MLLMB200_OK;
    cudaGraph_t g = nullptr;
    BD_CHECK(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
    const int st = enqueue_batched_step(b);
    cudaError_t e = cudaStreamEndCapture(d->stream, &g);
    if (st != MLLMB200_OK || e != cudaSuccess) {
      if (g) cudaGraphDestroy(g);
      if (st != MLLMB200_OK) return st;
      BD_CHECK(e);
    }
    e = cudaGraphInstantiate(&b->graph, g, 0);
    cudaGraphDestroy(g);
    BD_CHECK(e);
  }
  for (int i = 0; i < steps; ++i) {
    BD_CHECK(cudaGraphLaunch(b->graph, d->stream));
    advance();
  }
  return MLLMB200_OK;
}

// Synchronizes; copies to HOST memory history[first, first + count) of sequence `seq` (entry p = the token sampled
// after position p), its number of cached tokens, and the last logits [vocab] of that sequence; NULLs are skipped.
int mllmb200_qwen2_batch_read(void* handle, int seq, int first, int count, int* tokens_out, int* pos_out, float* logits_out) {
  auto* b = static_cast<BatchDecoder*>(handle);
  if (!b || seq < 0 || seq >= b->batch || first < 0 || count < 0 || first + count > b->base->cfg.max_ctx)
    return MLLMB200_INVALID_ARG;
  Decoder* d = b->base;
  BD_CHECK(cudaStreamSynchronize(d->stream));
  if (tokens_out && count)
    BD_CHECK(cudaMemcpy(tokens_out, b->history + (size_t)seq * d->cfg.max_ctx + first, (size_t)count * 4, cudaMemcpyDeviceToHost));
  if (pos_out) BD_CHECK(cudaMemcpy(pos_out, b->pos + seq, 4, cudaMemcpyDeviceToHost));
  if (logits_out)
    BD_CHECK(cudaMemcpy(logits_out, b->logits + (size_t)seq * d->cfg.vocab, (size_t)d->cfg.vocab * 4, cudaMemcpyDeviceToHost));
  return MLLMB200_OK;
}

}  // extern "C"
