// Host-side state of the decoder (shared by decoder.cu and decoder_persistent.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "../../include/mllmb200.h"

namespace mllmb200 {

struct PersistentState;  // decoder_persistent.cu

enum { kQ = 0, kK, kV, kO, kGate, kUp, kDown, kNumLinears };
constexpr int kHeadCtas = 148 * 4;

struct Layer {
  void* w[kNumLinears] = {};
  float *ln1 = nullptr, *ln2 = nullptr;
  float *cache_k = nullptr, *cache_v = nullptr;
};

struct Decoder {
  mllmb200_qwen2_config cfg{};
  std::vector<Layer> layers;
  float* final_norm = nullptr;
  const float* embedding = nullptr;  // borrowed, fp32 [vocab, hidden]
  const __half* lm_head = nullptr;   // borrowed, fp16 [vocab, hidden]
  float *sin_t = nullptr, *cos_t = nullptr;
  // activations (rows = max_ctx for prefill; decode uses row 0)
  float *h = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *o = nullptr;
  float *gate = nullptr, *up = nullptr, *act = nullptr, *down = nullptr, *logits = nullptr;
  uint8_t *rec_a = nullptr, *rec_b = nullptr;  // activation records (hidden-wide and inter-wide)
  float2 *hdr_a = nullptr, *hdr_b = nullptr;
  float2* best = nullptr;  // per-CTA argmax candidates of the lm_head kernel
  float *part_o = nullptr, *part_ml = nullptr;  // per-split attention partials (decode)
  int attn_chunk = 32, attn_splits = 1;
  void* ws = nullptr;  // workspace of the public forward (prefill)
  size_t ws_bytes = 0;
  int *pos = nullptr, *token = nullptr, *next = nullptr, *history = nullptr, *zero = nullptr;
  cudaStream_t stream = nullptr;
  cudaGraphExec_t graph = nullptr;
  PersistentState* persist = nullptr;  // persistent decode kernel state (built on first use)
  int profile = 0;                     // persistent kernel: record per-phase cycle counts
  int host_pos = 0;                    // tokens in the cache, tracked on the host to bound requests
  std::vector<void*> owned;
  int last_error = 0;
};

template <class T>
bool dev_alloc(Decoder* d, T** p, size_t count) {
  void* q = nullptr;
  if (cudaMalloc(&q, count * sizeof(T)) != cudaSuccess) return false;
  d->owned.push_back(q);
  *p = static_cast<T*>(q);
  return true;
}


}  // namespace mllmb200
