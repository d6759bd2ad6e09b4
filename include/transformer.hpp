#pragma once
// runtime::Transformer over the paged library: the reference's stack of 16 TransformerBlocks
// (src/runtime/transformer.hpp:7-30, src/runtime/transformer.cu:6-89; a block is
// src/runtime/transformer_block.cu:24-123: x + Attention(x), then a + FeedForward(a)) with the same
// constructor arguments, the same forward(input, output, position, seq_len) and the same cache
// accessors, taking raw device pointers where the reference takes its Tensor
// (src/runtime/tensor.hpp:9-41; data_bf16() is what a caller passes).
//
// What forward() runs:
//   seq_len == 1   pa_block_step over all 16 layers: five launches per layer chained by programmatic
//                  dependent launch, no allocation, no synchronisation between layers.  The
//                  reference's weights are one allocation per matrix; pa_block_step addresses layer l
//                  as base + l * stride, so the object calls it once for all layers when the 16
//                  pointers of every kind are equally spaced, and once per layer otherwise.
//   seq_len  > 1   per layer pa_rmsnorm, pa_qkv_project_append (tensor-core GEMM, RoPE and the cache
//                  append as its epilogue), pa_prefill, pa_out_project_rows (+ residual) and
//                  pa_ffn_rows (+ residual), on copies of the weights packed at construction (one
//                  more copy of the layers' weights: 1.9 GB).
// Like the reference's forward() it returns with `output` complete.  Errors print and exit, as the
// reference's CUDA_CHECK does.  One pool holds the cache of all layers: ceil(max_seq_len / 16) blocks
// per layer where the reference holds two [8, max_seq_len, 64] tensors per layer.  position must
// equal the number of tokens already cached; position == 0 starts a new sequence.
#include <cstdio>
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "paged_attention.h"
#include "weights.hpp"

namespace runtime {

class Transformer {
 public:
  Transformer(llama::LlamaWeights& weights, float* cos_table, float* sin_table, int max_seq_len)
      : cos_table_(cos_table), sin_table_(sin_table), max_seq_len_(max_seq_len) {
    int dev = 0;
    cuda(cudaGetDevice(&dev));
    const int blocks = (max_seq_len + PA_BLOCK_TOKENS - 1) / PA_BLOCK_TOKENS;
    pa(pa_pool_create(&pool_, dev, kLayers, blocks, 8, 1, blocks));
    pa(pa_seq_create(pool_, &seq_));
    for (int l = 0; l < kLayers; l++) {
      const auto& w = weights.layers[l];
      att_[l] = {};
      att_[l].input_norm = w.input_layernorm;
      att_[l].wq = w.q_proj;
      att_[l].wk = w.k_proj;
      att_[l].wv = w.v_proj;
      att_[l].wo = w.o_proj;
      att_[l].rms_eps = 1e-5f;
      att_[l].hidden = kHidden;
      ffn_[l] = {};
      ffn_[l].ffn_norm = w.post_attention_layernorm;
      ffn_[l].gate = w.gate_proj;
      ffn_[l].up = w.up_proj;
      ffn_[l].down = w.down_proj;
      ffn_[l].rms_eps = 1e-5f;
      ffn_[l].hidden = kHidden;
      ffn_[l].inter = kInter;
    }
    // equally spaced layers: one descriptor with strides serves every layer in one call
    const auto& a = weights.layers[0];
    const auto& b = weights.layers[1];
    strided_ = true;
    all_att_ = att_[0];
    all_att_.norm_layer_stride = b.input_layernorm - a.input_layernorm;
    all_att_.wq_layer_stride = b.q_proj - a.q_proj;
    all_att_.wkv_layer_stride = b.k_proj - a.k_proj;
    all_att_.wo_layer_stride = b.o_proj - a.o_proj;
    all_ffn_ = ffn_[0];
    all_ffn_.norm_layer_stride = b.post_attention_layernorm - a.post_attention_layernorm;
    all_ffn_.gate_layer_stride = b.gate_proj - a.gate_proj;
    all_ffn_.up_layer_stride = b.up_proj - a.up_proj;
    all_ffn_.down_layer_stride = b.down_proj - a.down_proj;
    for (int l = 0; l < kLayers; l++) {
      const auto& w = weights.layers[l];
      strided_ = strided_ && w.input_layernorm == a.input_layernorm + l * all_att_.norm_layer_stride &&
                 w.q_proj == a.q_proj + l * all_att_.wq_layer_stride && w.k_proj == a.k_proj + l * all_att_.wkv_layer_stride &&
                 w.v_proj == a.v_proj + l * all_att_.wkv_layer_stride && w.o_proj == a.o_proj + l * all_att_.wo_layer_stride &&
                 w.post_attention_layernorm == a.post_attention_layernorm + l * all_ffn_.norm_layer_stride &&
                 w.gate_proj == a.gate_proj + l * all_ffn_.gate_layer_stride &&
                 w.up_proj == a.up_proj + l * all_ffn_.up_layer_stride &&
                 w.down_proj == a.down_proj + l * all_ffn_.down_layer_stride;
    }
    cuda(cudaMalloc(&ping_, (size_t)2 * 8 * kHidden * sizeof(__nv_bfloat16)));
    cuda(cudaDeviceSynchronize());
  }
  Transformer(const Transformer&) = delete;
  Transformer& operator=(const Transformer&) = delete;
  ~Transformer() {
    cudaDeviceSynchronize();
    pa_pool_destroy(pool_);
    cudaFree(ping_);
    cudaFree(packed_);
    cudaFree(rows_);
    cudaFree(key_view_);
    cudaFree(value_view_);
  }

  // Set-up call for prompts of up to max_rows tokens: the packed weight copies and the rows between
  // the kernels of the prompt path (made on the first prompt otherwise).
  void reserve_prompt(int max_rows) {
    if (!packed_) {
      cuda(cudaMalloc(&packed_, (size_t)kLayers * kPackedLayer * sizeof(__nv_bfloat16)));
      for (int l = 0; l < kLayers; l++) {
        __nv_bfloat16* p = packed_ + (size_t)l * kPackedLayer;
        pa(pa_pack_projection_weights(att_[l].wq, p + kOffQ, kHidden, kHidden, nullptr));
        pa(pa_pack_projection_weights(att_[l].wk, p + kOffK, kHidden, 512, nullptr));
        pa(pa_pack_projection_weights(att_[l].wv, p + kOffV, kHidden, 512, nullptr));
        pa(pa_pack_projection_weights(att_[l].wo, p + kOffO, kHidden, kHidden, nullptr));
        pa(pa_pack_projection_weights(ffn_[l].gate, p + kOffG, kHidden, kInter, nullptr));
        pa(pa_pack_projection_weights(ffn_[l].up, p + kOffU, kHidden, kInter, nullptr));
        pa(pa_pack_projection_weights(ffn_[l].down, p + kOffD, kInter, kHidden, nullptr));
      }
    }
    if (max_rows > rows_cap_) {
      cuda(cudaDeviceSynchronize());
      cudaFree(rows_);
      // normalised rows, rotated q, attention rows, block middle rows, two block outputs in turn, FFN scratch
      cuda(cudaMalloc(&rows_, (size_t)max_rows * (6 * kHidden + kHidden + kInter) * sizeof(__nv_bfloat16)));
      rows_cap_ = max_rows;
    }
  }

  // input, output: [seq_len, 2048] bf16 on the device (the reference's Tensor::data_bf16())
  void forward(const __nv_bfloat16* input, __nv_bfloat16* output, int position, int seq_len) {
    const int tokens = seq_len;
    if (tokens < 1 || position < 0 || position + tokens > max_seq_len_) die("forward: position/seq_len outside the cache");
    int cached = 0;
    pa(pa_seq_length(pool_, seq_, &cached));
    if (position == 0 && cached > 0) {  // a new conversation: hand the blocks back and start over
      pa(pa_seq_free(pool_, seq_));
      pa(pa_seq_create(pool_, &seq_));
      cached = 0;
    }
    if (position != cached) die("forward: position must equal the number of cached tokens");
    pa(pa_seq_reserve(pool_, seq_, position + tokens));
    const int32_t id = seq_, n_new = tokens;
    pa(pa_batch_set(pool_, &id, &n_new, 1, nullptr));
    const float scale = 0.125f;  // 1 / sqrt(64), src/runtime/attention.cu:318
    if (tokens == 1) {
      if (strided_) {
        pa(pa_block_step(pool_, nullptr, 0, kLayers, &all_att_, &all_ffn_, input, output, cos_table_, sin_table_, scale,
                         nullptr));
      } else {
        const __nv_bfloat16* cur = input;
        for (int l = 0; l < kLayers; l++) {
          __nv_bfloat16* out = l == kLayers - 1 ? output : ping_ + (size_t)(l & 1) * 8 * kHidden;
          pa(pa_block_step(pool_, nullptr, l, l + 1, &att_[l], &ffn_[l], cur, out, cos_table_, sin_table_, scale, nullptr));
          cur = out;
        }
      }
    } else {
      reserve_prompt(tokens);
      const size_t r = (size_t)rows_cap_ * kHidden;
      __nv_bfloat16 *normalized = rows_, *q_rot = rows_ + r, *attn = rows_ + 2 * r, *mid = rows_ + 3 * r;
      __nv_bfloat16* pp[2] = {rows_ + 4 * r, rows_ + 5 * r};
      __nv_bfloat16* scratch = rows_ + 6 * r;
      const __nv_bfloat16* cur = input;
      for (int l = 0; l < kLayers; l++) {
        const __nv_bfloat16* p = packed_ + (size_t)l * kPackedLayer;
        __nv_bfloat16* out = l == kLayers - 1 ? output : pp[l & 1];
        pa(pa_rmsnorm(cur, att_[l].input_norm, normalized, tokens, kHidden, 1e-5f, nullptr));
        pa(pa_qkv_project_append(pool_, l, normalized, p + kOffQ, p + kOffK, p + kOffV, cos_table_, sin_table_, q_rot, kHidden,
                                 nullptr));
        pa(pa_prefill(pool_, l, q_rot, attn, nullptr, scale, nullptr));
        pa(pa_out_project_rows(pool_, attn, p + kOffO, cur, mid, tokens, kHidden, kHidden, nullptr));
        pa_ffn_weights f = ffn_[l];
        f.gate = p + kOffG;
        f.up = p + kOffU;
        f.down = p + kOffD;
        pa(pa_ffn_rows(pool_, &f, 0, mid, scratch, out, tokens, /*add_residual=*/1, nullptr));
        cur = out;
      }
    }
    pa(pa_pool_check(pool_, nullptr));  // synchronises: `output` is complete
  }

  // [8, max_seq_len, 64] of one layer, the view the reference keeps as its cache (rows beyond the
  // cached tokens are zero); refreshed from the paged cache on every call.
  const __nv_bfloat16* get_key_cache(int layer_idx) const {
    refresh_views(layer_idx);
    return key_view_;
  }
  const __nv_bfloat16* get_value_cache(int layer_idx) const {
    refresh_views(layer_idx);
    return value_view_;
  }

 private:
  static constexpr int kLayers = llama::NUM_LAYERS, kHidden = llama::HIDDEN_SIZE, kInter = llama::INTERMEDIATE_SIZE;
  static constexpr size_t kOffQ = 0, kOffK = kOffQ + (size_t)kHidden * kHidden, kOffV = kOffK + (size_t)kHidden * 512,
                          kOffO = kOffV + (size_t)kHidden * 512, kOffG = kOffO + (size_t)kHidden * kHidden,
                          kOffU = kOffG + (size_t)kHidden * kInter, kOffD = kOffU + (size_t)kHidden * kInter,
                          kPackedLayer = kOffD + (size_t)kInter * kHidden;
  static void die(const char* what) {
    fprintf(stderr, "runtime::Transformer: %s\n", what);
    exit(EXIT_FAILURE);
  }
  static void pa(int rc) {
    if (rc != PA_OK) die(pa_last_error());
  }
  static void cuda(cudaError_t e) {
    if (e != cudaSuccess) die(cudaGetErrorString(e));
  }
  void refresh_views(int layer) const {
    if (layer < 0 || layer >= kLayers) die("cache accessor: layer out of range");
    const size_t cache = (size_t)8 * max_seq_len_ * 64 * sizeof(__nv_bfloat16);
    if (!key_view_) {
      cuda(cudaMalloc(&key_view_, cache));
      cuda(cudaMalloc(&value_view_, cache));
    }
    cuda(cudaMemset(key_view_, 0, cache));
    cuda(cudaMemset(value_view_, 0, cache));
    int cached = 0;
    pa(pa_seq_length(pool_, seq_, &cached));
    if (cached > 0) pa(pa_gather_kv(pool_, layer, seq_, key_view_, value_view_, max_seq_len_, nullptr));
    cuda(cudaStreamSynchronize(nullptr));
  }

  float* cos_table_;
  float* sin_table_;
  int max_seq_len_;
  pa_pool* pool_ = nullptr;
  int seq_ = -1;
  pa_attention_weights att_[llama::NUM_LAYERS], all_att_;
  pa_ffn_weights ffn_[llama::NUM_LAYERS], all_ffn_;
  bool strided_ = false;
  __nv_bfloat16* ping_ = nullptr;
  __nv_bfloat16* packed_ = nullptr;
  __nv_bfloat16* rows_ = nullptr;
  int rows_cap_ = 0;
  mutable __nv_bfloat16 *key_view_ = nullptr, *value_view_ = nullptr;
};

}  // namespace runtime
