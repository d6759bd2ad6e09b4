#pragma once
// llama::LlamaWeights for the drop-in headers: the structs and constants of the reference's
// src/runtime/weights.hpp:7-64 under the same names, so that code written against it (and the
// reference's own weights.cu, which defines load_weights / free_weights) compiles unchanged.
#include <cstddef>
#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace llama {

constexpr int NUM_LAYERS = 16;
constexpr int HIDDEN_SIZE = 2048;
constexpr int INTERMEDIATE_SIZE = 8192;
constexpr int VOCAB_SIZE = 128256;
constexpr int NUM_ATTENTION_HEADS = 32;
constexpr int NUM_KV_HEADS = 8;
constexpr int HEAD_DIM = 64;

struct TransformerLayerWeights {
  __nv_bfloat16* input_layernorm = nullptr;           // [2048]
  __nv_bfloat16* q_proj = nullptr;                    // [2048, 2048] row-major, x @ W
  __nv_bfloat16* k_proj = nullptr;                    // [2048, 512]
  __nv_bfloat16* v_proj = nullptr;                    // [2048, 512]
  __nv_bfloat16* o_proj = nullptr;                    // [2048, 2048]
  __nv_bfloat16* post_attention_layernorm = nullptr;  // [2048]
  __nv_bfloat16* gate_proj = nullptr;                 // [2048, 8192]
  __nv_bfloat16* up_proj = nullptr;                   // [2048, 8192]
  __nv_bfloat16* down_proj = nullptr;                 // [8192, 2048]
};

struct LlamaWeights {
  __nv_bfloat16* embed_tokens = nullptr;  // [VOCAB_SIZE, HIDDEN_SIZE]
  TransformerLayerWeights layers[NUM_LAYERS];
  __nv_bfloat16* final_norm = nullptr;  // [HIDDEN_SIZE]
  __nv_bfloat16* lm_head = nullptr;     // [HIDDEN_SIZE, VOCAB_SIZE]
};

// defined by the reference's src/runtime/weights.cu
void load_weights(const char* weights_path, LlamaWeights& weights);
void free_weights(LlamaWeights& weights);

}  // namespace llama
