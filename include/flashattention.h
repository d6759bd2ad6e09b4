#pragma once
// Drop-in for the reference's src/kernels/flashattention/flashattention.h
// (lines 49-76): same namespace, enum, struct field order and defaults, same
// free function.  A translation unit that included the reference's header
// compiles against this one unchanged and links libpaged_attention.so instead
// of the reference's flashattention.cu.
//
// Behaviour on failure follows the reference: a CUDA error prints and exits
// (its CUDA_CHECK, flashattention.h:33-41), an unsupported head size aborts
// (flashattention.cu:454-459).
#include <cstdio>
#include <cstdlib>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "legacy_kernels.h"
#include "paged_attention.h"

#ifndef CUDA_CHECK
#define CUDA_CHECK(call)                                                       \
  do {                                                                         \
    cudaError_t err = (call);                                                  \
    if (err != cudaSuccess) {                                                  \
      fprintf(stderr, "CUDA error at %s:%d: %s\n", __FILE__, __LINE__,         \
              cudaGetErrorString(err));                                        \
      exit(EXIT_FAILURE);                                                      \
    }                                                                          \
  } while (0)
#endif

namespace transformer {

// FP16 == 0 so that a zero-initialised params struct keeps its old meaning.
enum class DType { FP16 = 0, BF16 = 1 };

struct FlashAttentionParams {
  const void *Q;
  const void *K;
  const void *V;
  void *O;
  float *L;          // [B*H, S] log-sum-exp (fp32), may be nullptr
  int batch_size;
  int num_heads;     // query heads
  int num_kv_heads;  // 0 (or == num_heads) means MHA
  int q_seq_len;
  int kv_seq_len;    // valid tokens in the cache
  int kv_stride;     // tokens between KV heads in memory
  int d_head;
  float scale;
  bool causal;
  DType dtype;
  cudaStream_t stream;
};

inline void launch_flash_attention(const FlashAttentionParams &params) {
  lt_flash_attention_params p;
  p.Q = params.Q;
  p.K = params.K;
  p.V = params.V;
  p.O = params.O;
  p.L = params.L;
  p.batch_size = params.batch_size;
  p.num_heads = params.num_heads;
  p.num_kv_heads = params.num_kv_heads;
  p.q_seq_len = params.q_seq_len;
  p.kv_seq_len = params.kv_seq_len;
  p.kv_stride = params.kv_stride;
  p.d_head = params.d_head;
  p.scale = params.scale;
  p.causal = params.causal ? 1 : 0;
  p.dtype = static_cast<int>(params.dtype);
  p.stream = params.stream;
  const int rc = lt_launch_flash_attention(&p);
  if (rc == PA_OK) return;
  if (params.d_head != 64 && params.d_head != 128) {
    fprintf(stderr, "flash_attention: unsupported d_head=%d (supported: 64, 128)\n", params.d_head);
    abort();
  }
  fprintf(stderr, "flash_attention: %s\n", pa_last_error());
  exit(EXIT_FAILURE);
}

}  // namespace transformer
