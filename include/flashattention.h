#pragma once
// Drop-in for the reference's src/kernels/flashattention/flashattention.h
// (lines 49-76): same namespace, enum, struct field order and defaults, same
// free function, defined out of line in libpaged_attention.so (csrc/compat_cxx.cu)
// under the same mangled name.  A translation unit that includes the reference's
// header or this one links libpaged_attention.so instead of the reference's
// flashattention.cu.
//
// Behaviour on failure follows the reference: a CUDA error prints and exits
// (its CUDA_CHECK, flashattention.h:33-41), an unsupported head size aborts
// (flashattention.cu:454-459).
#include <cstdio>
#include <cstdlib>
#include <cuda_fp16.h>
#include <cuda_runtime.h>


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

// Defined in libpaged_attention.so with this exact C++ signature, so a translation unit compiled
// against the reference's own header links to it just the same.
void launch_flash_attention(const FlashAttentionParams &params);

}  // namespace transformer
