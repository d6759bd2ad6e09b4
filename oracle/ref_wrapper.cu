// TEST INFRASTRUCTURE — not part of the product.
//
// extern "C" handles onto the reference's own, unmodified CUDA entry points
// for the KV-cache attention path, so tests and the bench's reference arm can
// drive them through ctypes.  The reference sources are compiled where they
// lie (see oracle/Makefile); nothing from them is copied into this file.
//
// What each handle calls in the reference:
//   ref_rope_qkv            -> launch_rope_qkv            (src/kernels/rope/rope.hpp:52-63)
//   ref_flash_attention     -> transformer::launch_flash_attention
//                              (src/kernels/flashattention/flashattention.h:54-76)
//   ref_flash_output_layout -> launch_flash_output_layout (src/runtime/layout.hpp:5-9)
//   ref_residual_add        -> transformer::residual_add  (src/kernels/residual_add/residual_add.hpp)
//   ref_rmsnorm             -> rmsnorm_launch<2048>       (src/kernels/rmsnorm/rmsnorm.hpp:6-14)
//   ref_gemm                -> launch_gemm_2048x2048 / _2048x512 / _2048x8192 / _8192x2048
//                              (src/kernels/gemm/*.hpp), chosen by shape as Attention::forward and
//                              FeedForward::forward choose them
//   ref_silu_mul            -> launch_silu_mul            (src/kernels/silu/silu_8192.hpp)
//   ref_argmax              -> launch_argmax              (src/kernels/sampling/argmax_128256.hpp)
//   ref_embedding           -> launch_embedding           (src/kernels/embedding/embedding.hpp)
//   ref_append_*            -> the append the reference performs inline in
//                              Attention::forward (src/runtime/attention.cu:239-262):
//                              2*8*tokens device-to-device copies of 128 bytes.
//                              That loop is not a callable function in the
//                              reference, so it is restated here twice: literally
//                              (one cudaMemcpy per 128 bytes) and as one strided
//                              cudaMemcpy2DAsync per head, which moves the same bytes.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "flashattention.h"
#include "gemm_2048x2048.hpp"
#include "argmax_128256.hpp"
#include "embedding.hpp"
#include "gemm_2048x128256.hpp"
#include "gemm_2048x512.hpp"
#include "gemm_2048x8192.hpp"
#include "gemm_8192x2048.hpp"
#include "layout.hpp"
#include "residual_add.hpp"
#include "rmsnorm.hpp"
#include "rope.hpp"
#include "silu_8192.hpp"

extern "C" {

void ref_rope_qkv(const void* q_in, void* q_out, const void* k_in, void* k_out,
                  const void* v_in, void* v_out, float* cos_table,
                  float* sin_table, int tokens, int position_offset) {
  launch_rope_qkv((const __nv_bfloat16*)q_in, (__nv_bfloat16*)q_out,
                  (const __nv_bfloat16*)k_in, (__nv_bfloat16*)k_out,
                  (const __nv_bfloat16*)v_in, (__nv_bfloat16*)v_out, cos_table,
                  sin_table, tokens, position_offset);
}

// Field-by-field fill of the reference's launch descriptor, exactly as
// Attention::forward does it (src/runtime/attention.cu:278-328).
void ref_flash_attention(const void* Q, const void* K, const void* V, void* O,
                         float* L, int batch, int heads, int kv_heads,
                         int q_seq_len, int kv_seq_len, int kv_stride,
                         float scale, int causal, void* stream) {
  transformer::FlashAttentionParams p{};
  p.Q = Q;
  p.K = K;
  p.V = V;
  p.O = O;
  p.L = L;
  p.batch_size = batch;
  p.num_heads = heads;
  p.num_kv_heads = kv_heads;
  p.q_seq_len = q_seq_len;
  p.kv_seq_len = kv_seq_len;
  p.kv_stride = kv_stride;
  p.d_head = 64;
  p.scale = scale;
  p.causal = causal != 0;
  p.dtype = transformer::DType::BF16;
  p.stream = (cudaStream_t)stream;
  transformer::launch_flash_attention(p);
}

// The GEMMs as Attention::forward (src/runtime/attention.cu:138-191) and FeedForward::forward
// (src/runtime/ffn.cu:84-127) call them: K = 2048, N = 2048 -> launch_gemm_2048x2048; N = 512 ->
// launch_gemm_2048x512; N = 8192 -> launch_gemm_2048x8192; K = 8192, N = 2048 -> launch_gemm_8192x2048.
int ref_gemm(const void* A, const void* B, void* C, int M, int N, int K) {
  const __nv_bfloat16* a = (const __nv_bfloat16*)A;
  const __nv_bfloat16* b = (const __nv_bfloat16*)B;
  __nv_bfloat16* c = (__nv_bfloat16*)C;
  if (K == 8192 && N == 2048)
    launch_gemm_8192x2048(a, b, c, M, N, K);
  else if (N == 2048)
    launch_gemm_2048x2048(a, b, c, M, N, K);
  else if (N == 512)
    launch_gemm_2048x512(a, b, c, M, N, K);
  else if (N == 8192)
    launch_gemm_2048x8192(a, b, c, M, N, K);
  else if (N == 128256)
    launch_gemm_2048x128256(a, b, c, M, N, K);  // the language-model head (src/runtime/llama_runtime.cu:895-902)
  else
    return 1;
  return (int)cudaGetLastError();
}

// token = argmax over the 128256 bf16 logits of one row (src/runtime/llama_runtime.cu:913-917).
void ref_argmax(const void* logits, int* token) { launch_argmax((const __nv_bfloat16*)logits, token, 0); }

// out[r, :] = table[tokens[r], :], rows of 2048 (src/runtime/llama_runtime.cu:846-851).
void ref_embedding(const int* tokens, const void* table, void* out, int rows) {
  launch_embedding(tokens, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, rows, 0);
}

// out = SiLU(gate) * up over rows x 8192 elements (src/runtime/ffn.cu:112-118).
void ref_silu_mul(const void* gate, const void* up, void* out, int rows) {
  launch_silu_mul((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (__nv_bfloat16*)out, rows, 8192);
}

// out = a + b as TransformerBlock::forward adds the attention output to the block input
// (src/runtime/transformer_block.cu:76-81).  The reference throws on bad arguments.
int ref_residual_add(const void* a, const void* b, void* out, long long n) {
  try {
    transformer::residual_add((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, (int64_t)n);
  } catch (...) {
    return 1;
  }
  return 0;
}

// RMSNorm over rows of 2048 as Attention::forward calls it (src/runtime/attention.cu:123).
void ref_rmsnorm(const void* in, const void* weight, void* out, int rows, float eps) {
  rmsnorm_launch<2048>((const __nv_bfloat16*)in, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, rows, eps, 256);
}

void ref_flash_output_layout(const void* in, void* out, int tokens) {
  launch_flash_output_layout((const __nv_bfloat16*)in, (__nv_bfloat16*)out,
                             tokens);
}

// Literal restatement of the append loop: k_flash/v_flash are [8, tokens, 64],
// the caches are [8, max_seq_len, 64].
int ref_append_memcpy_loop(void* key_cache, void* value_cache,
                           const void* k_flash, const void* v_flash,
                           int max_seq_len, int position, int tokens) {
  __nv_bfloat16* kc = (__nv_bfloat16*)key_cache;
  __nv_bfloat16* vc = (__nv_bfloat16*)value_cache;
  const __nv_bfloat16* kf = (const __nv_bfloat16*)k_flash;
  const __nv_bfloat16* vf = (const __nv_bfloat16*)v_flash;
  for (int h = 0; h < 8; h++) {
    for (int t = 0; t < tokens; t++) {
      cudaError_t e1 = cudaMemcpy(
          kc + (size_t)h * max_seq_len * 64 + (size_t)(position + t) * 64,
          kf + (size_t)h * tokens * 64 + (size_t)t * 64,
          64 * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice);
      cudaError_t e2 = cudaMemcpy(
          vc + (size_t)h * max_seq_len * 64 + (size_t)(position + t) * 64,
          vf + (size_t)h * tokens * 64 + (size_t)t * 64,
          64 * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice);
      if (e1 != cudaSuccess || e2 != cudaSuccess) return 1;
    }
  }
  return 0;
}

// Same bytes, one strided copy per head and tensor (16 API calls instead of
// 16*tokens), so that a kernel-to-kernel comparison is not drowned by the
// reference's host loop.
int ref_append_strided(void* key_cache, void* value_cache, const void* k_flash,
                       const void* v_flash, int max_seq_len, int position,
                       int tokens, void* stream) {
  __nv_bfloat16* kc = (__nv_bfloat16*)key_cache;
  __nv_bfloat16* vc = (__nv_bfloat16*)value_cache;
  const __nv_bfloat16* kf = (const __nv_bfloat16*)k_flash;
  const __nv_bfloat16* vf = (const __nv_bfloat16*)v_flash;
  size_t bytes = (size_t)tokens * 64 * sizeof(__nv_bfloat16);
  for (int h = 0; h < 8; h++) {
    cudaError_t e1 = cudaMemcpyAsync(
        kc + (size_t)h * max_seq_len * 64 + (size_t)position * 64,
        kf + (size_t)h * tokens * 64, bytes, cudaMemcpyDeviceToDevice,
        (cudaStream_t)stream);
    cudaError_t e2 = cudaMemcpyAsync(
        vc + (size_t)h * max_seq_len * 64 + (size_t)position * 64,
        vf + (size_t)h * tokens * 64, bytes, cudaMemcpyDeviceToDevice,
        (cudaStream_t)stream);
    if (e1 != cudaSuccess || e2 != cudaSuccess) return 1;
  }
  return 0;
}

}  // extern "C"
