/* C-ABI behind the drop-in C++ headers flashattention.h, rope.hpp and
 * layout.hpp of this directory: the reference's three kernel launchers for the
 * attention path, with the reference's data layouts (contiguous K/V cache,
 * head-major Q/O), served by the sm_100a kernels of this library.
 *
 *   lt_launch_flash_attention     transformer::launch_flash_attention,
 *                                 src/kernels/flashattention/flashattention.h:54-76
 *   lt_launch_rope_qkv            launch_rope_qkv, src/kernels/rope/rope.hpp:52-63
 *   lt_launch_flash_output_layout launch_flash_output_layout, src/runtime/layout.hpp:5-9
 *
 * Each returns a status (0 = ok, codes of paged_attention.h) and the message is
 * available from pa_last_error(); the C++ shims reproduce the reference's
 * behaviour on failure (print and exit, abort on an unsupported head size).
 *
 * lt_launch_flash_attention keeps a private paged pool per device: the
 * contiguous K/V it is handed are first repacked into the paged layout (one
 * extra pass over the cache, and an allocation whenever a larger cache than
 * before arrives), then the paged decode (q_seq_len == 1) or prefill kernel
 * runs.  Calls on one device share that pool: a call waits (on the device,
 * through an event) for the previous call's work even when it is given
 * another stream, and growing the pool synchronises the device.  It exists so
 * that existing callers keep working; callers that care about speed hold a
 * pa_pool themselves and never pay the repack.
 * Supported: bf16, d_head 64, num_heads == 4 * num_kv_heads, num_kv_heads in
 * {1, 2, 4, 8}; anything else returns PA_ERR_UNSUPPORTED. */
#ifndef LEGACY_KERNELS_H
#define LEGACY_KERNELS_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  const void* Q;   /* [batch*num_heads][q_seq_len][d_head] */
  const void* K;   /* [batch*num_kv_heads][kv_stride][d_head], first kv_seq_len rows valid */
  const void* V;
  void* O;         /* like Q */
  float* L;        /* [batch*num_heads][q_seq_len] natural-log-sum-exp, may be NULL */
  int batch_size, num_heads, num_kv_heads; /* num_kv_heads == 0 means num_heads */
  int q_seq_len, kv_seq_len, kv_stride, d_head;
  float scale;
  int causal;      /* query row i sees keys 0 .. (kv_seq_len - q_seq_len) + i */
  int dtype;       /* 0 = fp16, 1 = bf16 */
  void* stream;
} lt_flash_attention_params;

int lt_launch_flash_attention(const lt_flash_attention_params* params);

/* q_in [tokens][32][64] -> q_out [32][tokens][64] (RoPE), k likewise with 8
 * heads, v_in [tokens][8][64] -> v_out [8][tokens][64] (copy). */
int lt_launch_rope_qkv(const void* q_in, void* q_out, const void* k_in, void* k_out,
                       const void* v_in, void* v_out, const float* cos_table,
                       const float* sin_table, int tokens, int position_offset, void* stream);

/* in [32][tokens][64] -> out [tokens][2048] */
int lt_launch_flash_output_layout(const void* in, void* out, int tokens, void* stream);

#ifdef __cplusplus
}
#endif
#endif
