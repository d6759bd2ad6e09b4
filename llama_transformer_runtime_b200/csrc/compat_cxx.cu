// The reference's three kernel launchers as C++ symbols of this library:
//   transformer::launch_flash_attention(const FlashAttentionParams&)
//       src/kernels/flashattention/flashattention.h:76, defined in flashattention.cu:436-461
//   launch_rope_qkv(...)            src/kernels/rope/rope.hpp:52-63, defined in rope.cu:267-359
//   launch_flash_output_layout(...) src/runtime/layout.hpp:5-9, defined in layout.cu:43-76
// Same names, namespaces, argument types and struct layout, hence the same mangled names: an
// object file compiled against the reference's own headers (src/runtime/attention.cu includes them
// by relative path) links against libpaged_attention.so in place of the reference's
// flashattention.cu, rope.cu and layout.cu, with no source change.  Each forwards to the C entry
// of legacy_kernels.h and reproduces the reference's behaviour on failure: print and exit; abort
// on a head size that is neither 64 nor 128 (flashattention.cu:454-459).
#include <cstdio>
#include <cstdlib>

#include "../../include/flashattention.h"
#include "../../include/layout.hpp"
#include "../../include/legacy_kernels.h"
#include "../../include/paged_attention.h"
#include "../../include/rope.hpp"

namespace transformer {

void launch_flash_attention(const FlashAttentionParams& params) {
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

// Like the reference's launcher (rope.cu:305-358) it returns with the results complete: default
// stream, device synchronised.
void launch_rope_qkv(const __nv_bfloat16* q_in, __nv_bfloat16* q_out, const __nv_bfloat16* k_in,
                     __nv_bfloat16* k_out, const __nv_bfloat16* v_in, __nv_bfloat16* v_out, float* cos_table,
                     float* sin_table, int tokens, int position_offset) {
  const int rc = lt_launch_rope_qkv(q_in, q_out, k_in, k_out, v_in, v_out, cos_table, sin_table, tokens,
                                    position_offset, nullptr);
  if (rc != PA_OK) {
    printf("CUDA Error %s:%d : %s\n", __FILE__, __LINE__, pa_last_error());
    exit(EXIT_FAILURE);
  }
  CUDA_CHECK(cudaDeviceSynchronize());
}

void launch_flash_output_layout(const __nv_bfloat16* input, __nv_bfloat16* output, int tokens) {
  if (lt_launch_flash_output_layout(input, output, tokens, nullptr) != PA_OK) {
    printf("CUDA Error: %s\n", pa_last_error());
    exit(EXIT_FAILURE);
  }
}
