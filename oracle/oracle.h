/* TEST INFRASTRUCTURE — CPU restatement of the reference's KV-cache attention
 * path.  Only tests, the smoke check and the bench's CPU-baseline leg may link
 * or load this; the product never does.
 *
 * Parity status: the reference ships no golden vectors for this path (its
 * flash-attention test file is empty, its RoPE test contradicts its kernel),
 * so this oracle is pinned against outputs of the reference's own kernels run
 * on a B200 (fixtures under tests/golden/, made by tests/golden/make_golden.py)
 * and, in the GPU tests, against the reference kernels directly.
 *
 * All bf16 tensors are passed as uint16_t bit patterns.
 */
#ifndef ORACLE_H
#define ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_HEAD_DIM 64
#define ORC_ROTARY_DIM 32
#define ORC_BLOCK_TOKENS 16

uint16_t orc_f32_to_bf16(float x);
float orc_bf16_to_f32(uint16_t x);

/* fp32 cos/sin tables [seq_len][32] with Llama-3 frequency scaling.
 * Follows LlamaRuntime::build_rope_tables, src/runtime/llama_runtime.cu:320-451. */
void orc_build_rope_tables(float* cos_table, float* sin_table, int seq_len);

/* Half-split RoPE (pairs (i, i+32)), fp32 math, round-to-nearest-even to bf16.
 * Follows rope_q_kernel / rope_k_kernel, src/kernels/rope/rope.cu:23-210.
 * in  : [tokens][heads][64]
 * out : head-major [heads][tokens][64] when out_token_major == 0 (what the
 *       reference writes), token-major [tokens][heads][64] otherwise.
 * y0_variant selects how  y0 = x0*c - x1*s  is rounded (the compiler decides
 * this for the reference kernel; the GPU tests pin which one it is):
 *   0: two rounded products, rounded difference
 *   1: fmaf(x0, c, -(x1*s))
 *   2: fmaf(-x1, s, x0*c)
 * y1 is always fmaf(x0, s, x1*c). */
void orc_rope(const uint16_t* in, uint16_t* out, const float* cos_table,
              const float* sin_table, int tokens, int heads,
              int position_offset, int y0_variant, int out_token_major);

/* V layout change [tokens][8][64] -> [8][tokens][64], bit copy.
 * Follows transpose_v_kernel, src/kernels/rope/rope.cu:211-262. */
void orc_transpose_v(const uint16_t* v_in, uint16_t* v_out, int tokens,
                     int kv_heads);

/* Contiguous-cache append of one tensor: flash [kv_heads][tokens][64] into
 * cache [kv_heads][max_seq_len][64] at rows position..position+tokens-1.
 * Follows the copy loop in Attention::forward, src/runtime/attention.cu:239-262. */
void orc_append_contig(uint16_t* cache, const uint16_t* flash, int kv_heads,
                       int max_seq_len, int position, int tokens);

/* Paged placement model.  The LOGICAL pool is
 *   [num_blocks][kv_heads][2 (K,V)][16 slots][64]
 * and logical position p of a sequence lives in block table[p/16], slot p%16.
 * (The reference has no paged cache; this states where the same 64 values the
 * reference stores at cache[h][p][:] must land.) */
void orc_paged_append(uint16_t* pool, int kv_heads, const int32_t* table,
                      const uint16_t* k_flash, const uint16_t* v_flash,
                      int position, int tokens);
void orc_paged_gather(const uint16_t* pool, int kv_heads, const int32_t* table,
                      int length, uint16_t* k_out, uint16_t* v_out,
                      int out_stride_tokens);

/* Naive GQA attention in fp32 from bf16 inputs.
 * Semantics of flash_attention_fat_kernel, src/kernels/flashattention/flashattention.cu:98-376:
 *   score = scale * dot(q, k); column j visible to query row i iff
 *   !causal || j <= (kv_seq_len - q_seq_len) + i; softmax; O = P V / sum;
 *   LSE = natural-log-sum-exp of the scaled scores (:363-374).
 * Q [q_heads][q_seq_len][64], K/V [kv_heads][kv_stride][64] (first kv_seq_len
 * rows valid), O fp32 [q_heads][q_seq_len][64], LSE fp32 [q_heads][q_seq_len]
 * (may be NULL).  round_p_bf16 != 0 rounds each probability to bf16 before the
 * PV product while summing the unrounded one, as the reference kernel does
 * (:300-336); 0 is the plain fp32 definition. */
void orc_attention(const uint16_t* Q, const uint16_t* K, const uint16_t* V,
                   float* O, float* LSE, int q_heads, int kv_heads,
                   int q_seq_len, int kv_seq_len, int kv_stride, float scale,
                   int causal, int round_p_bf16);

/* Single-token decode over a LOGICAL paged pool through a block table
 * (gather + the same attention at q_seq_len = 1).  q [q_heads][64];
 * out fp32 [q_heads][64]; lse [q_heads] (may be NULL).  Token range
 * [tok_begin, tok_end) lets a caller compute a split-KV partial. */
void orc_decode_paged(const uint16_t* q, const uint16_t* pool, int q_heads,
                      int kv_heads, const int32_t* table, int tok_begin,
                      int tok_end, float scale, float* out, float* lse);

/* Exact merge of softmax partials over disjoint key ranges:
 *   lse = log(sum_p exp(lse_p)),  O = sum_p exp(lse_p - lse) O_p.
 * O_parts [n_parts][rows][64] (each already normalised by its own sum),
 * lse_parts [n_parts][rows]; a part with lse = -inf contributes nothing. */
void orc_lse_merge(const float* O_parts, const float* lse_parts, int n_parts,
                   int rows, float* O, float* lse);

/* [32][tokens][64] -> [tokens][2048].  Follows flash_output_layout_kernel,
 * src/runtime/layout.cu:11-42. */
void orc_output_layout_f32(const float* in, float* out, int heads, int tokens);
void orc_output_layout_bf16(const uint16_t* in, uint16_t* out, int heads,
                            int tokens);

/* C = A B as the reference's projection GEMMs define it
 * (src/kernels/gemm/gemm_2048x512.cu:82-290, gemm_2048x2048.cu:95-331: A [M, K]
 * row-major bf16, B [K, N] row-major bf16, fp32 tensor-core accumulation, C bf16
 * by round-to-nearest).  Here every dot product is accumulated in double and
 * rounded once, so a GPU result may differ by one bf16 ulp where its fp32
 * accumulation order lands on the other side of a rounding boundary. */
void orc_gemm_bf16(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K);

/* RMSNorm of rows of `hidden` bf16 values: y = bf16((x * r) * w), r = 1/sqrt(mean(x^2) + eps).
 * Follows rmsnorm_fwd_kernel, src/kernels/rmsnorm/rmsnorm.cu:51-110, including the order in which
 * its 256 threads add up the squares. */
void orc_rmsnorm(const uint16_t* x, const uint16_t* w, uint16_t* y, int rows, int hidden, float eps);
/* SiLU(gate) * up on bf16 values, fp32 arithmetic, bf16 result (src/kernels/silu/silu_8192.cu:55-100). */
void orc_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, long long n);

int orc_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
