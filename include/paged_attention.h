/* C-ABI of the B200 (sm_100a) paged KV-cache attention library.
 *
 * Plain C, plain pointers and sizes: this is the boundary a host binds
 * (C++, ctypes, cgo, JNI ...).  Fixed instantiation, as in the reference
 * (src/kernels/rope/rope.hpp:11-17): 64-wide heads, bf16, 4 query heads per
 * KV head, 16-token cache blocks.  bf16 tensors are passed as `void*`.
 *
 * Every entry returns a status (PA_OK == 0) and never exits or throws;
 * pa_last_error() gives the message of the calling thread's last failure.
 * Kernel entries are asynchronous on the stream they are given and do no
 * device synchronisation and no allocation: device memory is allocated only by
 * the set-up calls (pa_pool_create, pa_exchange_create,
 * pa_gather_create).  A pool's host-side calls are not
 * thread-safe per pool; calls on one pool that overlap on the GPU share its
 * split-KV workspace and therefore must be ordered on one stream.
 *
 * Which reference interface each group replaces:
 *   pool / sequence / block-table calls
 *       src/pagedattention/paged_attention.hpp (declared, 0 bytes) and the
 *       contiguous cache owned by runtime::Attention, src/runtime/attention.hpp:47-54,
 *       src/runtime/attention.cu:74-98.
 *   pa_append
 *       launch_rope_qkv, src/kernels/rope/rope.hpp:52-63, plus the append loop
 *       of Attention::forward, src/runtime/attention.cu:239-262.
 *   pa_decode
 *       transformer::launch_flash_attention with q_seq_len == 1,
 *       src/kernels/flashattention/flashattention.h:54-76 as called at
 *       src/runtime/attention.cu:278-334, plus launch_flash_output_layout,
 *       src/runtime/layout.hpp:5-9.
 *   pa_prefill
 *       the same pair for q_seq_len > 1 (causal, kv_len = position + tokens,
 *       src/runtime/attention.cu:303-313).
 *   pa_gather_kv
 *       Attention::get_key_cache / get_value_cache, src/runtime/attention.hpp:30-31
 *       (hands back the [8, L, 64] view the reference keeps as its cache).
 *   pa_build_rope_tables
 *       LlamaRuntime::build_rope_tables, src/runtime/llama_runtime.cu:320-451.
 */
#ifndef PAGED_ATTENTION_H
#define PAGED_ATTENTION_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PA_OK 0
#define PA_ERR_INVALID_ARG 1
#define PA_ERR_OUT_OF_BLOCKS 2
#define PA_ERR_UNSUPPORTED 3
#define PA_ERR_CUDA 4
#define PA_ERR_TIMEOUT 5 /* a bounded device-side wait gave up */
#define PA_ERR_STATE 6

#define PA_HEAD_DIM 64
#define PA_GROUP 4         /* query heads per KV head */
#define PA_BLOCK_TOKENS 16 /* tokens per cache block */
#define PA_TILE_BYTES 2048 /* one (block, head) K or V tile */

typedef struct pa_pool pa_pool;

const char* pa_last_error(void);

/* ---- pool ----------------------------------------------------------------
 * Device storage for `num_layers` caches of `num_blocks` blocks holding
 * `kv_heads` KV heads each (8 for the whole model, 8/n when heads are sharded
 * over n GPUs), the host free list, up to `max_seqs` block tables of
 * `max_blocks_per_seq` entries (host + device mirror) and the split-KV
 * workspace.  All device memory is allocated here, none per call. */
int pa_pool_create(pa_pool** out, int device, int num_layers, int num_blocks,
                   int kv_heads, int max_seqs, int max_blocks_per_seq);
int pa_pool_destroy(pa_pool* pool);
int pa_pool_free_blocks(const pa_pool* pool, int* n_free);
/* Order in which free blocks are handed out (order[0] first).  Only valid
 * while no block is in use; lets a seeded permutation reproduce a shuffled or
 * fragmented table exactly. */
int pa_pool_set_free_order(pa_pool* pool, const int32_t* order, int n);
/* Raw device storage of one layer's cache (for inspection by tests) and its
 * size in bytes.  Physical layout: tile(block, head, kv) at byte offset
 * ((block * kv_heads + head) * 2 + kv) * 2048, kv = 0 for K, 1 for V; inside a
 * tile token slot r (0..15) is a 128-byte row and its 16-byte chunk c (0..7)
 * sits at chunk position c ^ (r & 7) — the 128-byte shared-memory swizzle, so
 * a tile copied verbatim is bank-conflict free for ldmatrix and is the
 * canonical K-major operand layout of tcgen05.mma. */
int pa_pool_layer_storage(const pa_pool* pool, int layer, void** dev_ptr,
                          uint64_t* bytes);

/* ---- sequences and block tables (host) ------------------------------------ */
int pa_seq_create(pa_pool* pool, int* seq_id);
int pa_seq_free(pa_pool* pool, int seq_id);
/* Grow the sequence to `new_len` tokens, taking blocks from the free list as
 * needed.  All or nothing: PA_ERR_OUT_OF_BLOCKS leaves the sequence unchanged.
 * Never shrinks; an unchanged length is a no-op. */
int pa_seq_reserve(pa_pool* pool, int seq_id, int new_len);
int pa_seq_length(const pa_pool* pool, int seq_id, int* len);
/* Host view of the table: entry i holds the block of positions [16i, 16i+16).
 * The pointer stays valid until the sequence is freed. */
int pa_seq_block_table(const pa_pool* pool, int seq_id, const int32_t** table,
                       int* n_blocks);

/* ---- batch -----------------------------------------------------------------
 * Names the sequences the following pa_append / pa_decode / pa_prefill calls
 * work on, uploads pending block-table changes and the batch descriptor on
 * `stream`.  Row i of the per-sequence tensors belongs to seq_ids[i].
 * new_tokens[i] (NULL means 1 each) is how many tokens sequence i appends in
 * this step: they occupy its last new_tokens[i] positions, i.e. the caller has
 * already reserved the new length.  Token rows of q_in/k_in/v_in are the
 * sequences' new tokens concatenated in batch order. */
int pa_batch_set(pa_pool* pool, const int32_t* seq_ids, const int32_t* new_tokens,
                 int n_seqs, void* stream);

/* The same for sequences whose cache is sharded by token range over several
 * pools (one per GPU): the local cache of sequence i starts at RoPE position
 * kv_pos_offset[i]; it appends new_tokens[i] (possibly 0) tokens locally while
 * q_rows[i] query rows, the first at RoPE position q_pos[i], are rotated for
 * it.  NULL arrays take the defaults of pa_batch_set (offset 0, one query row
 * per new token, positions following the cache). */
int pa_batch_set_sharded(pa_pool* pool, const int32_t* seq_ids,
                         const int32_t* new_tokens, const int32_t* q_rows,
                         const int32_t* q_pos, const int32_t* kv_pos_offset,
                         int n_seqs, void* stream);

/* ---- kernels ---------------------------------------------------------------
 * pa_append: RoPE (half-split pairs, fp32, round to nearest even) on the new
 * tokens' Q and K, K and V scattered into the cache through the block table.
 *   q_in  [rows][q_heads][64]   k_in, v_in [rows][kv_heads][64]   (bf16)
 *   cos, sin fp32 [>= max position + 1][32]
 *   q_out [rows][q_heads][64] (may alias q_in; may be NULL to skip Q)
 * q_heads = 4 * kv_heads of the pool. */
int pa_append(pa_pool* pool, int layer, const void* q_in, const void* k_in,
              const void* v_in, const float* cos_table, const float* sin_table,
              void* q_out, void* stream);

/* pa_decode: one query token per batch sequence against its whole cache
 * (split-KV over CTAs, log-sum-exp combine).
 *   q        [n_seqs][q_heads][64] bf16 (RoPE applied)
 *   out      bf16, row i at out + i*out_stride, q_heads*64 valid columns
 *            (head-major: column h*64+d) — the [tokens, 2048] layout; may be NULL
 *   out_f32  fp32 [n_seqs][q_heads][64], normalised; may be NULL
 *   lse      fp32 [n_seqs][q_heads], natural-log-sum-exp of the scaled scores
 *            (-inf for an empty sequence); may be NULL */
int pa_decode(pa_pool* pool, int layer, const void* q, void* out,
              int64_t out_stride, float* out_f32, float* lse, float scale,
              void* stream);

/* pa_decode_step: one decode step over layers [layer_begin, layer_end): per
 * layer a pa_append of the batch's new tokens followed by a pa_decode, all on
 * `stream` — the attention part of the reference's layer loop
 * (Transformer::forward, src/runtime/transformer.cu:47-89, calling steps 5-7 of
 * Attention::forward, src/runtime/attention.cu:192-359) without a host round
 * trip per layer.  Layer l reads q_in + l*q_layer_stride, k_in/v_in +
 * l*kv_layer_stride, writes the rotated Q to q_rot + l*q_layer_stride (may
 * alias q_in) and its output rows to out + l*out_layer_stride (strides in
 * elements).  lse, if given, is [layers][n_seqs][q_heads].
 * A call over SEVERAL layers needs every layer's q/k/v before it starts, i.e.
 * inputs that do not depend on an earlier layer's output (a benchmark, a
 * speculative or layer-parallel schedule): the one-launch step streams layer
 * l+1 while layer l is still being combined.  In a real forward pass layer
 * l+1's projections consume layer l's output, so the host calls it one layer
 * at a time (layer_end = layer_begin + 1) between its projection launches, or
 * uses pa_attention_step, which chains projections, attention and output
 * projection per layer with the true data flow. */
int pa_decode_step(pa_pool* pool, int layer_begin, int layer_end, const void* q_in,
                   const void* k_in, const void* v_in, int64_t q_layer_stride,
                   int64_t kv_layer_stride, const float* cos_table,
                   const float* sin_table, void* q_rot, void* out, int64_t out_stride,
                   int64_t out_layer_stride, float* lse, float scale, void* stream);

/* pa_prefill: causal attention of the batch's new tokens (batch of ONE
 * sequence) against positions [0, kv_len) of its cache.
 *   q   [rows][q_heads][64] bf16 (RoPE applied)   out [rows][q_heads*64] bf16
 *   lse fp32 [q_heads][rows], may be NULL */
int pa_prefill(pa_pool* pool, int layer, const void* q, void* out, float* lse,
               float scale, void* stream);

/* Merge split-KV partials from n_parts disjoint key ranges (e.g. one per GPU):
 *   o_parts [n_parts][rows][64] fp32 normalised, lse_parts [n_parts][rows];
 *   out bf16 [rows][64] (may be NULL), out_f32 / lse_out optional. */
int pa_merge_partials(const float* o_parts, const float* lse_parts, int n_parts,
                      int rows, void* out, float* out_f32, float* lse_out,
                      void* stream);

/* Un-page one sequence of the batch-independent cache: K and V as
 * [kv_heads][out_stride_tokens][64] bf16, first `length` rows written. */
int pa_gather_kv(pa_pool* pool, int layer, int seq_id, void* k_out, void* v_out,
                 int out_stride_tokens, void* stream);

/* ---- sequence-range sharding over several GPUs (one process per GPU) --------
 * The reference is single-GPU; this is the exchange long-context decode needs
 * once a sequence's cache is split by token range over n pools.  Each rank's
 * decode kernel stores its partial (normalised O, LSE) into every rank's
 * receive buffer with peer stores.  In pa_decode_step_sharded every value
 * travels as an 8-byte word {value, step number}; the CTA that combined a
 * (sequence, head) polls its own memory (bounded, PA_ERR_TIMEOUT via
 * pa_pool_check) until all ranks' words of its rows carry the step number and
 * merges them.  pa_decode_push / pa_exchange_merge use fp32 rows and one flag
 * per (rank, head) instead.  No rank ever loads from a peer.  Buffers are shared
 * through CUDA IPC handles of
 * PA_EXCHANGE_HANDLE_BYTES bytes that the host passes between processes.
 * All ranks must issue the same sequence of sharded steps. */
typedef struct pa_exchange pa_exchange;
#define PA_EXCHANGE_HANDLE_BYTES 64
int pa_exchange_create(pa_exchange** out, int device, int rank, int world, int n_seqs,
                       int kv_heads);
int pa_exchange_handle(pa_exchange* x, void* handle64);
/* handles: world * PA_EXCHANGE_HANDLE_BYTES bytes in rank order */
int pa_exchange_connect(pa_exchange* x, const void* handles);
/* The same mapping for a host that drives several GPUs from ONE process (it has
 * enabled peer access itself): every rank's receive buffer as a plain pointer. */
int pa_exchange_buffer(pa_exchange* x, void** dev_ptr, uint64_t* bytes);
int pa_exchange_connect_ptrs(pa_exchange* x, void* const* peer_buffers);
int pa_exchange_destroy(pa_exchange* x);
/* The two halves of a sharded decode of one layer: pa_decode_push runs the
 * decode kernel, which pushes this rank's partials to all ranks;
 * pa_exchange_merge waits for all ranks' partials of that step and writes the
 * merged bf16 rows.  (pa_decode_step_sharded does both inside one kernel, for
 * all layers of the step in one cooperative launch when the batch allows it.) */
int pa_decode_push(pa_pool* pool, pa_exchange* x, int layer, const void* q, float scale,
                   void* stream);
int pa_exchange_merge(pa_pool* pool, pa_exchange* x, void* out, int64_t out_stride,
                      void* stream);
/* pa_decode_step for a range-sharded batch (see pa_batch_set_sharded); k_in and
 * v_in may be NULL on ranks that append nothing.  out receives the merged rows. */
int pa_decode_step_sharded(pa_pool* pool, pa_exchange* x, int layer_begin, int layer_end,
                           const void* q_in, const void* k_in, const void* v_in,
                           int64_t q_layer_stride, int64_t kv_layer_stride,
                           const float* cos_table, const float* sin_table, void* q_rot,
                           void* out, int64_t out_stride, int64_t out_layer_stride,
                           float scale, void* stream);

/* The same step for `world` (at most 4) ranks whose pools live on ONE GPU — a
 * rehearsal of a multi-GPU deployment on a single device, and the way the
 * in-kernel exchange is exercised where only one GPU is available.  Ranks wait
 * on each other's words, and separate launches on one GPU are not guaranteed to
 * run at the same time, so all ranks' steps run as ONE cooperative launch:
 * every rank's step must fit SMs/world CTAs (at least 2 layers, one query row
 * and at most one new token per sequence, q_rot apart from q_in; force fewer
 * split-KV chunks with pa_pool_set_decode_chunk_blocks).  Arrays are indexed by
 * rank; the exchanges are connected with pa_exchange_connect_ptrs.  No
 * counterpart in the reference. */
int pa_decode_step_sharded_colocated(pa_pool* const* pools, pa_exchange* const* xs, int world,
                                     int layer_begin, int layer_end, const void* const* q_in,
                                     const void* const* k_in, const void* const* v_in,
                                     int64_t q_layer_stride, int64_t kv_layer_stride,
                                     const float* cos_table, const float* sin_table,
                                     void* const* q_rot, void* const* out, int64_t out_stride,
                                     int64_t out_layer_stride, float scale, void* stream);

/* ---- KV-head sharding over several GPUs ---------------------------------------
 * Each rank's pool holds 8/n KV heads (kv_heads of pa_pool_create) and serves
 * the 4*8/n query heads of those groups; every rank needs the full
 * [sequences, 2048] attention rows afterwards.  The all-gather is fused into the
 * decode kernel: finished rows are stored into the column slice of every rank's
 * row buffer by peer stores and counted per (source rank, layer); one wait at
 * the end of the step (bounded, PA_ERR_TIMEOUT via pa_pool_check) replaces all
 * per-layer collectives.  Buffers travel between processes as CUDA IPC handles
 * (PA_EXCHANGE_HANDLE_BYTES each), or as plain pointers inside one process. */
typedef struct pa_gather pa_gather;
int pa_gather_create(pa_gather** out, int device, int rank, int world, int n_seqs,
                     int layers, int kv_heads);
int pa_gather_handle(pa_gather* g, void* handle64);
int pa_gather_connect(pa_gather* g, const void* handles);
int pa_gather_buffer(pa_gather* g, void** dev_ptr, uint64_t* bytes);
int pa_gather_connect_ptrs(pa_gather* g, void* const* peer_buffers);
int pa_gather_destroy(pa_gather* g);
/* One decode step over all layers of the gather (append fused in, see
 * pa_decode_step).  With wait != 0 it ends with the arrival wait and *rows is
 * this step's [layers][n_seqs][2048 * ...] bf16 rows on this device (valid until
 * the step after next); with wait == 0 call pa_gather_wait later. */
int pa_decode_step_gathered(pa_pool* pool, pa_gather* g, const void* q_in, const void* k_in,
                            const void* v_in, int64_t q_layer_stride, int64_t kv_layer_stride,
                            const float* cos_table, const float* sin_table, void* q_rot,
                            float scale, int wait, void* stream, void** rows);
int pa_gather_wait(pa_pool* pool, pa_gather* g, void* stream, void** rows);

/* pa_decode_noalloc: pa_decode for hosts that are not allowed to allocate
 * device memory — a plug-in inside a serving process that owns the whole GPU
 * through its own arena, a latency-critical loop that cannot afford the
 * device-wide synchronisation an allocation implies, a process with a fixed,
 * audited memory budget.  It has no counterpart in the reference; it exists
 * because pa_pool_create (which allocates) is closed to such callers.
 * Everything is caller-owned: the cache layer in this library's physical
 * layout (see pa_pool_layer_storage), device block tables
 * [n_seqs][table_stride], host kv_lens[n_seqs], q [n_seqs][4*kv_heads][64],
 * out rows of out_stride elements, optional lse [n_seqs][4*kv_heads].
 * The split-KV scratch is a fixed array inside the library image (271104
 * bytes = 264.75 KiB, held by every GPU that loads the library until exit), hence the
 * limit: at most PA_NOALLOC_MAX_SEQS sequences per call, larger batches are
 * rejected with PA_ERR_UNSUPPORTED.  No cudaMalloc/cudaFree or allocating
 * library routine is called.  All calls on a device share that array and it
 * keeps the previous call's contents (the entry re-zeroes what must start at
 * zero): calls that overlap on the GPU — different streams, no ordering —
 * race.  The first call on each device also resolves the array's device
 * address; make it before any stream capture begins.  A stream that is being
 * captured is refused with PA_ERR_STATE: the entry copies its batch descriptor
 * from host memory that does not outlive the call and plans its split from
 * the host array kv_lens.
 * The kernels record a block id outside [0, num_blocks) (block 0 is read in its
 * place, so that call's rows are wrong) or a bounded wait that ran out in a status word of
 * the same array; it stays there until pa_decode_noalloc_check(stream), which
 * synchronises the stream, returns PA_ERR_INVALID_ARG / PA_ERR_TIMEOUT / PA_OK
 * and clears the word.  It allocates nothing either and has no counterpart in
 * the reference. */
#define PA_NOALLOC_MAX_SEQS 8
int pa_decode_noalloc(const void* cache_layer, int num_blocks, int kv_heads,
                      const int32_t* block_tables, int table_stride,
                      const int32_t* kv_lens, int n_seqs, const void* q, void* out,
                      int64_t out_stride, float* lse, float scale, void* stream);
int pa_decode_noalloc_check(void* stream);

/* ---- one decode step through the attention blocks, layers chained by their data ----
 * Replaces Attention::forward at seq_len == 1 (src/runtime/attention.cu:99-390: RMSNorm, three
 * projection GEMMs, RoPE kernels, append copies, attention kernel, layout kernel, output
 * projection, with a device synchronisation after each and per-call allocations), the attention
 * residual of TransformerBlock::forward (src/runtime/transformer_block.cu:76-81) and the layer
 * loop of Transformer::forward (src/runtime/transformer.cu:47-89) as far as attention goes.
 * Per layer l of [layer_begin, layer_end):
 *     xn      = RMSNorm(x_l, input_norm[l])             (skipped when input_norm is NULL)
 *     q, k, v = xn Wq[l], xn Wk[l], xn Wv[l]
 *     attn    = append (RoPE on K) + decode attention (RoPE on Q) over the layer's cache
 *     x_{l+1} = attn Wo[l] (+ x_l when add_residual != 0)
 * x_l of the first layer is x_in [rows, hidden], the last layer's result goes to x_out; rows =
 * sequences of the active batch (at most 8, one query row each).  A caller with an FFN between
 * the attention blocks calls it one layer at a time.  Three launches per layer, chained by
 * programmatic dependent launch; intermediate rows live in the pool (no allocation, no host
 * synchronisation).  `exchange` (nullable) is the range-sharded variant: every rank projects the
 * same rows, the rank that appends does so, partials are exchanged and merged in the decode
 * kernel.  Weight pointers address layer 0 of the model. */
typedef struct pa_attention_weights {
  const void* input_norm; /* [layers][hidden] bf16, nullable */
  const void* wq;         /* [layers][hidden, q_heads*64] row-major (the reference's layout) */
  const void* wk;         /* [layers][hidden, kv_heads*64] */
  const void* wv;
  const void* wo;         /* [layers][q_heads*64, hidden] */
  int64_t norm_layer_stride, wq_layer_stride, wkv_layer_stride, wo_layer_stride; /* elements */
  float rms_eps;          /* the reference passes 1e-5 */
  int hidden;
} pa_attention_weights;
int pa_attention_step(pa_pool* pool, pa_exchange* exchange, int layer_begin, int layer_end,
                      const pa_attention_weights* weights, const void* x_in, void* x_out,
                      int add_residual, const float* cos_table, const float* sin_table, float scale,
                      void* stream);

/* ---- the component after the attention block: the feed-forward block of a decode step -------
 * Replaces runtime::FeedForward::forward (src/runtime/ffn.cu:34-145: rmsnorm_launch<2048>,
 * launch_gemm_2048x8192 twice, launch_silu_mul, launch_gemm_8192x2048, per-call temporaries) and
 * the residual add that follows it (src/runtime/transformer_block.cu:76-81) for decode shapes
 * (1 to 8 rows), as two weight-streaming launches:
 *     xn  = RMSNorm(x, ffn_norm[layer])                      (skipped when ffn_norm is NULL)
 *     h   = bf16(SiLU(bf16(xn Wgate)) * bf16(xn Wup))        -> h_scratch [rows, inter]
 *     out = bf16(h Wdown), then bf16(x + out) when add_residual != 0
 * Weights row-major as the reference holds them: gate, up [hidden, inter], down [inter, hidden];
 * pointers address layer 0.  Built for hidden 2048 and intermediate 8192.  out may alias x. */
typedef struct pa_ffn_weights {
  const void* ffn_norm; /* [layers][hidden] bf16, nullable */
  const void* gate;     /* [layers][hidden, inter] */
  const void* up;       /* [layers][hidden, inter] */
  const void* down;     /* [layers][inter, hidden] */
  int64_t norm_layer_stride, gate_layer_stride, up_layer_stride, down_layer_stride; /* elements */
  float rms_eps;        /* the reference passes 1e-5 */
  int hidden, inter;
} pa_ffn_weights;
int pa_ffn(const pa_ffn_weights* weights, int layer, const void* x, void* h_scratch, void* out, int rows,
           int add_residual, void* stream);
/* The same block for prompt chunks (any number of rows) on the tensor cores: RMSNorm kernel, then
 * two launches of the projection GEMM of pa_qkv_project_append: gate and up as ONE GEMM whose tiles
 * hold a gate head and the up head of the same columns, with SiLU(gate) * up as the epilogue, and
 * the down projection (+ residual).  gate, up and down of `weights` are PACKED by
 * pa_pack_projection_weights (hidden x inter, hidden x inter, inter x hidden); ffn_norm is plain.
 * scratch: rows * (hidden + inter) bf16, 16-byte aligned; x 16-byte aligned; out must not alias x. */
int pa_ffn_rows(pa_pool* pool, const pa_ffn_weights* weights, int layer, const void* x, void* scratch, void* out,
                int rows, int add_residual, void* stream);
/* One decode step through whole transformer blocks of layers [layer_begin, layer_end), as
 * runtime::TransformerBlock::forward chains them (src/runtime/transformer_block.cu:40-90):
 *     a       = x_l + Attention(x_l)      (pa_attention_step of one layer, add_residual = 1)
 *     x_{l+1} = a + FeedForward(a)        (pa_ffn, add_residual = 1)
 * Five launches per layer, every one behind the first chained by programmatic dependent launch;
 * all intermediate rows live in the pool.  Same batch rules as pa_attention_step. */
int pa_block_step(pa_pool* pool, pa_exchange* exchange, int layer_begin, int layer_end,
                  const pa_attention_weights* attention, const pa_ffn_weights* ffn, const void* x_in,
                  void* x_out, const float* cos_table, const float* sin_table, float scale, void* stream);

/* ---- the end of a decode step: language-model head and greedy sampling ----------------------
 * pa_lm_head replaces rmsnorm_launch<2048> + launch_gemm_2048x128256 of the reference's decode
 * loop (src/runtime/llama_runtime.cu:880-905): logits [rows, vocab] bf16 = RMSNorm(x, final_norm)
 * W_lm, W_lm [hidden, vocab] row-major as the reference holds it, final_norm nullable; 1 to 8
 * rows, vocab a multiple of 32.  pa_argmax replaces launch_argmax
 * (src/kernels/sampling/argmax_128256.cu) and the cudaMalloc / blocking copy / cudaFree around it
 * (llama_runtime.cu:907-930): tokens[r] = index of the largest logit of row r; equal largest values
 * are told apart as the structure of the reference's kernel does (its 256 threads, lanes and warps
 * in bit-reversed order, then the smallest index).  Top-k sampling (topk_128256.cu) is not built. */
int pa_lm_head(const void* x, const void* final_norm, float eps, const void* w_lm, void* logits, int rows,
               int hidden, int vocab, void* stream);
int pa_argmax(const void* logits, int32_t* tokens, int rows, int vocab, void* stream);

/* ---- a whole decode step of the model ---------------------------------------------------------
 * pa_embedding replaces launch_embedding (src/kernels/embedding/embedding.cu:31-95): out[r, :] =
 * table[tokens[r], :], bf16 rows of `hidden` elements, ids read on the device; an id outside
 * [0, vocab) gives a row of zeros (the reference reads outside the table).
 *
 * pa_decode_token replaces the body of LlamaRuntime::decode_forward
 * (src/runtime/llama_runtime.cu:822-945) for the sequences of the active batch (pa_batch_set, one new
 * token each, at most 8): ids -> embedding -> the pool's layers as pa_block_step runs them -> final
 * RMSNorm + language-model head -> greedy token.  tokens_in, tokens_out: device int32 [sequences]
 * (they may be the same buffer); logits: device bf16 [sequences, vocab], the caller's.  No host
 * synchronisation, no allocation; chained != 0 says the ids are the output of the step enqueued
 * just before on this stream (the embedding kernel is then a dependent launch too).  An id out of
 * range is recorded in the pool's status word (pa_pool_check). */
typedef struct pa_model_weights {
  const void* embed_tokens;              /* [vocab, hidden] bf16 */
  const pa_attention_weights* attention; /* every layer's attention block */
  const pa_ffn_weights* ffn;             /* every layer's feed-forward block */
  const void* final_norm;                /* [hidden] bf16, nullable */
  const void* lm_head;                   /* [hidden, vocab] bf16 row-major */
  int vocab;                             /* a multiple of 32 */
  float rms_eps;                         /* of the final norm */
} pa_model_weights;
int pa_embedding(const int32_t* tokens, const void* table, void* out, int rows, int hidden, int vocab, void* stream);
int pa_decode_token(pa_pool* pool, const pa_model_weights* model, const int32_t* tokens_in, int32_t* tokens_out,
                    void* logits, const float* cos_table, const float* sin_table, float scale, int chained,
                    void* stream);

/* Host: fp32 cos/sin tables [seq_len][32], Llama-3 frequency scaling. */
int pa_build_rope_tables(float* cos_table, float* sin_table, int seq_len);

/* Device status word of the pool: 0, or PA_ERR_TIMEOUT / PA_ERR_INVALID_ARG
 * recorded by a kernel (bounded wait ran out, block id out of range).
 * Synchronises `stream`, reads and clears the word. */
int pa_pool_check(pa_pool* pool, void* stream);

/* Tuning knobs (0 keeps the built-in heuristic): blocks per split-KV chunk. */
int pa_pool_set_decode_chunk_blocks(pa_pool* pool, int chunk_blocks);
/* The kernel of one layer (pa_decode, pa_attention_step, a one-layer pa_decode_step): the chunks of a
 * (sequence, head) as one thread-block cluster of 2, 4, 8 or 16 CTAs that combine through distributed
 * shared memory.  0 (default): the planner uses it for short contexts whose clusters are all
 * resident at once; -1: never.  No counterpart in the reference. */
int pa_pool_set_decode_cluster(pa_pool* pool, int mode);
/* pa_decode_step and pa_decode_step_sharded run the layers of a step as one
 * cooperative launch when the batch allows it (enable != 0, the default);
 * enable == 0 keeps one kernel per layer.  No counterpart in the reference. */
int pa_pool_set_step_kernel(pa_pool* pool, int enable);
/* allow == 0: the layers of a multi-layer decode step neither share a launch nor overlap (no
 * programmatic dependent launch): layer l+1 starts when layer l's rows are final, as it must when
 * its inputs depend on them.  The default (allow != 0) lets independent layers overlap. */
int pa_pool_set_layer_overlap(pa_pool* pool, int allow);
/* Combining CTAs per (sequence, KV head) in the one-launch step: 1, 2 or 4; 0 = heuristic. */
int pa_pool_set_step_combiners(pa_pool* pool, int combiners);
/* How many decode steps of this pool ran as one launch so far. */
int pa_pool_step_launches(pa_pool* pool, long long* count);
/* Warps per decode CTA and 4 KiB ring stages per warp (built shapes only). */
int pa_pool_set_decode_shape(pa_pool* pool, int warps, int stages);

/* ---- producer side of the path: Q/K/V projections of a decode step -----------
 * Replaces, for decode shapes (rows = sequences of the step, at most 8), the
 * reference's launch_gemm_2048x2048 + 2 x launch_gemm_2048x512 per layer
 * (src/runtime/attention.cu:138-191; src/kernels/gemm/gemm_2048x2048.hpp,
 * gemm_2048x512.hpp: A [M, K] row-major, B [K, N] row-major, bf16 in, fp32
 * accumulation, bf16 out).  x [layers][rows, hidden]; wq [layers][hidden, q_cols];
 * wk, wv [layers][hidden, kv_cols]; q [layers][rows, q_cols]; k, v
 * [layers][rows, kv_cols]; all bf16, layer strides in elements.  One launch for
 * all layers; the outputs are what pa_decode_step takes as q_in, k_in, v_in. */
int pa_qkv_project(const void* x, const void* wq, const void* wk, const void* wv, void* q, void* k,
                   void* v, int rows, int layers, int hidden, int q_cols, int kv_cols,
                   int64_t x_layer_stride, int64_t wq_layer_stride, int64_t wkv_layer_stride,
                   int64_t q_layer_stride, int64_t kv_layer_stride, void* stream);

/* The same projections with the RMSNorm that precedes them in Attention::forward
 * (src/runtime/attention.cu:118-131 calling rmsnorm_launch<2048>, src/kernels/rmsnorm/rmsnorm.cu:51-148)
 * as the kernel's prologue: x <- bf16((x * rsqrt(mean(x^2) + eps)) * norm_weight) on the staged
 * rows, with the reference kernel's arithmetic and summation order (bit-equal normalised rows for
 * hidden 2048).  norm_weight [layers][hidden] bf16. */
int pa_rmsnorm_qkv_project(const void* x, const void* norm_weight, int64_t norm_layer_stride, float eps,
                           const void* wq, const void* wk, const void* wv, void* q, void* k, void* v,
                           int rows, int layers, int hidden, int q_cols, int kv_cols,
                           int64_t x_layer_stride, int64_t wq_layer_stride, int64_t wkv_layer_stride,
                           int64_t q_layer_stride, int64_t kv_layer_stride, void* stream);
/* RMSNorm over any number of rows (prompt chunks, whose projections run on the tensor cores):
 * y [rows, hidden] = the same arithmetic; hidden a multiple of 256, at most 2048; y may alias x. */
int pa_rmsnorm(const void* x, const void* weight, void* y, int rows, int hidden, float eps, void* stream);

/* ---- consumer side of the path: output projection + attention residual ---------
 * out = bf16(residual + bf16(attn W_o)) for the rows of a decode step (at most 8),
 * all layers in one launch.  Replaces launch_gemm_2048x2048 on the attention
 * output (src/runtime/attention.cu:367-375) and transformer::residual_add
 * (src/runtime/transformer_block.cu:76-81; src/kernels/residual_add/residual_add.cu:14-38)
 * with their rounding: the GEMM result is rounded to bf16, the sum once more.
 * attn [layers][rows, hidden]; wo [layers][hidden, cols] row-major; residual
 * (nullable) and out [layers][rows, cols], both with out_layer_stride. */
int pa_out_project(const void* attn, const void* wo, const void* residual, void* out, int rows, int layers,
                   int hidden, int cols, int64_t attn_layer_stride, int64_t wo_layer_stride,
                   int64_t out_layer_stride, void* stream);
/* The same for prompt chunks (any number of rows), on the tensor cores: the projection GEMM of
 * pa_qkv_project_append with a plain epilogue.  wo_packed from pa_pack_projection_weights; cols a
 * multiple of 256; attn [rows, hidden] (16-byte aligned, read in place through a tensor map),
 * residual (nullable) and out [rows, cols].  Uses the pool's status word. */
int pa_out_project_rows(pa_pool* pool, const void* attn, const void* wo_packed, const void* residual,
                        void* out, int rows, int hidden, int cols, void* stream);
/* pa_qkv_project on weights repacked by pa_pack_projection_weights (the format
 * pa_qkv_project_append reads, so one copy of the weights serves decode and
 * prefill): the stream becomes 8 KiB contiguous bursts through a bulk-copy ring.
 * status_word: device int that receives PA_ERR_TIMEOUT if a bounded wait runs
 * out (a pool's status word or the caller's own). */
int pa_qkv_project_packed(const void* x, const void* wq_packed, const void* wk_packed, const void* wv_packed,
                          void* q, void* k, void* v, int rows, int layers, int hidden, int q_cols,
                          int kv_cols, int64_t x_layer_stride, int64_t wq_layer_stride,
                          int64_t wkv_layer_stride, int64_t q_layer_stride, int64_t kv_layer_stride,
                          int* status_word, void* stream);
/* One-time repacking of a row-major [hidden, cols] bf16 weight matrix (the
 * reference's layout) into the tile image pa_qkv_project_append copies with one
 * bulk copy per k-step: per 64 rows and 64 columns an 8 KiB block of 128-byte
 * rows, 16-byte chunk c of row r at c ^ (r & 7).  Same size as the input, must
 * not alias it.  Done at model load; no counterpart in the reference. */
int pa_pack_projection_weights(const void* w, void* packed, int hidden, int cols, void* stream);
/* The same projections for the new tokens of the active batch (prefill shapes),
 * on the tensor cores, with RoPE and the cache append as the epilogue: one launch
 * for what the reference does with 3 GEMM launches, 3 RoPE/transpose kernels and
 * 2*8*tokens copies per layer (src/runtime/attention.cu:138-262).  x [rows, hidden]
 * in batch order (rows = the batch's new tokens, which must also be its query
 * rows); weights packed by pa_pack_projection_weights; q_out [rows, q_heads*64] receives the rotated queries,
 * K (rotated) and V go straight into the layer's paged cache.  Needs 4 or 8 KV
 * heads in the pool; x 16-byte aligned (it is read in place through a tensor map). */
int pa_qkv_project_append(pa_pool* pool, int layer, const void* x, const void* wq, const void* wk,
                          const void* wv, const float* cos_table, const float* sin_table, void* q_out,
                          int hidden, void* stream);

#ifdef __cplusplus
}
#endif
#endif
