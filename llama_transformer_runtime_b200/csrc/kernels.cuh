// Launch descriptors and launcher prototypes of the sm_100a kernels.
#pragma once
#include "pa_common.cuh"

namespace pa {

struct AppendParams {
  const __nv_bfloat16* q_in;
  const __nv_bfloat16* k_in;
  const __nv_bfloat16* v_in;
  __nv_bfloat16* q_out;  // nullptr: leave Q alone
  const float* cos_table;
  const float* sin_table;
  char* storage;              // this layer's cache
  const int32_t* tables;      // device mirror [max_seqs][max_blocks_per_seq]
  const BatchEntry* batch;    // device, n_seqs entries
  int* status;
  int kv_heads, num_blocks, max_blocks_per_seq;
};
cudaError_t launch_append(const AppendParams& p, int n_seqs, int max_new, cudaStream_t stream);

struct GatherParams {
  const char* storage;
  const int32_t* table;  // device row of one sequence
  __nv_bfloat16* k_out;
  __nv_bfloat16* v_out;
  int* status;
  int kv_heads, num_blocks, length, out_stride;
};
cudaError_t launch_gather(const GatherParams& p, cudaStream_t stream);

// Split-KV decode.  Grid (max_chunks, kv_heads, n_seqs); CTA (x, h, z) streams
// blocks [x*chunk_blocks, (x+1)*chunk_blocks) of sequence z's table for KV head
// h and serves the 4 query heads of that group.
struct DecodeParams {
  const __nv_bfloat16* q;     // [n_seqs][q_heads][64]
  __nv_bfloat16* out;         // bf16 rows, stride out_stride elements (nullable)
  float* out_f32;             // [n_seqs][q_heads][64] (nullable)
  float* lse;                 // [n_seqs][q_heads] (nullable)
  const char* storage;
  const int32_t* tables;
  const BatchEntry* batch;
  float* ws_acc;              // workspace: [item][4][64] un-normalised partial sums
  float* ws_ml;               // workspace: [item][2][4] running max (base-2 scaled) and sum
  unsigned int* ws_count;     // arrival tickets, one per (batch row, kv head), zero between launches
  int* status;
  long long out_stride;
  float scale_log2;           // scale * log2(e)
  int kv_heads, num_blocks, max_blocks_per_seq, chunk_blocks, max_chunks;
  // Cross-GPU exchange of split-KV partials (sequence-range sharding); off when
  // xchg_world == 0.  Receive buffer of rank g: data [2 slots][world][rows][65]
  // fp32 (64 normalised outputs + natural-log LSE), flags [world][groups] u32.
  float* xchg_peer[8] = {};
  unsigned int* xchg_flag[8] = {};
  int xchg_world = 0, xchg_rank = 0, xchg_rows = 0, xchg_groups = 0, xchg_slot = 0;
  unsigned int xchg_seq = 0;
  // merged bf16 rows written by the combining CTA itself after it has waited
  // for all ranks' partials of its (sequence, KV head); nullptr: a separate
  // merge kernel does it
  __nv_bfloat16* xchg_out = nullptr;
  long long xchg_out_stride = 0;
  // In-kernel merge: partials travel as 8-byte words {value, step number}
  // (xchg_ll[g] = rank g's word region, [kXchgWordSlots][world][rows][65] words, slot = step modulo kXchgWordSlots), so a
  // word is valid as soon as it carries this step's number: no fence, no flag.
  unsigned long long* xchg_ll[8] = {};
  // KV-head sharding: this rank's heads are columns [hs_col0, hs_col0 + q_heads*64)
  // of rows of hs_stride elements; the finished rows are stored into every
  // rank's row buffer (all-gather by peer stores) and counted in every rank's
  // arrival counter for (this rank, this layer).  Off when hs_world == 0.
  __nv_bfloat16* hs_rows[8] = {};
  unsigned int* hs_counter[8] = {};
  int hs_world = 0, hs_col0 = 0;
  long long hs_stride = 0;
  // Fused append (one new token per sequence at most): q is un-rotated, the
  // kernel rotates it and appends k_new/v_new rows (RoPE on K) to the cache.
  // launched with programmatic stream serialization (see the griddepcontrol points in the
  // kernel).  1: behind the previous layer's decode kernel, whose workspace it shares — the
  // inputs are ready, it waits before it writes.  2: behind the kernel that produces q, k_new and
  // v_new — it waits before it reads them, after its first cache copies are under way.
  int pdl = 0;
  // > 0 (the kernel of one layer only): the max_chunks CTAs of a (sequence, head) are one thread-block
  // cluster of this size; they combine through distributed shared memory instead of the workspace,
  // the arrival counter and the last-arriver's loads
  int cluster = 0;
  int fuse = 0;
  const __nv_bfloat16* k_new = nullptr;  // [rows][kv_heads][64], row e.kv_row_off
  const __nv_bfloat16* v_new = nullptr;
  const float* cos_table = nullptr;
  const float* sin_table = nullptr;
  char* storage_w = nullptr;             // == storage, writable
  __nv_bfloat16* q_rot_out = nullptr;    // rotated Q [n_seqs][q_heads][64] (nullable, must not alias q)
};
constexpr int kXchgRowFloats = kHeadDim + 1;
// Slots of the {value, step} word region (slot = step number modulo this).  With C combining CTAs
// per (sequence, head) on alternate layers a peer can be C layers ahead of a slot a rank still
// polls: the slot count must be a multiple of C and at least 2 C.  C is 1, 2 or 4.
constexpr unsigned int kXchgWordSlots = 8;

// A whole multi-layer decode step in one cooperative launch (decode_step_kernel):
// `base` holds layer 0's parameters; layer l adds l strides to every per-layer
// pointer, uses workspace slice l and exchange step base.xchg_seq + l.
struct DecodeStepParams {
  DecodeParams base;
  int layers = 0, n_seqs = 0;
  long long q_layer_stride = 0, kv_layer_stride = 0, out_layer_stride = 0, lse_layer_stride = 0;
  unsigned long long layer_bytes = 0;  // cache bytes per layer
  int ws_layer_items = 0;              // workspace items per layer (n_seqs * kv_heads * max_chunks)
  // streaming CTAs of sequence z: [seq_first[z], seq_first[z+1]) = its chunks x its heads
  // (ragged batches get exactly the CTAs they need); n_stream = seq_first[n_seqs]
  int n_stream = 0;
  unsigned short seq_first[41] = {};
  int combiners = 1;  // combining CTAs per (sequence, head): they take the layers in turn
};
constexpr int kMaxStepLayers = 64;
constexpr int kMaxStepSeqs = 40;
// CTAs of the step launch: streaming ones plus one combining CTA per (sequence, head)
inline int decode_step_ctas(const DecodeStepParams& sp) {
  return sp.n_stream + sp.combiners * sp.n_seqs * sp.base.kv_heads;
}
cudaError_t launch_decode_step(const DecodeStepParams& sp, int warps, int stages, cudaStream_t stream);
// The steps of up to kMaxColocatedRanks ranks whose pools share one GPU, as ONE cooperative launch
// (8-warp, 4-stage CTAs): rank r owns CTAs [r * ctas_per_rank, (r + 1) * ctas_per_rank).
constexpr int kMaxColocatedRanks = 4;
struct ColocatedStepParams {
  DecodeStepParams rank[kMaxColocatedRanks];
  int world = 0, ctas_per_rank = 0;
};
static_assert(sizeof(ColocatedStepParams) <= 4000, "kernel parameter space");
cudaError_t launch_decode_step_colocated(const ColocatedStepParams& cp, cudaStream_t stream);

// Waits (bounded) until every rank's partial of step `seq` has landed in this
// rank's receive buffer, then merges them: out rows bf16, stride out_stride.
struct ExchangeMergeParams {
  const float* data;           // this rank's receive buffer
  const unsigned int* flags;   // [world][groups]
  __nv_bfloat16* out;
  int* status;
  long long out_stride;
  int world, rows, groups, slot, q_heads;
  unsigned int seq;
};
cudaError_t launch_exchange_merge(const ExchangeMergeParams& p, cudaStream_t stream);
cudaError_t launch_decode(const DecodeParams& p, int n_seqs, int warps, int stages,
                          cudaStream_t stream);
bool decode_shape_supported(int warps, int stages);
size_t decode_ws_acc_floats_per_item();
int decode_cluster_limit(int warps, int stages);

// Prefill attention: for every batch sequence z, its n_q query rows (positions
// q_pos0 ...) against keys [0, kv_len) of its paged cache.  Row `row` of head h
// of sequence z is at q + z*q_seq_stride + (q_row_off+row)*q_row_stride +
// h*q_head_stride (elements), likewise for out: the token-major layout of the
// native API and the head-major one of the reference's launcher are both strides.
struct PrefillParams {
  const __nv_bfloat16* q;   // RoPE applied
  __nv_bfloat16* out;
  float* lse;               // [z][q_heads][n_q] (nullable)
  const char* storage;
  const int32_t* tables;
  const BatchEntry* batch;
  int* status;
  long long q_seq_stride, q_row_stride, q_head_stride;
  long long o_seq_stride, o_row_stride, o_head_stride;
  long long lse_seq_stride;
  float scale_log2;
  int kv_heads, num_blocks, max_blocks_per_seq, causal;
  // Work distribution of the persistent CTAs: *work counts the items handed
  // out and must be zero at launch; the launch clears *work_clear, the counter
  // a later launch will use.  grid_y and n_items are filled by launch_prefill.
  int* work = nullptr;
  int* work_clear = nullptr;
  int grid_y = 0, n_items = 0;
};
// n_q: the largest query-row count of any batch sequence
cudaError_t launch_prefill(const PrefillParams& p, int n_seqs, int n_q, cudaStream_t stream);

// Projection GEMM with RoPE + paged append epilogue (qkv_gemm.cu).
struct QkvGemmParams {
  const __nv_bfloat16* x;      // [rows, hidden] row-major, 16-byte aligned (read through a tensor map)
  const __nv_bfloat16* wq;     // [hidden, q_cols] packed by launch_pack_weights
  const __nv_bfloat16* wk;     // [hidden, kv_cols] packed
  const __nv_bfloat16* wv;     // [hidden, kv_cols] packed
  __nv_bfloat16* q_out;        // [rows, q_cols], RoPE applied
  char* storage;               // the layer's cache
  const int32_t* tables;
  const BatchEntry* batch;
  const float* cos_table;
  const float* sin_table;
  int* status;
  int rows, hidden, q_cols, kv_cols, kv_heads, n_seqs, num_blocks, max_blocks_per_seq;
  // linear == 1: one matrix (wq, q_cols columns), q_out = bf16(residual + bf16(x wq)) with plain
  // [rows, q_cols] rows; no RoPE, no cache, the batch and table fields are unused.
  // linear == 2: the gate and up projections of a feed-forward block as one GEMM: wq = gate, wk = up
  // (each [hidden, q_cols / 2] packed), q_out [rows, q_cols / 2] = bf16(SiLU(bf16(x gate)) * bf16(x up))
  int linear = 0;
  const __nv_bfloat16* residual = nullptr;  // [rows, q_cols], nullable
  int tile_heads = 0;  // heads per pair tile, 4 or 6; 0: the launcher chooses
};
cudaError_t launch_qkv_gemm(const QkvGemmParams& p, cudaStream_t stream);
// row-major [hidden, cols] -> per (64 k-rows, 64 columns) an 8 KiB block in the GEMM's shared-memory layout
cudaError_t launch_pack_weights(const void* src, void* dst, int hidden, int cols, cudaStream_t stream);

struct MergeParams {
  const float* o_parts;    // [n_parts][rows][64]
  const float* lse_parts;  // [n_parts][rows]
  __nv_bfloat16* out;      // [rows][64] (nullable)
  float* out_f32;          // nullable
  float* lse_out;          // nullable
  int n_parts, rows;
};
cudaError_t launch_merge(const MergeParams& p, cudaStream_t stream);

}  // namespace pa
