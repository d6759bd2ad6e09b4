// C-ABI layer (include/paged_attention.h): argument checks, pool ownership and
// launches.  No torch types, no exceptions across the boundary, no allocation
// outside the set-up call pa_pool_create.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "../../include/paged_attention.h"
#include "block_pool.hpp"
#include "kernels.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define PA_CUDA(call)                                                                   \
  do {                                                                                  \
    cudaError_t _e = (call);                                                            \
    if (_e != cudaSuccess)                                                              \
      return fail(PA_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e),  \
                  __FILE__, __LINE__);                                                  \
  } while (0)

constexpr int kWsItems = 148 * 64;  // split-KV partials the workspace can hold
constexpr int kMaxStepRows = 8;     // sequences of a decode step that pa_attention_step chains
constexpr int kMaxStepHidden = 2048;
constexpr int kMaxStepInter = 8192;   // feed-forward intermediate width pa_block_step has room for

// Restores the caller's current device on scope exit.
struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) ok = false;
    if (ok && prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace

namespace pa {
// For entry points that live in other translation units.
void set_last_error(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }
}  // namespace pa

struct pa_pool {
  pa::BlockPool host;
  int device, num_layers, kv_heads;
  size_t layer_bytes = 0;
  char* storage = nullptr;
  int32_t* d_tables = nullptr;
  pa::BatchEntry* d_batch = nullptr;
  float* ws_acc = nullptr;
  float* ws_ml = nullptr;
  unsigned int* ws_count = nullptr;
  int* d_status = nullptr;
  std::vector<pa::BatchEntry> batch;  // host copy of the active batch
  int max_new = 0, total_rows = 0, max_kv_blocks = 0;
  int chunk_blocks_override = 0;
  int decode_warps = 0, decode_stages = 0;  // 0: chosen per batch
  int sm_count = 0;
  bool no_step_kernel = false;  // pa_pool_set_step_kernel(pool, 0): one kernel per layer
  bool no_layer_overlap = false;  // pa_pool_set_layer_overlap(pool, 0): a layer starts after the previous one has finished
  int step_combiners_override = 0;  // pa_pool_set_step_combiners
  bool step_has_exchange = false;   // the step being planned ends every layer with a cross-rank exchange
  long long step_launches = 0;  // decode steps that ran as one cooperative launch
  // rows of a decode step between the kernels of pa_attention_step: q, k, v, rotated q, attention
  // output and two block inputs in turn, kMaxStepRows rows each; behind them the feed-forward block's
  // input and activated rows, and the embedded and final rows of pa_decode_token
  __nv_bfloat16* step_ws = nullptr;
  int cluster_mode = 0;  // one-layer decode kernel: 0 = planner decides, -1 = never clusters, 2/4/8/16 = that cluster size
  int* prefill_work = nullptr;  // 64 item counters, one per prefill launch in rotation, zero when idle
  unsigned prefill_launches = 0;
  pa_pool(int nb, int ms, int mb) : host(nb, ms, mb) {}
};

struct pa_exchange;
namespace pa {
bool exchange_fill(pa_exchange* x, DecodeParams& d, ExchangeMergeParams& m);
bool exchange_current(pa_exchange* x, ExchangeMergeParams& m);
void exchange_advance(pa_exchange* x, int steps);
void exchange_unfill(pa_exchange* x);
int exchange_rows(const pa_exchange* x);
int exchange_groups(const pa_exchange* x);
}  // namespace pa
// projection launchers of qkv_project.cu, with the programmatic-dependent-launch flag
namespace pa {
int qkv_project_impl(const void* x, const void* norm_weight, int64_t norm_layer_stride, float eps, const void* wq,
                     const void* wk, const void* wv, void* q, void* k, void* v, int rows, int layers, int hidden,
                     int q_cols, int kv_cols, int64_t x_layer_stride, int64_t wq_layer_stride,
                     int64_t wkv_layer_stride, int64_t q_layer_stride, int64_t kv_layer_stride, int pdl, void* stream);
int out_project_impl(const void* attn, const void* wo, const void* residual, void* out, int rows, int layers,
                     int hidden, int cols, int64_t attn_layer_stride, int64_t wo_layer_stride,
                     int64_t residual_layer_stride, int64_t out_layer_stride, int pdl, void* stream);
int ffn_impl(const void* x, const void* norm_w, float eps, const void* wg, const void* wu, const void* wd,
             const void* residual, void* h, void* out, int rows, int hidden, int inter, int pdl, void* stream);
int embedding_impl(const int32_t* tokens, const void* table, void* out, int rows, int hidden, int vocab, int* status,
                   int pdl, void* stream);
int lm_head_impl(const void* x, const void* final_norm, float eps, const void* w_lm, void* logits, int rows, int hidden,
                 int vocab, int pdl, void* stream);
int argmax_impl(const void* logits, int32_t* tokens, int rows, int vocab, int pdl, void* stream);
}  // namespace pa

struct pa_gather;
namespace pa {
bool gather_begin(pa_gather* g);
bool gather_fill(pa_gather* g, int layer, int n_seqs, int kv_heads, DecodeParams& d);
cudaError_t gather_wait(pa_gather* g, int* status, cudaStream_t stream, void** rows);
int gather_layers(const pa_gather* g);
}  // namespace pa

extern "C" {

const char* pa_last_error(void) { return g_err; }

int pa_pool_create(pa_pool** out, int device, int num_layers, int num_blocks, int kv_heads,
                   int max_seqs, int max_blocks_per_seq) {
  if (!out) return fail(PA_ERR_INVALID_ARG, "pa_pool_create: out is NULL");
  *out = nullptr;
  if (num_layers <= 0 || num_blocks <= 0 || max_seqs <= 0 || max_blocks_per_seq <= 0)
    return fail(PA_ERR_INVALID_ARG, "pa_pool_create: sizes must be positive");
  if (kv_heads != 1 && kv_heads != 2 && kv_heads != 4 && kv_heads != 8)
    return fail(PA_ERR_UNSUPPORTED, "pa_pool_create: kv_heads must be 1, 2, 4 or 8 (got %d)", kv_heads);
  pa_pool* p = new (std::nothrow) pa_pool(num_blocks, max_seqs, max_blocks_per_seq);
  if (!p) return fail(PA_ERR_INVALID_ARG, "pa_pool_create: out of host memory");
  p->device = device;
  p->num_layers = num_layers;
  p->kv_heads = kv_heads;
  p->layer_bytes = (size_t)num_blocks * kv_heads * pa::kPairBytes;
  if (device >= 0) {
    // device < 0 makes a host-only pool (allocator and tables, no kernels)
    DeviceGuard g(device);
    cudaError_t e = g.ok ? cudaSuccess : cudaErrorInvalidDevice;
    auto alloc = [&](void** ptr, size_t bytes) {
      if (e == cudaSuccess) e = cudaMalloc(ptr, bytes);
      if (e == cudaSuccess) e = cudaMemset(*ptr, 0, bytes);
    };
    alloc((void**)&p->storage, p->layer_bytes * num_layers);
    alloc((void**)&p->d_tables, (size_t)max_seqs * max_blocks_per_seq * sizeof(int32_t));
    alloc((void**)&p->d_batch, (size_t)max_seqs * sizeof(pa::BatchEntry));
    alloc((void**)&p->ws_acc, (size_t)kWsItems * pa::decode_ws_acc_floats_per_item() * sizeof(float));
    alloc((void**)&p->ws_ml, (size_t)kWsItems * 2 * pa::kGroup * sizeof(float));
    alloc((void**)&p->ws_count, (size_t)max_seqs * kv_heads * pa::kMaxStepLayers * sizeof(unsigned int));
    alloc((void**)&p->prefill_work, 64 * sizeof(int));
    alloc((void**)&p->step_ws, (size_t)kMaxStepRows * (3 * kv_heads * pa::kGroup * pa::kHeadDim +
                                                        2 * kv_heads * pa::kHeadDim + 5 * kMaxStepHidden + kMaxStepInter) *
                                   sizeof(__nv_bfloat16));
    alloc((void**)&p->d_status, sizeof(int));
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
      int code = fail(PA_ERR_CUDA, "pa_pool_create: device allocation failed: %s", cudaGetErrorString(e));
      cudaGetLastError();
      pa_pool_destroy(p);
      return code;
    }
  }
  *out = p;
  return PA_OK;
}

int pa_pool_destroy(pa_pool* p) {
  if (!p) return PA_OK;
  if (p->device >= 0) {
    DeviceGuard g(p->device);
    cudaFree(p->storage);
    cudaFree(p->d_tables);
    cudaFree(p->d_batch);
    cudaFree(p->ws_acc);
    cudaFree(p->ws_ml);
    cudaFree(p->ws_count);
    cudaFree(p->prefill_work);
    cudaFree(p->step_ws);
    cudaFree(p->d_status);
  }
  delete p;
  return PA_OK;
}

int pa_pool_free_blocks(const pa_pool* p, int* n_free) {
  if (!p || !n_free) return fail(PA_ERR_INVALID_ARG, "pa_pool_free_blocks: NULL argument");
  *n_free = p->host.free_blocks();
  return PA_OK;
}

int pa_pool_set_free_order(pa_pool* p, const int32_t* order, int n) {
  if (!p || !order) return fail(PA_ERR_INVALID_ARG, "pa_pool_set_free_order: NULL argument");
  if (!p->host.set_free_order(order, n))
    return fail(PA_ERR_INVALID_ARG,
                "pa_pool_set_free_order: needs a permutation of all %d blocks while none is in use",
                p->host.num_blocks());
  return PA_OK;
}

int pa_pool_layer_storage(const pa_pool* p, int layer, void** dev_ptr, uint64_t* bytes) {
  if (!p || layer < 0 || layer >= p->num_layers)
    return fail(PA_ERR_INVALID_ARG, "pa_pool_layer_storage: bad pool or layer");
  if (dev_ptr) *dev_ptr = p->storage ? p->storage + (size_t)layer * p->layer_bytes : nullptr;
  if (bytes) *bytes = p->layer_bytes;
  return PA_OK;
}

int pa_seq_create(pa_pool* p, int* seq_id) {
  if (!p || !seq_id) return fail(PA_ERR_INVALID_ARG, "pa_seq_create: NULL argument");
  int s = p->host.create();
  if (s < 0) return fail(PA_ERR_OUT_OF_BLOCKS, "pa_seq_create: all %d sequence ids in use", p->host.max_seqs());
  *seq_id = s;
  return PA_OK;
}

int pa_seq_free(pa_pool* p, int seq_id) {
  if (!p || !p->host.release(seq_id)) return fail(PA_ERR_INVALID_ARG, "pa_seq_free: unknown sequence %d", seq_id);
  return PA_OK;
}

int pa_seq_reserve(pa_pool* p, int seq_id, int new_len) {
  if (!p) return fail(PA_ERR_INVALID_ARG, "pa_seq_reserve: NULL pool");
  int r = p->host.reserve(seq_id, new_len);
  if (r == 1)
    return fail(PA_ERR_INVALID_ARG, "pa_seq_reserve: bad sequence %d or length %d (table holds %d blocks)",
                seq_id, new_len, p->host.max_blocks_per_seq());
  if (r == 2)
    return fail(PA_ERR_OUT_OF_BLOCKS, "pa_seq_reserve: %d free blocks cannot grow sequence %d to %d tokens",
                p->host.free_blocks(), seq_id, new_len);
  return PA_OK;
}

int pa_seq_length(const pa_pool* p, int seq_id, int* len) {
  if (!p || !len || !p->host.valid(seq_id)) return fail(PA_ERR_INVALID_ARG, "pa_seq_length: bad argument");
  *len = p->host.length(seq_id);
  return PA_OK;
}

int pa_seq_block_table(const pa_pool* p, int seq_id, const int32_t** table, int* n_blocks) {
  if (!p || !p->host.valid(seq_id)) return fail(PA_ERR_INVALID_ARG, "pa_seq_block_table: bad argument");
  if (table) *table = p->host.table(seq_id);
  if (n_blocks) *n_blocks = p->host.table_size(seq_id);
  return PA_OK;
}

static int upload_tables(pa_pool* p, cudaStream_t st) {
  const int mb = p->host.max_blocks_per_seq();
  for (const auto& d : p->host.dirty()) {
    if (d.hi <= d.lo) continue;
    PA_CUDA(cudaMemcpyAsync(p->d_tables + (size_t)d.seq * mb + d.lo,
                            p->host.all_tables() + (size_t)d.seq * mb + d.lo,
                            (size_t)(d.hi - d.lo) * sizeof(int32_t), cudaMemcpyHostToDevice, st));
  }
  p->host.clear_dirty();
  return PA_OK;
}

int pa_batch_set_sharded(pa_pool* p, const int32_t* seq_ids, const int32_t* new_tokens,
                         const int32_t* q_rows, const int32_t* q_pos, const int32_t* kv_pos_offset,
                         int n_seqs, void* stream) {
  if (!p || !seq_ids) return fail(PA_ERR_INVALID_ARG, "pa_batch_set: NULL argument");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_batch_set: host-only pool");
  if (n_seqs <= 0 || n_seqs > p->host.max_seqs())
    return fail(PA_ERR_INVALID_ARG, "pa_batch_set: n_seqs %d outside 1..%d", n_seqs, p->host.max_seqs());
  std::vector<pa::BatchEntry> b(n_seqs);
  int kv_row = 0, q_row = 0, max_new = 0, max_blocks = 0;
  for (int i = 0; i < n_seqs; i++) {
    if (!p->host.valid(seq_ids[i])) return fail(PA_ERR_INVALID_ARG, "pa_batch_set: unknown sequence %d", seq_ids[i]);
    const int nn = new_tokens ? new_tokens[i] : 1;
    const int len = p->host.length(seq_ids[i]);
    if (nn < 0 || nn > len)
      return fail(PA_ERR_INVALID_ARG, "pa_batch_set: sequence %d has %d tokens, cannot append %d", seq_ids[i], len, nn);
    const int nq = q_rows ? q_rows[i] : nn;
    const int off = kv_pos_offset ? kv_pos_offset[i] : 0;
    const int qp = q_pos ? q_pos[i] : off + len - nn;
    if (nq < 0 || qp < 0 || off < 0) return fail(PA_ERR_INVALID_ARG, "pa_batch_set: negative row count or position");
    b[i] = {seq_ids[i], len, nn, kv_row, nq, q_row, qp, off};
    kv_row += nn;
    q_row += nq;
    if (nn > max_new) max_new = nn;
    if (nq > max_new) max_new = nq;
    if (p->host.table_size(seq_ids[i]) > max_blocks) max_blocks = p->host.table_size(seq_ids[i]);
  }
  DeviceGuard g(p->device);
  cudaStream_t st = (cudaStream_t)stream;
  int r = upload_tables(p, st);
  if (r != PA_OK) return r;
  // pageable source: the runtime stages it before returning, so `b` may die
  PA_CUDA(cudaMemcpyAsync(p->d_batch, b.data(), (size_t)n_seqs * sizeof(pa::BatchEntry),
                          cudaMemcpyHostToDevice, st));
  p->batch.swap(b);
  p->max_new = max_new;
  p->total_rows = q_row;
  p->max_kv_blocks = max_blocks;
  return PA_OK;
}

int pa_batch_set(pa_pool* p, const int32_t* seq_ids, const int32_t* new_tokens, int n_seqs,
                 void* stream) {
  return pa_batch_set_sharded(p, seq_ids, new_tokens, nullptr, nullptr, nullptr, n_seqs, stream);
}

int pa_append(pa_pool* p, int layer, const void* q_in, const void* k_in, const void* v_in,
              const float* cos_table, const float* sin_table, void* q_out, void* stream) {
  if (!p || !cos_table || !sin_table) return fail(PA_ERR_INVALID_ARG, "pa_append: NULL argument");
  if (q_out && !q_in) return fail(PA_ERR_INVALID_ARG, "pa_append: q_out given without q_in");
  if (!k_in || !v_in)
    for (const auto& e : p->batch)
      if (e.n_new > 0) return fail(PA_ERR_INVALID_ARG, "pa_append: the batch appends tokens but k_in/v_in is NULL");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_append: host-only pool");
  if (layer < 0 || layer >= p->num_layers) return fail(PA_ERR_INVALID_ARG, "pa_append: layer %d out of range", layer);
  if (p->batch.empty()) return fail(PA_ERR_STATE, "pa_append: no active batch (call pa_batch_set)");
  DeviceGuard g(p->device);
  pa::AppendParams a;
  a.q_in = (const __nv_bfloat16*)q_in;
  a.k_in = (const __nv_bfloat16*)k_in;
  a.v_in = (const __nv_bfloat16*)v_in;
  a.q_out = (__nv_bfloat16*)q_out;
  a.cos_table = cos_table;
  a.sin_table = sin_table;
  a.storage = p->storage + (size_t)layer * p->layer_bytes;
  a.tables = p->d_tables;
  a.batch = p->d_batch;
  a.status = p->d_status;
  a.kv_heads = p->kv_heads;
  a.num_blocks = p->host.num_blocks();
  a.max_blocks_per_seq = p->host.max_blocks_per_seq();
  PA_CUDA(pa::launch_append(a, (int)p->batch.size(), p->max_new, (cudaStream_t)stream));
  return PA_OK;
}

// Blocks per split-KV chunk: aim at about two CTAs per resident slot
// (3 CTAs of 4 warps per SM on 148 SMs), at least one block per warp and
// stage, and never more chunks than the workspace can hold.
// Split-KV plan of the active batch.  Measured on B200: CTAs that all start and
// end together cost a ramp-up and a drain per wave, so the best plan is ONE
// wave — 8-warp CTAs, one per SM, each streaming a long run of blocks.  When
// the batch has more (sequence, KV head) pairs than SMs that is impossible and
// smaller CTAs (4 warps, 3 per SM) in several ragged waves are used instead.
struct DecodePlan {
  int warps, stages, chunk_blocks;
};

static long long plan_ctas(const pa_pool* p, int cb) {
  long long n = 0;
  for (const auto& e : p->batch) {
    const int nb = (e.kv_len + pa::kBlockTokens - 1) / pa::kBlockTokens;
    n += nb > 0 ? (nb + cb - 1) / cb : 1;
  }
  return n * p->kv_heads;
}

// Combining CTAs per (sequence, head) in the one-launch step.  A combining CTA needs about 4 us
// per layer (wait, combine, exchange); the streaming CTAs finish a layer in (bytes per layer) /
// (HBM rate).  When a layer streams for less than that, 2 or 4 combining CTAs take the layers in
// turn; when it streams for longer a second one would only take SMs from the stream.  The count is
// 1, 2 or 4: the exchange's word slots must be a multiple of it (kXchgWordSlots).
static int step_combiners(const pa_pool* p) {
  if (p->step_combiners_override > 0) return p->step_combiners_override;
  long long tokens = 0;
  for (const auto& e : p->batch) tokens += e.kv_len;
  const long long bytes_per_layer = tokens * p->kv_heads * 2 * pa::kHeadDim * 2;
  // With a cross-rank exchange a combining CTA also pushes the pair's words to the peers and waits for
  // theirs: one CTA per pair keeps up with about 20 us of streaming per layer (2 GPUs on 131072 tokens:
  // 12 907 GB/s with one, 12 757 with two), not with 10 us (4 GPUs: 22 494 with one, 23 283 with two).
  const long long one = p->step_has_exchange ? 100ll * 1000 * 1000 : 48ll * 1000 * 1000;
  if (bytes_per_layer > one) return 1;  // without exchange: more than about 8 us of streaming
  if (bytes_per_layer > 16ll * 1000 * 1000) return 2;
  return 4;
}

static DecodePlan pick_plan(const pa_pool* p) {
  DecodePlan plan{p->decode_warps, p->decode_stages, p->chunk_blocks_override};
  const int sms = p->sm_count > 0 ? p->sm_count : 148;
  const long long pairs = (long long)p->batch.size() * p->kv_heads;
  if (plan.warps == 0) {
    plan.warps = pairs <= sms ? 8 : 4;
    plan.stages = 4;
  }
  if (plan.chunk_blocks == 0) {
    if (pairs <= sms) {
      // Smallest chunk for which every CTA is resident at once.  One or two SMs per
      // (sequence, head) pair stay free: the CTA that combines a pair outlives
      // the others by the combine and the exchange, and in a multi-layer step
      // the next layer's CTAs (programmatic dependent launch) would otherwise
      // queue behind it — the whole step then advances at stream + combine
      // instead of at the stream rate.
      const int budget = pairs * 4 <= sms ? sms - step_combiners(p) * (int)pairs : sms;
      int lo = 1, hi = p->max_kv_blocks > 1 ? p->max_kv_blocks : 1;
      while (lo < hi) {
        const int mid = (lo + hi) / 2;
        if (plan_ctas(p, mid) <= budget) hi = mid; else lo = mid + 1;
      }
      plan.chunk_blocks = lo;
    } else {
      long long total = 0;
      for (const auto& e : p->batch) total += (e.kv_len + pa::kBlockTokens - 1) / pa::kBlockTokens;
      total *= p->kv_heads;
      long long cb = total / ((long long)sms * 3 * 4);
      plan.chunk_blocks = (int)(cb < 32 ? 32 : cb);
    }
  }
  return plan;
}

// x != nullptr: sequence-range sharded decode.  with_merge == false only pushes
// the partials; the merge of that step is then launched by pa_exchange_merge.
// Inputs of the fused append (pa_decode_step): q is then the un-rotated query.
struct FusedAppend {
  const void* k_new;
  const void* v_new;
  const float* cos_table;
  const float* sin_table;
  void* q_rot_out;
  int pdl;  // 1: may overlap the previous layer's decode kernel; 2: waits for the kernel that made q, k, v
};

// The append can ride inside the decode kernel when every sequence brings one
// query row (row i = batch entry i) and at most one new token.
static bool can_fuse_append(const pa_pool* p) {
  int i = 0;
  for (const auto& e : p->batch) {
    if (e.n_q != 1 || e.q_row_off != i || e.n_new > 1) return false;
    i++;
  }
  return true;
}

static int decode_impl(pa_pool* p, int layer, const void* q, void* out, int64_t out_stride, float* out_f32,
                       float* lse, float scale, void* stream, pa_exchange* x, bool with_merge = true,
                       const FusedAppend* fz = nullptr, pa_gather* hg = nullptr, int hg_layer = 0,
                       pa::DecodeParams* capture = nullptr, DecodePlan* plan_out = nullptr) {
  if (!p || !q) return fail(PA_ERR_INVALID_ARG, "pa_decode: NULL argument");
  if (!out && !out_f32 && !(x && !with_merge) && !hg) return fail(PA_ERR_INVALID_ARG, "pa_decode: no output buffer");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_decode: host-only pool");
  if (layer < 0 || layer >= p->num_layers) return fail(PA_ERR_INVALID_ARG, "pa_decode: layer %d out of range", layer);
  if (p->batch.empty()) return fail(PA_ERR_STATE, "pa_decode: no active batch (call pa_batch_set)");
  if (out && out_stride < (int64_t)p->kv_heads * pa::kGroup * pa::kHeadDim)
    return fail(PA_ERR_INVALID_ARG, "pa_decode: out_stride %lld shorter than a row", (long long)out_stride);
  const int n_seqs = (int)p->batch.size();
  DecodePlan plan = pick_plan(p);
  int cb = plan.chunk_blocks;
  // the combine keeps 48 bytes per chunk in the (then idle) tile ring
  const int scratch_chunks = plan.warps * plan.stages * pa::kPairBytes / 48;
  auto chunks_for = [&](int c) { int m = (p->max_kv_blocks + c - 1) / c; return m < 1 ? 1 : m; };
  int max_chunks = chunks_for(cb);
  while (max_chunks > 1 && ((long long)max_chunks * p->kv_heads * n_seqs > kWsItems || max_chunks > scratch_chunks)) {
    cb *= 2;
    max_chunks = chunks_for(cb);
  }
  DeviceGuard g(p->device);
  // Cluster form (the kernel of one layer, short contexts): the chunks of a (sequence, head) are one
  // thread-block cluster and combine through distributed shared memory — no workspace round trip, no
  // arrival counter, no last-arriver loads, which at a few thousand tokens cost several times the
  // streaming itself.  The planner takes it when every cluster can be resident at once and a chunk
  // still holds a few blocks; long contexts keep the workspace form, whose chunks use every SM.
  int cluster = 0;
  if (!capture && p->cluster_mode >= 0 && p->chunk_blocks_override == 0) {
    const int sms = p->sm_count > 0 ? p->sm_count : 148;
    const long long pairs = (long long)n_seqs * p->kv_heads;
    int want = p->cluster_mode;
    // measured on B200 (batch 1, one kernel per layer): at 1024 tokens clusters of 8 take 7.2 us
    // against 10.9 us for the workspace form, at 4096 tokens 10.7 against 11.2, at 16384 tokens 18.4
    // against 14.3 (64 streaming CTAs instead of 144); clusters of 16 are slower at every length
    if (want == 0 && !hg && p->max_kv_blocks <= 320) {
      want = 8;
      while (want >= 2 && pairs * want > sms) want /= 2;
      while (want >= 2 && p->max_kv_blocks < 4 * want) want /= 2;  // a chunk keeps at least 4 blocks
    }
    if (want >= 2) {
      const int limit = pa::decode_cluster_limit(plan.warps, plan.stages);
      while (want > limit && want >= 2) want /= 2;
    }
    if (want >= 2 && want <= 16 && p->max_kv_blocks >= want) {
      cb = (p->max_kv_blocks + want - 1) / want;
      max_chunks = want;  // CTAs beyond a sequence's own chunk count idle through the two cluster meetings
      cluster = want;
    }
  }
  pa::DecodeParams d;
  d.cluster = cluster;
  d.q = (const __nv_bfloat16*)q;
  d.out = (__nv_bfloat16*)out;
  d.out_f32 = out_f32;
  d.lse = lse;
  d.storage = p->storage + (size_t)layer * p->layer_bytes;
  d.tables = p->d_tables;
  d.batch = p->d_batch;
  d.ws_acc = p->ws_acc;
  d.ws_ml = p->ws_ml;
  d.ws_count = p->ws_count;
  d.status = p->d_status;
  d.out_stride = out_stride;
  d.scale_log2 = scale * pa::kLog2e;
  d.kv_heads = p->kv_heads;
  d.num_blocks = p->host.num_blocks();
  d.max_blocks_per_seq = p->host.max_blocks_per_seq();
  d.chunk_blocks = cb;
  d.max_chunks = max_chunks;
  if (fz) {
    d.fuse = 1;
    d.k_new = (const __nv_bfloat16*)fz->k_new;
    d.v_new = (const __nv_bfloat16*)fz->v_new;
    d.cos_table = fz->cos_table;
    d.sin_table = fz->sin_table;
    d.storage_w = p->storage + (size_t)layer * p->layer_bytes;
    d.q_rot_out = fz->q_rot_out == q ? nullptr : (__nv_bfloat16*)fz->q_rot_out;
    d.pdl = fz->pdl;
  }
  if (hg && !pa::gather_fill(hg, hg_layer, n_seqs, p->kv_heads, d))
    return fail(PA_ERR_INVALID_ARG, "pa_decode_step_gathered: the gather was created for another batch, layer count or head count, or is not connected");
  if (plan_out) *plan_out = plan;
  if (!x) {
    if (capture) {
      *capture = d;
      return PA_OK;
    }
    PA_CUDA(pa::launch_decode(d, n_seqs, plan.warps, plan.stages, (cudaStream_t)stream));
    return PA_OK;
  }
  // sequence-range sharding: partials go to every rank's receive buffer, the
  // merge kernel writes the bf16 rows once all ranks' partials have landed
  if (pa::exchange_rows(x) != n_seqs * p->kv_heads * pa::kGroup || pa::exchange_groups(x) != n_seqs * p->kv_heads)
    return fail(PA_ERR_INVALID_ARG, "pa_decode_step_sharded: the exchange was created for another batch size or head count");
  pa::ExchangeMergeParams m;
  if (!pa::exchange_fill(x, d, m)) return fail(PA_ERR_STATE, "pa_decode_step_sharded: exchange not connected");
  d.out = nullptr;
  d.out_f32 = nullptr;
  d.lse = nullptr;
  m.out = (__nv_bfloat16*)out;
  m.out_stride = out_stride;
  m.status = p->d_status;
  m.q_heads = p->kv_heads * pa::kGroup;
  if (with_merge) {
    // the combining CTA of each (sequence, KV head) waits for the other ranks
    // and merges its rows itself: no second launch
    d.xchg_out = (__nv_bfloat16*)out;
    d.xchg_out_stride = out_stride;
  }
  if (capture) {
    *capture = d;
    return PA_OK;
  }
  PA_CUDA(pa::launch_decode(d, n_seqs, plan.warps, plan.stages, (cudaStream_t)stream));
  return PA_OK;
}

// Launch descriptor of the layers [layer_begin, layer_end) of a fused decode step as ONE
// cooperative launch (decode_step_kernel), when the batch fits `sm_budget` SMs: every CTA resident
// at once (streaming CTAs + one or two combining CTAs per (sequence, head)), a workspace slice per
// layer.  Returns 1 when sp/plan describe the launch, 0 when the caller should run the layers one
// kernel each, < 0 on error.  With an exchange it has taken ONE step number (exchange_fill); the
// caller adds layers - 1 more when it launches, or hands the one back (exchange_unfill).
static int build_step_params(pa_pool* p, pa_exchange* x, int layer_begin, int layer_end, const void* q_in,
                             const void* k_in, const void* v_in, int64_t q_layer_stride, int64_t kv_layer_stride,
                             const float* cos_table, const float* sin_table, void* q_rot, void* out,
                             int64_t out_stride, int64_t out_layer_stride, float* lse, float scale, int sm_budget,
                             pa::DecodeStepParams& sp, DecodePlan& plan) {
  const int layers = layer_end - layer_begin;
  if (layers < 2 || layers > pa::kMaxStepLayers || p->device < 0 || p->batch.empty() || p->no_step_kernel ||
      p->no_layer_overlap)
    return 0;
  const int n_seqs = (int)p->batch.size();
  if (n_seqs > pa::kMaxStepSeqs) return 0;
  const int sms = sm_budget;
  const long long pairs = (long long)n_seqs * p->kv_heads;
  if (pairs * 4 > sms) return 0;
  const FusedAppend fz{k_in, v_in, cos_table, sin_table, q_rot, 0};
  const int saved_sms = p->sm_count;
  p->sm_count = sms;  // the split plan aims at the SMs this step may use
  p->step_has_exchange = x != nullptr;
  int r = decode_impl(p, layer_begin, q_in, out, out_stride, nullptr, lse, scale, nullptr, x, true, &fz, nullptr, 0,
                      &sp.base, &plan);
  p->sm_count = saved_sms;
  if (r != PA_OK) return r < 0 ? r : -r;
  if (!((plan.warps == 8 && (plan.stages == 4 || plan.stages == 3)) || (plan.warps == 4 && plan.stages == 4)) ||
      sp.base.max_chunks < 1) {
    if (x) pa::exchange_unfill(x);
    return 0;
  }
  sp.layers = layers;
  sp.n_seqs = n_seqs;
  sp.q_layer_stride = q_layer_stride;
  sp.kv_layer_stride = kv_layer_stride;
  sp.out_layer_stride = out_layer_stride;
  sp.lse_layer_stride = (long long)n_seqs * p->kv_heads * pa::kGroup;
  sp.layer_bytes = p->layer_bytes;
  sp.ws_layer_items = n_seqs * p->kv_heads * sp.base.max_chunks;
  {
    int first = 0;
    for (int z = 0; z < n_seqs; z++) {
      const int n_blocks = (p->batch[z].kv_len + pa::kBlockTokens - 1) / pa::kBlockTokens;
      int chunks = (n_blocks + sp.base.chunk_blocks - 1) / sp.base.chunk_blocks;
      if (chunks < 1) chunks = 1;
      sp.seq_first[z] = (unsigned short)first;
      first += chunks * p->kv_heads;
    }
    sp.seq_first[n_seqs] = (unsigned short)first;
    sp.n_stream = first;
  }
  // one CTA per SM (the ring of an 8-warp CTA fills most of an SM's shared memory); two combining
  // CTAs per pair when they fit
  sp.combiners = step_combiners(p);
  while (sp.combiners > 1 && sp.n_stream + sp.combiners * n_seqs * p->kv_heads > sms) sp.combiners /= 2;
  if (pa::decode_step_ctas(sp) > sms || (long long)sp.ws_layer_items * layers > kWsItems) {
    if (x) pa::exchange_unfill(x);
    return 0;
  }
  sp.base.pdl = 0;
  return 1;
}

static int try_step_launch(pa_pool* p, pa_exchange* x, int layer_begin, int layer_end, const void* q_in,
                           const void* k_in, const void* v_in, int64_t q_layer_stride, int64_t kv_layer_stride,
                           const float* cos_table, const float* sin_table, void* q_rot, void* out,
                           int64_t out_stride, int64_t out_layer_stride, float* lse, float scale, void* stream) {
  pa::DecodeStepParams sp;
  DecodePlan plan{};
  const int sms = p->sm_count > 0 ? p->sm_count : 148;
  const int t = build_step_params(p, x, layer_begin, layer_end, q_in, k_in, v_in, q_layer_stride, kv_layer_stride,
                                  cos_table, sin_table, q_rot, out, out_stride, out_layer_stride, lse, scale, sms, sp,
                                  plan);
  if (t != 1) return t;
  if (x) pa::exchange_advance(x, sp.layers - 1);  // layer l is exchange step seq0 + l
  DeviceGuard g(p->device);
  cudaError_t e = pa::launch_decode_step(sp, plan.warps, plan.stages, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    fail(PA_ERR_CUDA, "decode step launch: %s", cudaGetErrorString(e));
    return -PA_ERR_CUDA;
  }
  p->step_launches++;
  return 1;
}

int pa_decode_push(pa_pool* p, pa_exchange* x, int layer, const void* q, float scale, void* stream) {
  if (!x) return fail(PA_ERR_INVALID_ARG, "pa_decode_push: NULL exchange");
  return decode_impl(p, layer, q, nullptr, 0, nullptr, nullptr, scale, stream, x, false);
}

int pa_exchange_merge(pa_pool* p, pa_exchange* x, void* out, int64_t out_stride, void* stream) {
  if (!p || !x || !out) return fail(PA_ERR_INVALID_ARG, "pa_exchange_merge: NULL argument");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_exchange_merge: host-only pool");
  pa::ExchangeMergeParams m;
  if (!pa::exchange_current(x, m)) return fail(PA_ERR_STATE, "pa_exchange_merge: no exchange step in flight");
  if (out_stride < (int64_t)p->kv_heads * pa::kGroup * pa::kHeadDim)
    return fail(PA_ERR_INVALID_ARG, "pa_exchange_merge: out_stride shorter than a row");
  DeviceGuard g(p->device);
  m.out = (__nv_bfloat16*)out;
  m.out_stride = out_stride;
  m.status = p->d_status;
  m.q_heads = p->kv_heads * pa::kGroup;
  PA_CUDA(pa::launch_exchange_merge(m, (cudaStream_t)stream));
  return PA_OK;
}

int pa_decode(pa_pool* p, int layer, const void* q, void* out, int64_t out_stride, float* out_f32,
              float* lse, float scale, void* stream) {
  return decode_impl(p, layer, q, out, out_stride, out_f32, lse, scale, stream, nullptr);
}

int pa_gather_wait(pa_pool* p, pa_gather* g, void* stream, void** rows) {
  if (!p || !g || p->device < 0) return fail(PA_ERR_INVALID_ARG, "pa_gather_wait: bad argument");
  DeviceGuard guard(p->device);
  PA_CUDA(pa::gather_wait(g, p->d_status, (cudaStream_t)stream, rows));
  return PA_OK;
}

int pa_decode_step_gathered(pa_pool* p, pa_gather* g, const void* q_in, const void* k_in, const void* v_in,
                            int64_t q_layer_stride, int64_t kv_layer_stride, const float* cos_table,
                            const float* sin_table, void* q_rot, float scale, int wait, void* stream,
                            void** rows) {
  if (!p || !g || !q_in || !k_in || !v_in || !q_rot || !cos_table || !sin_table)
    return fail(PA_ERR_INVALID_ARG, "pa_decode_step_gathered: NULL argument");
  const int layers = pa::gather_layers(g);
  if (layers > p->num_layers) return fail(PA_ERR_INVALID_ARG, "pa_decode_step_gathered: the pool has fewer layers than the gather");
  if (!can_fuse_append(p)) return fail(PA_ERR_UNSUPPORTED, "pa_decode_step_gathered: needs one query row and at most one new token per sequence");
  if (!pa::gather_begin(g)) return fail(PA_ERR_STATE, "pa_decode_step_gathered: gather not connected");
  for (int l = 0; l < layers; l++) {
    const __nv_bfloat16* qi = (const __nv_bfloat16*)q_in + (size_t)l * q_layer_stride;
    const __nv_bfloat16* ki = (const __nv_bfloat16*)k_in + (size_t)l * kv_layer_stride;
    const __nv_bfloat16* vi = (const __nv_bfloat16*)v_in + (size_t)l * kv_layer_stride;
    __nv_bfloat16* qr = (__nv_bfloat16*)q_rot + (size_t)l * q_layer_stride;
    const FusedAppend fz{ki, vi, cos_table, sin_table, qr, l > 0 && !p->no_layer_overlap ? 1 : 0};
    int r = decode_impl(p, l, qi, nullptr, 0, nullptr, nullptr, scale, stream, nullptr, true, &fz, g, l);
    if (r != PA_OK) return r;
  }
  if (wait) return pa_gather_wait(p, g, stream, rows);
  return PA_OK;
}

int pa_decode_step_sharded(pa_pool* p, pa_exchange* x, int layer_begin, int layer_end, const void* q_in,
                           const void* k_in, const void* v_in, int64_t q_layer_stride,
                           int64_t kv_layer_stride, const float* cos_table, const float* sin_table,
                           void* q_rot, void* out, int64_t out_stride, int64_t out_layer_stride,
                           float scale, void* stream) {
  if (!p || !x || !q_in || !q_rot || !out) return fail(PA_ERR_INVALID_ARG, "pa_decode_step_sharded: NULL argument");
  if (layer_begin < 0 || layer_end > p->num_layers || layer_begin > layer_end)
    return fail(PA_ERR_INVALID_ARG, "pa_decode_step_sharded: layers [%d, %d) out of range", layer_begin, layer_end);
  // fused when the batch allows it; k_in/v_in may only be missing if nothing is appended
  bool fuse = cos_table && sin_table && can_fuse_append(p);
  for (const auto& e : p->batch)
    if (e.n_new > 0 && (!k_in || !v_in)) return fail(PA_ERR_INVALID_ARG, "decode step: the batch appends tokens but k_in/v_in is NULL");
  if (fuse && q_rot != q_in) {
    const int t = try_step_launch(p, x, layer_begin, layer_end, q_in, k_in, v_in, q_layer_stride, kv_layer_stride,
                                  cos_table, sin_table, q_rot, out, out_stride, out_layer_stride, nullptr, scale, stream);
    if (t < 0) return -t;
    if (t == 1) return PA_OK;
  }
  for (int l = layer_begin; l < layer_end; l++) {
    const int i = l - layer_begin;
    const __nv_bfloat16* qi = (const __nv_bfloat16*)q_in + (size_t)i * q_layer_stride;
    const __nv_bfloat16* ki = k_in ? (const __nv_bfloat16*)k_in + (size_t)i * kv_layer_stride : nullptr;
    const __nv_bfloat16* vi = v_in ? (const __nv_bfloat16*)v_in + (size_t)i * kv_layer_stride : nullptr;
    __nv_bfloat16* qr = (__nv_bfloat16*)q_rot + (size_t)i * q_layer_stride;
    __nv_bfloat16* o = (__nv_bfloat16*)out + (size_t)i * out_layer_stride;
    int r;
    if (fuse) {
      // one kernel per layer: RoPE(Q), RoPE(K) + append, decode, exchange, merge
      const FusedAppend fz{ki, vi, cos_table, sin_table, qr, l > layer_begin && !p->no_layer_overlap ? 1 : 0};
      r = decode_impl(p, l, qi, o, out_stride, nullptr, nullptr, scale, stream, x, true, &fz);
    } else {
      r = pa_append(p, l, qi, ki, vi, cos_table, sin_table, qr, stream);
      if (r == PA_OK) r = decode_impl(p, l, qr, o, out_stride, nullptr, nullptr, scale, stream, x);
    }
    if (r != PA_OK) return r;
  }
  return PA_OK;
}

int pa_decode_step_sharded_colocated(pa_pool* const* pools, pa_exchange* const* xs, int world, int layer_begin,
                                     int layer_end, const void* const* q_in, const void* const* k_in,
                                     const void* const* v_in, int64_t q_layer_stride, int64_t kv_layer_stride,
                                     const float* cos_table, const float* sin_table, void* const* q_rot,
                                     void* const* out, int64_t out_stride, int64_t out_layer_stride, float scale,
                                     void* stream) {
  if (!pools || !xs || !q_in || !q_rot || !out || !cos_table || !sin_table)
    return fail(PA_ERR_INVALID_ARG, "pa_decode_step_sharded_colocated: NULL argument");
  if (world < 1 || world > pa::kMaxColocatedRanks)
    return fail(PA_ERR_UNSUPPORTED, "pa_decode_step_sharded_colocated: 1..%d ranks per GPU", pa::kMaxColocatedRanks);
  pa::ColocatedStepParams cp;
  cp.world = world;
  const int dev = pools[0] ? pools[0]->device : -1;
  if (dev < 0) return fail(PA_ERR_STATE, "pa_decode_step_sharded_colocated: host-only pool");
  const int sms = pools[0]->sm_count > 0 ? pools[0]->sm_count : 148;
  int built = 0, rc = PA_OK;
  for (int r = 0; r < world && rc == PA_OK; r++) {
    pa_pool* p = pools[r];
    if (!p || !xs[r] || !q_in[r] || !q_rot[r] || !out[r] || p->device != dev) {
      rc = fail(PA_ERR_INVALID_ARG, "pa_decode_step_sharded_colocated: rank %d: NULL argument or a pool of another device", r);
      break;
    }
    if (layer_begin < 0 || layer_end > p->num_layers || layer_begin > layer_end) {
      rc = fail(PA_ERR_INVALID_ARG, "pa_decode_step_sharded_colocated: layers [%d, %d) out of range", layer_begin, layer_end);
      break;
    }
    const void* ki = k_in ? k_in[r] : nullptr;
    const void* vi = v_in ? v_in[r] : nullptr;
    bool ok = can_fuse_append(p) && q_rot[r] != q_in[r];
    for (const auto& e : p->batch)
      if (e.n_new > 0 && (!ki || !vi)) ok = false;
    if (!ok) {
      rc = fail(PA_ERR_UNSUPPORTED, "pa_decode_step_sharded_colocated: rank %d: needs one query row and at most one new token "
                                    "per sequence, k_in/v_in where tokens are appended, and q_rot apart from q_in", r);
      break;
    }
    DecodePlan plan{};
    const int t = build_step_params(p, xs[r], layer_begin, layer_end, q_in[r], ki, vi, q_layer_stride, kv_layer_stride,
                                    cos_table, sin_table, q_rot[r], out[r], out_stride, out_layer_stride, nullptr, scale,
                                    sms / world, cp.rank[r], plan);
    if (t < 0) {
      rc = -t;
      break;
    }
    if (t == 1) built++;  // this rank holds one exchange step number now
    if (t == 0 || plan.warps != 8 || plan.stages != 4) {
      rc = fail(PA_ERR_UNSUPPORTED, "pa_decode_step_sharded_colocated: rank %d's step does not fit %d SMs as one launch of "
                                    "8-warp CTAs (at least 2 layers; fewer chunks via pa_pool_set_decode_chunk_blocks)",
                r, sms / world);
      break;
    }
    const int ctas = pa::decode_step_ctas(cp.rank[r]);
    if (ctas > cp.ctas_per_rank) cp.ctas_per_rank = ctas;
  }
  if (rc == PA_OK && cp.world * cp.ctas_per_rank > sms)
    rc = fail(PA_ERR_UNSUPPORTED, "pa_decode_step_sharded_colocated: %d CTAs do not fit %d SMs", cp.world * cp.ctas_per_rank, sms);
  if (rc != PA_OK) {
    for (int r = 0; r < built; r++) pa::exchange_unfill(xs[r]);
    return rc;
  }
  for (int r = 0; r < world; r++) pa::exchange_advance(xs[r], layer_end - layer_begin - 1);
  DeviceGuard g(dev);
  PA_CUDA(pa::launch_decode_step_colocated(cp, (cudaStream_t)stream));
  for (int r = 0; r < world; r++) pools[r]->step_launches++;
  return PA_OK;
}

// One decode step through the attention blocks of layers [layer_begin, layer_end) with the true
// data flow: per layer three launches — projections (RMSNorm in front when a norm weight is given),
// decode attention with the append fused in, output projection (+ residual) — chained by
// programmatic dependent launch: each kernel starts the part of its work that does not depend on
// the kernel in front (weight loads, cache copies) while that kernel finishes, and waits before it
// reads its output.  All intermediate rows live in the pool's step workspace.
static int step_layers(pa_pool* p, pa_exchange* x, int layer_begin, int layer_end, const pa_attention_weights* w,
                       const pa_ffn_weights* f, const void* x_in, void* x_out, int add_residual,
                       const float* cos_table, const float* sin_table, float scale, void* stream,
                       bool follows_own_kernel = false) {
  if (!p || !w || !x_in || !x_out || !cos_table || !sin_table)
    return fail(PA_ERR_INVALID_ARG, "pa_attention_step: NULL argument");
  if (!w->wq || !w->wk || !w->wv || !w->wo) return fail(PA_ERR_INVALID_ARG, "pa_attention_step: NULL weight");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_attention_step: host-only pool");
  if (layer_begin < 0 || layer_end > p->num_layers || layer_begin >= layer_end)
    return fail(PA_ERR_INVALID_ARG, "pa_attention_step: layers [%d, %d) out of range", layer_begin, layer_end);
  if (p->batch.empty()) return fail(PA_ERR_STATE, "pa_attention_step: no active batch (call pa_batch_set)");
  const int rows = (int)p->batch.size();
  if (rows > kMaxStepRows) return fail(PA_ERR_UNSUPPORTED, "pa_attention_step: at most %d sequences per step", kMaxStepRows);
  if (!can_fuse_append(p))
    return fail(PA_ERR_UNSUPPORTED, "pa_attention_step: needs one query row and at most one new token per sequence");
  const int hidden = w->hidden;
  if (hidden < 64 || hidden > kMaxStepHidden || hidden % 64 != 0)
    return fail(PA_ERR_UNSUPPORTED, "pa_attention_step: hidden must be a multiple of 64, at most %d", kMaxStepHidden);
  if (layer_end - layer_begin > 1 && x_out == x_in)
    return fail(PA_ERR_INVALID_ARG, "pa_attention_step: x_out must not alias x_in over several layers");
  const int q_cols = p->kv_heads * pa::kGroup * pa::kHeadDim, kv_cols = p->kv_heads * pa::kHeadDim;
  __nv_bfloat16* ws = p->step_ws;
  __nv_bfloat16* q = ws;
  __nv_bfloat16* k = q + (size_t)kMaxStepRows * q_cols;
  __nv_bfloat16* v = k + (size_t)kMaxStepRows * kv_cols;
  __nv_bfloat16* q_rot = v + (size_t)kMaxStepRows * kv_cols;
  __nv_bfloat16* attn = q_rot + (size_t)kMaxStepRows * q_cols;
  __nv_bfloat16* xpp[2] = {attn + (size_t)kMaxStepRows * q_cols,
                           attn + (size_t)kMaxStepRows * q_cols + (size_t)kMaxStepRows * kMaxStepHidden};
  __nv_bfloat16* x_mid = xpp[1] + (size_t)kMaxStepRows * kMaxStepHidden;   // block input of the feed-forward block
  __nv_bfloat16* h_rows = x_mid + (size_t)kMaxStepRows * kMaxStepHidden;   // its activated rows [rows, inter]
  bool appends = false;
  for (const auto& e : p->batch) appends = appends || e.n_new > 0;
  DeviceGuard g(p->device);
  const __nv_bfloat16* cur = (const __nv_bfloat16*)x_in;
  for (int l = layer_begin; l < layer_end; l++) {
    const bool first = l == layer_begin;
    const __nv_bfloat16* norm = w->input_norm ? (const __nv_bfloat16*)w->input_norm + (size_t)l * w->norm_layer_stride : nullptr;
    const __nv_bfloat16* wq = (const __nv_bfloat16*)w->wq + (size_t)l * w->wq_layer_stride;
    const __nv_bfloat16* wk = (const __nv_bfloat16*)w->wk + (size_t)l * w->wkv_layer_stride;
    const __nv_bfloat16* wv = (const __nv_bfloat16*)w->wv + (size_t)l * w->wkv_layer_stride;
    const __nv_bfloat16* wo = (const __nv_bfloat16*)w->wo + (size_t)l * w->wo_layer_stride;
    // the first kernel of the call follows work this library knows nothing about: plain launch
    // (unless the caller is pa_decode_token, whose embedding kernel is in front)
    int r = pa::qkv_project_impl(cur, norm, 0, w->rms_eps, wq, wk, wv, q, k, v, rows, 1, hidden, q_cols, kv_cols, 0, 0, 0,
                                 0, 0, first && !follows_own_kernel ? 0 : 1, stream);
    if (r != PA_OK) return r;
    const FusedAppend fz{appends ? k : nullptr, appends ? v : nullptr, cos_table, sin_table, q_rot, 2};
    r = decode_impl(p, l, q, attn, q_cols, nullptr, nullptr, scale, stream, x, true, &fz);
    if (r != PA_OK) return r;
    __nv_bfloat16* out = l == layer_end - 1 ? (__nv_bfloat16*)x_out : xpp[(l - layer_begin) & 1];
    // with a feed-forward block behind it the attention block writes the pool's row buffer
    __nv_bfloat16* attn_out = f ? x_mid : out;
    r = pa::out_project_impl(attn, wo, add_residual ? cur : nullptr, attn_out, rows, 1, q_cols, hidden, 0, 0, 0, 0, 1, stream);
    if (r != PA_OK) return r;
    if (f) {
      const __nv_bfloat16* fn = f->ffn_norm ? (const __nv_bfloat16*)f->ffn_norm + (size_t)l * f->norm_layer_stride : nullptr;
      r = pa::ffn_impl(x_mid, fn, f->rms_eps, (const __nv_bfloat16*)f->gate + (size_t)l * f->gate_layer_stride,
                       (const __nv_bfloat16*)f->up + (size_t)l * f->up_layer_stride,
                       (const __nv_bfloat16*)f->down + (size_t)l * f->down_layer_stride, x_mid, h_rows, out, rows,
                       f->hidden, f->inter, 1, stream);
      if (r != PA_OK) return r;
    }
    cur = out;
  }
  return PA_OK;
}

int pa_attention_step(pa_pool* p, pa_exchange* x, int layer_begin, int layer_end, const pa_attention_weights* w,
                      const void* x_in, void* x_out, int add_residual, const float* cos_table,
                      const float* sin_table, float scale, void* stream) {
  return step_layers(p, x, layer_begin, layer_end, w, nullptr, x_in, x_out, add_residual, cos_table, sin_table, scale,
                     stream);
}

int pa_block_step(pa_pool* p, pa_exchange* x, int layer_begin, int layer_end, const pa_attention_weights* w,
                  const pa_ffn_weights* f, const void* x_in, void* x_out, const float* cos_table,
                  const float* sin_table, float scale, void* stream) {
  if (!f || !f->gate || !f->up || !f->down) return fail(PA_ERR_INVALID_ARG, "pa_block_step: NULL feed-forward weight");
  if (w && f->hidden != w->hidden) return fail(PA_ERR_INVALID_ARG, "pa_block_step: the two blocks disagree on hidden");
  if (f->inter > kMaxStepInter) return fail(PA_ERR_UNSUPPORTED, "pa_block_step: intermediate width above %d", kMaxStepInter);
  return step_layers(p, x, layer_begin, layer_end, w, f, x_in, x_out, 1, cos_table, sin_table, scale, stream);
}

// One decode step of the whole model for the active batch, the body of the reference's
// LlamaRuntime::decode_forward (src/runtime/llama_runtime.cu:822-945) without its blocking copies,
// its per-token cudaMalloc / cudaFree and its seven device synchronisations: token ids (on the
// device) -> embedding rows -> every layer's block (pa_block_step's chain) -> final RMSNorm +
// language-model head -> greedy token, all on `stream`, every kernel behind the first a dependent
// launch.  tokens_out may be tokens_in, so consecutive steps run without the host reading a token.
int pa_decode_token(pa_pool* p, const pa_model_weights* m, const int32_t* tokens_in, int32_t* tokens_out, void* logits,
                    const float* cos_table, const float* sin_table, float scale, int chained, void* stream) {
  if (!p || !m || !tokens_in || !tokens_out || !logits)
    return fail(PA_ERR_INVALID_ARG, "pa_decode_token: NULL argument");
  if (!m->embed_tokens || !m->attention || !m->ffn || !m->lm_head)
    return fail(PA_ERR_INVALID_ARG, "pa_decode_token: NULL weight");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_decode_token: host-only pool");
  if (p->batch.empty()) return fail(PA_ERR_STATE, "pa_decode_token: no active batch (call pa_batch_set)");
  const int rows = (int)p->batch.size();
  if (rows > kMaxStepRows) return fail(PA_ERR_UNSUPPORTED, "pa_decode_token: at most %d sequences per step", kMaxStepRows);
  const int hidden = m->attention->hidden;
  if (hidden < 64 || hidden > kMaxStepHidden || hidden % 64 != 0)
    return fail(PA_ERR_UNSUPPORTED, "pa_decode_token: hidden must be a multiple of 64, at most %d", kMaxStepHidden);
  if (m->vocab < 32 || m->vocab % 32 != 0) return fail(PA_ERR_UNSUPPORTED, "pa_decode_token: vocab must be a multiple of 32");
  const int q_cols = p->kv_heads * pa::kGroup * pa::kHeadDim, kv_cols = p->kv_heads * pa::kHeadDim;
  __nv_bfloat16* x_tok = p->step_ws + (size_t)kMaxStepRows * (3 * q_cols + 2 * kv_cols + 3 * kMaxStepHidden + kMaxStepInter);
  __nv_bfloat16* x_fin = x_tok + (size_t)kMaxStepRows * kMaxStepHidden;
  {
    DeviceGuard g(p->device);
    // chained != 0: the ids are the output of the step enqueued just before on this stream
    const int r = pa::embedding_impl(tokens_in, m->embed_tokens, x_tok, rows, hidden, m->vocab, p->d_status,
                                     chained ? 1 : 0, stream);
    if (r != PA_OK) return r;
  }
  const pa_ffn_weights* f = m->ffn;
  if (!f->gate || !f->up || !f->down) return fail(PA_ERR_INVALID_ARG, "pa_decode_token: NULL feed-forward weight");
  if (f->hidden != hidden) return fail(PA_ERR_INVALID_ARG, "pa_decode_token: the two blocks disagree on hidden");
  if (f->inter > kMaxStepInter) return fail(PA_ERR_UNSUPPORTED, "pa_decode_token: intermediate width above %d", kMaxStepInter);
  int r = step_layers(p, nullptr, 0, p->num_layers, m->attention, f, x_tok, x_fin, 1, cos_table, sin_table, scale, stream,
                      /*follows_own_kernel=*/true);
  if (r != PA_OK) return r;
  DeviceGuard g(p->device);
  r = pa::lm_head_impl(x_fin, m->final_norm, m->rms_eps, m->lm_head, logits, rows, hidden, m->vocab, 1, stream);
  if (r != PA_OK) return r;
  r = pa::argmax_impl(logits, tokens_out, rows, m->vocab, 1, stream);
  if (r != PA_OK) return r;
  return PA_OK;
}

int pa_decode_step(pa_pool* p, int layer_begin, int layer_end, const void* q_in, const void* k_in,
                   const void* v_in, int64_t q_layer_stride, int64_t kv_layer_stride,
                   const float* cos_table, const float* sin_table, void* q_rot, void* out,
                   int64_t out_stride, int64_t out_layer_stride, float* lse, float scale,
                   void* stream) {
  if (!p || !q_in || !q_rot || !out) return fail(PA_ERR_INVALID_ARG, "pa_decode_step: NULL argument");
  if (layer_begin < 0 || layer_end > p->num_layers || layer_begin > layer_end)
    return fail(PA_ERR_INVALID_ARG, "pa_decode_step: layers [%d, %d) out of range", layer_begin, layer_end);
  const int n_seqs = (int)p->batch.size();
  const int q_heads = p->kv_heads * pa::kGroup;
  // fused when the batch allows it; k_in/v_in may only be missing if nothing is appended
  bool fuse = cos_table && sin_table && can_fuse_append(p);
  for (const auto& e : p->batch)
    if (e.n_new > 0 && (!k_in || !v_in)) return fail(PA_ERR_INVALID_ARG, "decode step: the batch appends tokens but k_in/v_in is NULL");
  if (fuse && q_rot != q_in) {
    const int t = try_step_launch(p, nullptr, layer_begin, layer_end, q_in, k_in, v_in, q_layer_stride,
                                  kv_layer_stride, cos_table, sin_table, q_rot, out, out_stride, out_layer_stride,
                                  lse, scale, stream);
    if (t < 0) return -t;
    if (t == 1) return PA_OK;
  }
  for (int l = layer_begin; l < layer_end; l++) {
    const int i = l - layer_begin;
    const __nv_bfloat16* qi = (const __nv_bfloat16*)q_in + (size_t)i * q_layer_stride;
    const __nv_bfloat16* ki = k_in ? (const __nv_bfloat16*)k_in + (size_t)i * kv_layer_stride : nullptr;
    const __nv_bfloat16* vi = v_in ? (const __nv_bfloat16*)v_in + (size_t)i * kv_layer_stride : nullptr;
    __nv_bfloat16* qr = (__nv_bfloat16*)q_rot + (size_t)i * q_layer_stride;
    __nv_bfloat16* o = (__nv_bfloat16*)out + (size_t)i * out_layer_stride;
    float* lse_l = lse ? lse + (size_t)i * n_seqs * q_heads : nullptr;
    int r;
    if (fuse) {
      const FusedAppend fz{ki, vi, cos_table, sin_table, qr, l > layer_begin && !p->no_layer_overlap ? 1 : 0};
      r = decode_impl(p, l, qi, o, out_stride, nullptr, lse_l, scale, stream, nullptr, true, &fz);
    } else {
      r = pa_append(p, l, qi, ki, vi, cos_table, sin_table, qr, stream);
      if (r == PA_OK) r = pa_decode(p, l, qr, o, out_stride, nullptr, lse_l, scale, stream);
    }
    if (r != PA_OK) return r;
  }
  return PA_OK;
}

int pa_prefill(pa_pool* p, int layer, const void* q, void* out, float* lse, float scale, void* stream) {
  if (!p || !q || !out) return fail(PA_ERR_INVALID_ARG, "pa_prefill: NULL argument");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_prefill: host-only pool");
  if (layer < 0 || layer >= p->num_layers) return fail(PA_ERR_INVALID_ARG, "pa_prefill: layer %d out of range", layer);
  if (p->batch.size() != 1) return fail(PA_ERR_UNSUPPORTED, "pa_prefill: the batch must hold exactly one sequence (has %zu)", p->batch.size());
  const pa::BatchEntry& e = p->batch[0];
  if (e.n_q < 1 || e.kv_len < 1 || e.q_pos0 < 0)
    return fail(PA_ERR_INVALID_ARG, "pa_prefill: needs at least one query row and one cached token");
  DeviceGuard g(p->device);
  pa::PrefillParams a;
  a.q = (const __nv_bfloat16*)q;
  a.out = (__nv_bfloat16*)out;
  a.lse = lse;
  a.storage = p->storage + (size_t)layer * p->layer_bytes;
  a.tables = p->d_tables;
  a.batch = p->d_batch;
  a.status = p->d_status;
  const long long row = (long long)p->kv_heads * pa::kGroup * pa::kHeadDim;
  a.q_seq_stride = a.o_seq_stride = a.lse_seq_stride = 0;
  a.q_row_stride = a.o_row_stride = row;
  a.q_head_stride = a.o_head_stride = pa::kHeadDim;
  a.causal = 1;
  a.scale_log2 = scale * pa::kLog2e;
  a.kv_heads = p->kv_heads;
  a.num_blocks = p->host.num_blocks();
  a.max_blocks_per_seq = p->host.max_blocks_per_seq();
  // launch i draws items from counter i % 64 and clears counter (i + 32) % 64
  a.work = p->prefill_work + (p->prefill_launches % 64u);
  a.work_clear = p->prefill_work + ((p->prefill_launches + 32u) % 64u);
  p->prefill_launches++;
  PA_CUDA(pa::launch_prefill(a, 1, e.n_q, (cudaStream_t)stream));
  return PA_OK;
}

}  // extern "C"

namespace pa {
// Prefill of every sequence of the active batch with caller-given tensor
// strides (used by the legacy launcher, whose Q/O are head-major).
int prefill_strided(pa_pool* p, int layer, const void* q, void* out, float* lse, long long q_seq_stride,
                    long long q_row_stride, long long q_head_stride, long long o_seq_stride,
                    long long o_row_stride, long long o_head_stride, long long lse_seq_stride,
                    int causal, float scale, void* stream) {
  if (!p || !q || !out || p->device < 0 || p->batch.empty() || layer < 0 || layer >= p->num_layers)
    return fail(PA_ERR_INVALID_ARG, "prefill_strided: bad argument");
  int n_q = 0;
  for (const auto& e : p->batch) {
    if (e.n_q < 1 || e.kv_len < 1 || e.q_pos0 < 0) return fail(PA_ERR_INVALID_ARG, "prefill_strided: empty sequence");
    if (e.n_q > n_q) n_q = e.n_q;
  }
  DeviceGuard g(p->device);
  PrefillParams a;
  a.q = (const __nv_bfloat16*)q;
  a.out = (__nv_bfloat16*)out;
  a.lse = lse;
  a.storage = p->storage + (size_t)layer * p->layer_bytes;
  a.tables = p->d_tables;
  a.batch = p->d_batch;
  a.status = p->d_status;
  a.q_seq_stride = q_seq_stride;
  a.q_row_stride = q_row_stride;
  a.q_head_stride = q_head_stride;
  a.o_seq_stride = o_seq_stride;
  a.o_row_stride = o_row_stride;
  a.o_head_stride = o_head_stride;
  a.lse_seq_stride = lse_seq_stride;
  a.causal = causal;
  a.scale_log2 = scale * kLog2e;
  a.kv_heads = p->kv_heads;
  a.num_blocks = p->host.num_blocks();
  a.max_blocks_per_seq = p->host.max_blocks_per_seq();
  a.work = p->prefill_work + (p->prefill_launches % 64u);
  a.work_clear = p->prefill_work + ((p->prefill_launches + 32u) % 64u);
  p->prefill_launches++;
  PA_CUDA(launch_prefill(a, (int)p->batch.size(), n_q, (cudaStream_t)stream));
  return PA_OK;
}
}  // namespace pa

extern "C" {

int pa_merge_partials(const float* o_parts, const float* lse_parts, int n_parts, int rows, void* out,
                      float* out_f32, float* lse_out, void* stream) {
  if (!o_parts || !lse_parts || n_parts <= 0 || rows <= 0)
    return fail(PA_ERR_INVALID_ARG, "pa_merge_partials: bad argument");
  if (!out && !out_f32) return fail(PA_ERR_INVALID_ARG, "pa_merge_partials: no output buffer");
  pa::MergeParams m{o_parts, lse_parts, (__nv_bfloat16*)out, out_f32, lse_out, n_parts, rows};
  PA_CUDA(pa::launch_merge(m, (cudaStream_t)stream));
  return PA_OK;
}

int pa_gather_kv(pa_pool* p, int layer, int seq_id, void* k_out, void* v_out, int out_stride_tokens,
                 void* stream) {
  if (!p || !k_out || !v_out) return fail(PA_ERR_INVALID_ARG, "pa_gather_kv: NULL argument");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_gather_kv: host-only pool");
  if (layer < 0 || layer >= p->num_layers || !p->host.valid(seq_id))
    return fail(PA_ERR_INVALID_ARG, "pa_gather_kv: bad layer or sequence");
  const int len = p->host.length(seq_id);
  if (out_stride_tokens < len) return fail(PA_ERR_INVALID_ARG, "pa_gather_kv: out_stride_tokens %d < length %d", out_stride_tokens, len);
  DeviceGuard g(p->device);
  int r = upload_tables(p, (cudaStream_t)stream);
  if (r != PA_OK) return r;
  pa::GatherParams gp;
  gp.storage = p->storage + (size_t)layer * p->layer_bytes;
  gp.table = p->d_tables + (size_t)seq_id * p->host.max_blocks_per_seq();
  gp.k_out = (__nv_bfloat16*)k_out;
  gp.v_out = (__nv_bfloat16*)v_out;
  gp.status = p->d_status;
  gp.kv_heads = p->kv_heads;
  gp.num_blocks = p->host.num_blocks();
  gp.length = len;
  gp.out_stride = out_stride_tokens;
  PA_CUDA(pa::launch_gather(gp, (cudaStream_t)stream));
  return PA_OK;
}

// Host fp32 tables exactly as the reference builds them
// (src/runtime/llama_runtime.cu:320-451): float arithmetic throughout,
// theta 500000, Llama-3 scaling (factor 32, low 1, high 4, original context 8192).
int pa_build_rope_tables(float* cos_table, float* sin_table, int seq_len) {
  if (!cos_table || !sin_table || seq_len <= 0) return fail(PA_ERR_INVALID_ARG, "pa_build_rope_tables: bad argument");
  const float theta = 500000.0f, factor = 32.0f, low_ff = 1.0f, high_ff = 4.0f, orig = 8192.0f;
  for (int pair = 0; pair < 32; pair++) {
    const float inv_freq = 1.0f / std::pow(theta, (float)(2 * pair) / 64.0f);
    const float wavelen = 2.0f * (float)M_PI / inv_freq;
    float inv;
    if (wavelen < orig / high_ff) {
      inv = inv_freq;
    } else if (wavelen <= orig / low_ff) {
      const float smooth = (orig / wavelen - low_ff) / (high_ff - low_ff);
      inv = (1.0f - smooth) * (inv_freq / factor) + smooth * inv_freq;
    } else {
      inv = inv_freq / factor;
    }
    for (int pos = 0; pos < seq_len; pos++) {
      const float angle = (float)pos * inv;
      cos_table[(size_t)pos * 32 + pair] = std::cos(angle);
      sin_table[(size_t)pos * 32 + pair] = std::sin(angle);
    }
  }
  return PA_OK;
}

int pa_pool_check(pa_pool* p, void* stream) {
  if (!p || p->device < 0) return fail(PA_ERR_INVALID_ARG, "pa_pool_check: bad pool");
  DeviceGuard g(p->device);
  int st = 0;
  PA_CUDA(cudaMemcpyAsync(&st, p->d_status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  PA_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (st == 0) return PA_OK;
  PA_CUDA(cudaMemsetAsync(p->d_status, 0, sizeof(int), (cudaStream_t)stream));
  // a kernel that gave up may have left arrival counts behind; the next launch must find zeros
  PA_CUDA(cudaMemsetAsync(p->ws_count, 0, (size_t)p->host.max_seqs() * p->kv_heads * pa::kMaxStepLayers * sizeof(unsigned int),
                          (cudaStream_t)stream));
  if (st == pa::kStatusTimeout) return fail(PA_ERR_TIMEOUT, "a kernel gave up waiting for a bulk copy");
  return fail(PA_ERR_INVALID_ARG, "a kernel met a block id outside the pool");
}

int pa_pool_set_decode_cluster(pa_pool* p, int mode) {
  if (!p || !(mode == -1 || mode == 0 || mode == 2 || mode == 4 || mode == 8 || mode == 16))
    return fail(PA_ERR_INVALID_ARG, "pa_pool_set_decode_cluster: -1 (off), 0 (planner), 2, 4, 8 or 16");
  p->cluster_mode = mode;
  return PA_OK;
}

int pa_pool_set_decode_chunk_blocks(pa_pool* p, int chunk_blocks) {
  if (!p || chunk_blocks < 0) return fail(PA_ERR_INVALID_ARG, "pa_pool_set_decode_chunk_blocks: bad argument");
  p->chunk_blocks_override = chunk_blocks;
  return PA_OK;
}

int pa_pool_set_step_kernel(pa_pool* p, int enable) {
  if (!p) return fail(PA_ERR_INVALID_ARG, "pa_pool_set_step_kernel: NULL pool");
  p->no_step_kernel = enable == 0;
  return PA_OK;
}

int pa_pack_projection_weights(const void* w, void* packed, int hidden, int cols, void* stream) {
  if (!w || !packed || w == packed) return fail(PA_ERR_INVALID_ARG, "pa_pack_projection_weights: NULL or aliased argument");
  if (hidden < 64 || hidden % 64 != 0 || cols < 64 || cols % 64 != 0)
    return fail(PA_ERR_UNSUPPORTED, "pa_pack_projection_weights: hidden and cols must be multiples of 64");
  PA_CUDA(pa::launch_pack_weights(w, packed, hidden, cols, (cudaStream_t)stream));
  return PA_OK;
}

int pa_qkv_project_append(pa_pool* p, int layer, const void* x, const void* wq, const void* wk, const void* wv,
                          const float* cos_table, const float* sin_table, void* q_out, int hidden, void* stream) {
  if (!p || !x || !wq || !wk || !wv || !cos_table || !sin_table || !q_out)
    return fail(PA_ERR_INVALID_ARG, "pa_qkv_project_append: NULL argument");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_qkv_project_append: host-only pool");
  if (layer < 0 || layer >= p->num_layers) return fail(PA_ERR_INVALID_ARG, "pa_qkv_project_append: layer %d out of range", layer);
  if (p->batch.empty()) return fail(PA_ERR_STATE, "pa_qkv_project_append: no active batch (call pa_batch_set)");
  if (hidden < 64 || hidden % 64 != 0) return fail(PA_ERR_UNSUPPORTED, "pa_qkv_project_append: hidden must be a multiple of 64");
  if (p->kv_heads % 4 != 0)
    return fail(PA_ERR_UNSUPPORTED, "pa_qkv_project_append: needs a multiple of 4 KV heads per pool (256-column tiles)");
  int rows = 0;
  for (const auto& e : p->batch) {
    if (e.n_q != e.n_new || e.q_row_off != e.kv_row_off)
      return fail(PA_ERR_UNSUPPORTED, "pa_qkv_project_append: every sequence must bring the same rows as queries and as new tokens");
    rows += e.n_new;
  }
  if (rows == 0) return PA_OK;
  DeviceGuard g(p->device);
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return fail(PA_ERR_INVALID_ARG, "pa_qkv_project_append: x must be 16-byte aligned");
  pa::QkvGemmParams a;
  a.x = (const __nv_bfloat16*)x;
  a.wq = (const __nv_bfloat16*)wq;
  a.wk = (const __nv_bfloat16*)wk;
  a.wv = (const __nv_bfloat16*)wv;
  a.q_out = (__nv_bfloat16*)q_out;
  a.storage = p->storage + (size_t)layer * p->layer_bytes;
  a.tables = p->d_tables;
  a.batch = p->d_batch;
  a.cos_table = cos_table;
  a.sin_table = sin_table;
  a.status = p->d_status;
  a.rows = rows;
  a.hidden = hidden;
  a.q_cols = p->kv_heads * pa::kGroup * pa::kHeadDim;
  a.kv_cols = p->kv_heads * pa::kHeadDim;
  a.kv_heads = p->kv_heads;
  a.n_seqs = (int)p->batch.size();
  a.num_blocks = p->host.num_blocks();
  a.max_blocks_per_seq = p->host.max_blocks_per_seq();
  PA_CUDA(pa::launch_qkv_gemm(a, (cudaStream_t)stream));
  return PA_OK;
}

int pa_out_project_rows(pa_pool* p, const void* attn, const void* wo_packed, const void* residual, void* out,
                        int rows, int hidden, int cols, void* stream) {
  if (!p || !attn || !wo_packed || !out) return fail(PA_ERR_INVALID_ARG, "pa_out_project_rows: NULL argument");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_out_project_rows: host-only pool");
  if (rows < 1) return PA_OK;
  if (hidden < 64 || hidden % 64 != 0 || cols < 256 || cols % 256 != 0)
    return fail(PA_ERR_UNSUPPORTED, "pa_out_project_rows: hidden must be a multiple of 64, cols a multiple of 256");
  DeviceGuard g(p->device);
  if ((reinterpret_cast<uintptr_t>(attn) & 15u) != 0) return fail(PA_ERR_INVALID_ARG, "pa_out_project_rows: attn must be 16-byte aligned");
  pa::QkvGemmParams a = {};
  a.x = (const __nv_bfloat16*)attn;
  a.wq = a.wk = a.wv = (const __nv_bfloat16*)wo_packed;
  a.q_out = (__nv_bfloat16*)out;
  a.status = p->d_status;
  a.rows = rows;
  a.hidden = hidden;
  a.q_cols = cols;
  a.kv_cols = 256;
  a.linear = 1;
  a.residual = (const __nv_bfloat16*)residual;
  PA_CUDA(pa::launch_qkv_gemm(a, (cudaStream_t)stream));
  return PA_OK;
}

static int linear_rows(pa_pool* p, const void* x, const void* w_packed, const void* residual, void* out, int rows,
                       int k, int n, void* stream) {
  pa::QkvGemmParams a = {};
  a.x = (const __nv_bfloat16*)x;
  a.wq = a.wk = a.wv = (const __nv_bfloat16*)w_packed;
  a.q_out = (__nv_bfloat16*)out;
  a.status = p->d_status;
  a.rows = rows;
  a.hidden = k;
  a.q_cols = n;
  a.kv_cols = 256;
  a.linear = 1;
  a.residual = (const __nv_bfloat16*)residual;
  PA_CUDA(pa::launch_qkv_gemm(a, (cudaStream_t)stream));
  return PA_OK;
}

int pa_ffn_rows(pa_pool* p, const pa_ffn_weights* w, int layer, const void* x, void* scratch, void* out, int rows,
                int add_residual, void* stream) {
  if (!p || !w || !x || !scratch || !out) return fail(PA_ERR_INVALID_ARG, "pa_ffn_rows: NULL argument");
  if (!w->gate || !w->up || !w->down) return fail(PA_ERR_INVALID_ARG, "pa_ffn_rows: NULL weight");
  if (p->device < 0) return fail(PA_ERR_STATE, "pa_ffn_rows: host-only pool");
  if (layer < 0) return fail(PA_ERR_INVALID_ARG, "pa_ffn_rows: negative layer");
  if (rows < 1) return PA_OK;
  const int hidden = w->hidden, inter = w->inter;
  if (hidden < 256 || hidden > 2048 || hidden % 256 != 0 || inter < 128 || inter % 128 != 0)
    return fail(PA_ERR_UNSUPPORTED, "pa_ffn_rows: hidden a multiple of 256 up to 2048, intermediate a multiple of 128");
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(scratch)) & 15u) != 0)
    return fail(PA_ERR_INVALID_ARG, "pa_ffn_rows: x and scratch must be 16-byte aligned");
  DeviceGuard g(p->device);
  __nv_bfloat16* xn = (__nv_bfloat16*)scratch;
  __nv_bfloat16* gate = xn + (size_t)rows * hidden;  // the activated rows [rows, inter]
  const __nv_bfloat16* in = (const __nv_bfloat16*)x;
  if (w->ffn_norm) {
    const int r = pa_rmsnorm(x, (const __nv_bfloat16*)w->ffn_norm + (size_t)layer * w->norm_layer_stride, xn, rows, hidden,
                             w->rms_eps, stream);
    if (r != PA_OK) return r;
    in = xn;
  }
  // gate and up as one GEMM whose epilogue is SiLU(gate) * up: its tiles hold a gate head and the up
  // head of the same columns side by side
  {
    pa::QkvGemmParams a = {};
    a.x = in;
    a.wq = (const __nv_bfloat16*)w->gate + (size_t)layer * w->gate_layer_stride;
    a.wk = a.wv = (const __nv_bfloat16*)w->up + (size_t)layer * w->up_layer_stride;
    a.q_out = gate;
    a.status = p->d_status;
    a.rows = rows;
    a.hidden = hidden;
    a.q_cols = 2 * inter;
    a.kv_cols = 256;
    a.linear = 2;
    PA_CUDA(pa::launch_qkv_gemm(a, (cudaStream_t)stream));
  }
  return linear_rows(p, gate, (const __nv_bfloat16*)w->down + (size_t)layer * w->down_layer_stride,
                     add_residual ? x : nullptr, out, rows, inter, hidden, stream);
}

int pa_pool_set_layer_overlap(pa_pool* p, int allow) {
  if (!p) return fail(PA_ERR_INVALID_ARG, "pa_pool_set_layer_overlap: NULL pool");
  p->no_layer_overlap = allow == 0;
  return PA_OK;
}

int pa_pool_set_step_combiners(pa_pool* p, int combiners) {
  if (!p || (combiners != 0 && combiners != 1 && combiners != 2 && combiners != 4))
    return fail(PA_ERR_INVALID_ARG, "pa_pool_set_step_combiners: 0 (heuristic), 1, 2 or 4");
  p->step_combiners_override = combiners;
  return PA_OK;
}

int pa_pool_step_launches(pa_pool* p, long long* count) {
  if (!p || !count) return fail(PA_ERR_INVALID_ARG, "pa_pool_step_launches: NULL argument");
  *count = p->step_launches;
  return PA_OK;
}

int pa_pool_set_decode_shape(pa_pool* p, int warps, int stages) {
  if (!p) return fail(PA_ERR_INVALID_ARG, "pa_pool_set_decode_shape: NULL pool");
  if (!(warps == 0 && stages == 0) && !pa::decode_shape_supported(warps, stages))
    return fail(PA_ERR_UNSUPPORTED, "pa_pool_set_decode_shape: %d warps x %d stages is not built", warps, stages);
  p->decode_warps = warps;
  p->decode_stages = stages;
  return PA_OK;
}

}  // extern "C"
