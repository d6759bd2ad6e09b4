// The reference's three kernel launchers for the attention path, with the
// reference's data layouts, on top of the paged sm_100a kernels
// (include/legacy_kernels.h; C++ drop-in headers in include/).
#include <cstdio>
#include <mutex>
#include <vector>

#include "../../include/legacy_kernels.h"
#include "../../include/paged_attention.h"
#include "kernels.cuh"
#include "rope.cuh"

namespace pa {
void set_last_error(const char* msg);
// capi.cu: prefill of the active batch with caller-given tensor strides
int prefill_strided(pa_pool* p, int layer, const void* q, void* out, float* lse, long long q_seq_stride,
                    long long q_row_stride, long long q_head_stride, long long o_seq_stride,
                    long long o_row_stride, long long o_head_stride, long long lse_seq_stride,
                    int causal, float scale, void* stream);
}  // namespace pa

namespace {

int cfail(int code, const char* msg) {
  pa::set_last_error(msg);
  return code;
}

// ---- launch_rope_qkv: src/kernels/rope/rope.cu:23-359 in one launch ----------
// One thread per (token, head, chunk pair); Q and K are rotated and written
// head-major, V is copied head-major.
constexpr int kQH = 32, kKH = 8;
__global__ void __launch_bounds__(256)
legacy_rope_kernel(const __nv_bfloat16* q_in, __nv_bfloat16* q_out, const __nv_bfloat16* k_in,
                   __nv_bfloat16* k_out, const __nv_bfloat16* v_in, __nv_bfloat16* v_out,
                   const float* cos_table, const float* sin_table, int tokens, int position_offset) {
  const int units_per_tok = (kQH + 2 * kKH) * 4;
  const long long total = (long long)tokens * units_per_tok;
  for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < total;
       u += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(u / units_per_tok);
    int w = (int)(u - (long long)t * units_per_tok);
    const int c = w & 3;
    int h = w >> 2;
    const int pos = t + position_offset;
    if (h < kQH + kKH) {
      const bool is_q = h < kQH;
      if (!is_q) h -= kQH;
      const int heads = is_q ? kQH : kKH;
      const uint4* src = reinterpret_cast<const uint4*>((is_q ? q_in : k_in) + ((size_t)t * heads + h) * pa::kHeadDim);
      uint4* dst = reinterpret_cast<uint4*>((is_q ? q_out : k_out) + ((size_t)h * tokens + t) * pa::kHeadDim);
      const float4* cs = reinterpret_cast<const float4*>(cos_table + (size_t)pos * 32 + c * 8);
      const float4* sn = reinterpret_cast<const float4*>(sin_table + (size_t)pos * 32 + c * 8);
      float4 c8[2] = {cs[0], cs[1]}, s8[2] = {sn[0], sn[1]};
      uint4 ylo, yhi;
      pa::rope_chunks<1>(src[c], src[c + 4], reinterpret_cast<const float*>(c8),
                         reinterpret_cast<const float*>(s8), ylo, yhi);
      dst[c] = ylo;
      dst[c + 4] = yhi;
    } else {
      h -= kQH + kKH;
      const uint4* src = reinterpret_cast<const uint4*>(v_in + ((size_t)t * kKH + h) * pa::kHeadDim);
      uint4* dst = reinterpret_cast<uint4*>(v_out + ((size_t)h * tokens + t) * pa::kHeadDim);
      dst[c] = src[c];
      dst[c + 4] = src[c + 4];
    }
  }
}

// ---- launch_flash_output_layout: src/runtime/layout.cu:11-42, 16 bytes per thread
__global__ void __launch_bounds__(256)
legacy_layout_kernel(const uint4* in, uint4* out, int tokens) {
  const long long total = (long long)tokens * kQH * 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i & 7);
    const long long r = i >> 3;
    const int t = (int)(r % tokens), h = (int)(r / tokens);
    out[((long long)t * kQH + h) * 8 + c] = in[i];
  }
}

// ---- contiguous K/V -> paged layout -------------------------------------------
// Sequence b owns blocks [b*blocks_per_seq, (b+1)*blocks_per_seq) in order
// (checked on the host against the pool's tables).
__global__ void __launch_bounds__(256)
pack_kernel(const __nv_bfloat16* K, const __nv_bfloat16* V, char* storage, int batch, int kv_heads,
            int kv_len, int kv_stride, int blocks_per_seq) {
  const long long total = (long long)batch * kv_heads * kv_len * 16;  // 16-byte chunks of K and V
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i & 7);
    const int kv = (int)((i >> 3) & 1);
    long long r = i >> 4;
    const int pos = (int)(r % kv_len);
    r /= kv_len;
    const int h = (int)(r % kv_heads), b = (int)(r / kv_heads);
    const __nv_bfloat16* src = (kv ? V : K) + (((size_t)b * kv_heads + h) * kv_stride + pos) * pa::kHeadDim;
    const int blk = b * blocks_per_seq + pos / pa::kBlockTok;
    char* tile = storage + pa::tile_off(blk, kv_heads, h, kv);
    *reinterpret_cast<uint4*>(tile + pa::tile_chunk_off(pos % pa::kBlockTok, c)) =
        reinterpret_cast<const uint4*>(src)[c];
  }
}

struct CompatState {
  pa_pool* pool = nullptr;
  int kv_heads = 0, max_seqs = 0, blocks_per_seq = 0;
  std::vector<int> seqs;
  // Calls on one device share the private pool (cache, tables, split-KV workspace): a call on
  // another stream first waits for the previous call's work (recorded here), so concurrent
  // streams are serialised on the pool instead of racing on it.
  cudaEvent_t last = nullptr;
};
CompatState g_state[64];
std::mutex g_mutex;

int grid_for(long long total) {
  long long b = (total + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 148 * 32 ? 148 * 32 : b));
}

}  // namespace

extern "C" {

int lt_launch_rope_qkv(const void* q_in, void* q_out, const void* k_in, void* k_out, const void* v_in,
                       void* v_out, const float* cos_table, const float* sin_table, int tokens,
                       int position_offset, void* stream) {
  if (!q_in || !q_out || !k_in || !k_out || !v_in || !v_out || !cos_table || !sin_table)
    return cfail(PA_ERR_INVALID_ARG, "lt_launch_rope_qkv: NULL argument");
  if (tokens <= 0 || position_offset < 0) return cfail(PA_ERR_INVALID_ARG, "lt_launch_rope_qkv: bad token count or position");
  legacy_rope_kernel<<<grid_for((long long)tokens * (kQH + 2 * kKH) * 4), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)q_in, (__nv_bfloat16*)q_out, (const __nv_bfloat16*)k_in, (__nv_bfloat16*)k_out,
      (const __nv_bfloat16*)v_in, (__nv_bfloat16*)v_out, cos_table, sin_table, tokens, position_offset);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cfail(PA_ERR_CUDA, cudaGetErrorString(e));
  return PA_OK;
}

int lt_launch_flash_output_layout(const void* in, void* out, int tokens, void* stream) {
  if (!in || !out || tokens <= 0) return cfail(PA_ERR_INVALID_ARG, "lt_launch_flash_output_layout: bad argument");
  legacy_layout_kernel<<<grid_for((long long)tokens * kQH * 8), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)in, (uint4*)out, tokens);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cfail(PA_ERR_CUDA, cudaGetErrorString(e));
  return PA_OK;
}

int lt_launch_flash_attention(const lt_flash_attention_params* a) {
  if (!a || !a->Q || !a->K || !a->V || !a->O) return cfail(PA_ERR_INVALID_ARG, "lt_launch_flash_attention: NULL argument");
  const int kvh = a->num_kv_heads > 0 ? a->num_kv_heads : a->num_heads;
  if (a->d_head != 64) return cfail(PA_ERR_UNSUPPORTED, "lt_launch_flash_attention: only d_head 64 is built");
  if (a->dtype != 1) return cfail(PA_ERR_UNSUPPORTED, "lt_launch_flash_attention: only bf16 is built");
  if (a->num_heads != 4 * kvh || (kvh != 1 && kvh != 2 && kvh != 4 && kvh != 8))
    return cfail(PA_ERR_UNSUPPORTED, "lt_launch_flash_attention: needs num_heads == 4 * num_kv_heads, num_kv_heads in {1,2,4,8}");
  if (a->batch_size < 1 || a->q_seq_len < 1 || a->kv_seq_len < 1 || a->kv_stride < a->kv_seq_len)
    return cfail(PA_ERR_INVALID_ARG, "lt_launch_flash_attention: bad sizes");
  if (a->causal && a->kv_seq_len < a->q_seq_len)
    return cfail(PA_ERR_INVALID_ARG, "lt_launch_flash_attention: causal attention needs kv_seq_len >= q_seq_len");
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cfail(PA_ERR_CUDA, "no current device");
  std::lock_guard<std::mutex> lock(g_mutex);
  CompatState& s = g_state[dev];
  const int nb = (a->kv_seq_len + pa::kBlockTok - 1) / pa::kBlockTok;
  cudaStream_t st = (cudaStream_t)a->stream;
  int rc;
  if (!s.last && cudaEventCreateWithFlags(&s.last, cudaEventDisableTiming) != cudaSuccess)
    return cfail(PA_ERR_CUDA, "lt_launch_flash_attention: cannot create an event");
  if (cudaStreamWaitEvent(st, s.last, 0) != cudaSuccess) return cfail(PA_ERR_CUDA, "lt_launch_flash_attention: cudaStreamWaitEvent failed");
  if (!s.pool || s.kv_heads != kvh || s.max_seqs < a->batch_size || s.blocks_per_seq < nb) {
    if (s.pool) {
      cudaDeviceSynchronize();  // earlier calls may still read the old pool
      pa_pool_destroy(s.pool);
      cudaEvent_t keep = s.last;
      s = CompatState();
      s.last = keep;
    }
    const int cap = nb + nb / 4 + 16;  // room to grow without reallocating every call
    rc = pa_pool_create(&s.pool, dev, 1, a->batch_size * cap, kvh, a->batch_size, cap);
    if (rc != PA_OK) return rc;
    s.kv_heads = kvh;
    s.max_seqs = a->batch_size;
    s.blocks_per_seq = cap;
  }
  // fresh tables: sequence b takes blocks b*nb .. b*nb+nb-1 of the identity free order
  for (int id : s.seqs) pa_seq_free(s.pool, id);
  s.seqs.clear();
  std::vector<int32_t> order((size_t)s.max_seqs * s.blocks_per_seq);
  for (size_t i = 0; i < order.size(); i++) order[i] = (int32_t)i;
  rc = pa_pool_set_free_order(s.pool, order.data(), (int)order.size());
  if (rc != PA_OK) return rc;
  std::vector<int32_t> ids(a->batch_size), zeros(a->batch_size, 0), qrows(a->batch_size, a->q_seq_len),
      qpos(a->batch_size, a->kv_seq_len - a->q_seq_len);
  for (int b = 0; b < a->batch_size; b++) {
    int id = -1;
    rc = pa_seq_create(s.pool, &id);
    if (rc == PA_OK) rc = pa_seq_reserve(s.pool, id, a->kv_seq_len);
    if (rc != PA_OK) return rc;
    s.seqs.push_back(id);
    ids[b] = id;
    const int32_t* t = nullptr;
    int n = 0;
    pa_seq_block_table(s.pool, id, &t, &n);
    for (int i = 0; i < n; i++)
      if (t[i] != b * nb + i) return cfail(PA_ERR_STATE, "lt_launch_flash_attention: unexpected block table");
  }
  void* storage = nullptr;
  pa_pool_layer_storage(s.pool, 0, &storage, nullptr);
  pack_kernel<<<grid_for((long long)a->batch_size * kvh * a->kv_seq_len * 16), 256, 0, st>>>(
      (const __nv_bfloat16*)a->K, (const __nv_bfloat16*)a->V, (char*)storage, a->batch_size, kvh, a->kv_seq_len,
      a->kv_stride, nb);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cfail(PA_ERR_CUDA, cudaGetErrorString(e));
  rc = pa_batch_set_sharded(s.pool, ids.data(), zeros.data(), qrows.data(), qpos.data(), nullptr, a->batch_size, st);
  if (rc != PA_OK) return rc;
  const long long hq = a->num_heads;
  if (a->q_seq_len == 1) {
    rc = pa_decode(s.pool, 0, a->Q, a->O, hq * 64, nullptr, a->L, a->scale, st);
    cudaEventRecord(s.last, st);
    return rc;
  }
  // head-major Q/O: row r of head h of sequence b is at ((b*heads + h)*q_seq_len + r)*64.
  // The kernel adds the batch's running row offset (b*q_seq_len rows) on top of
  // the per-sequence stride, so that part is taken out of the stride here.
  const long long sq = a->q_seq_len;
  const long long seq_stride = hq * sq * 64 - sq * 64;
  rc = pa::prefill_strided(s.pool, 0, a->Q, a->O, a->L, seq_stride, 64, sq * 64, seq_stride, 64, sq * 64, hq * sq,
                           a->causal ? 1 : 0, a->scale, st);
  cudaEventRecord(s.last, st);
  return rc;
}

}  // extern "C"
