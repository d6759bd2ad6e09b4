// pa_decode_noalloc: paged decode attention for callers that must not allocate.
//
// Some hosts cannot call cudaMalloc at all: a plug-in living inside a serving
// process that owns every byte of the GPU through its own arena, code running
// on a latency-critical loop where an allocation's implicit device-wide
// synchronisation would stall every other stream, or a process whose memory
// budget is fixed at start-up and audited.  pa_pool_create is closed to them
// (it allocates the cache, the tables and the split-KV workspace).  This entry
// lets them run the same decode kernel over buffers they already own: they
// pass the cache layer, the block tables, Q and the output; the only memory
// the kernel needs beyond that — split-KV partials, arrival tickets, the batch
// descriptor and a status word — lives in the fixed array below.
//
// The array is part of the loaded library image: every GPU that loads the
// library holds kScratchBytes (271104 bytes, 264.75 KiB) until the process exits.
#include <cstdio>
#include <mutex>

#include "../../include/paged_attention.h"
#include "kernels.cuh"

namespace {

constexpr int kMaxSeqs = PA_NOALLOC_MAX_SEQS;
constexpr int kMaxItems = 256;  // split-KV partials (sequence x KV head x chunk) per call
constexpr int kMaxDevices = 64;

// Layout of the scratch array (byte offsets, each part 256-byte aligned).
constexpr size_t kOffAcc = 0;                                                      // [kMaxItems][4][64] fp32
constexpr size_t kOffMl = kOffAcc + (size_t)kMaxItems * pa::kGroup * pa::kHeadDim * 4;  // [kMaxItems][2][4] fp32
constexpr size_t kOffCount = kOffMl + (size_t)kMaxItems * 2 * pa::kGroup * 4;       // [kMaxSeqs * 8] tickets
constexpr size_t kOffBatch = kOffCount + 256;                                      // [kMaxSeqs] BatchEntry
constexpr size_t kOffStatus = kOffBatch + 256;                                     // status word
constexpr size_t kScratchBytes = kOffStatus + 256;
static_assert(kMaxSeqs * 8 * sizeof(unsigned int) <= 256, "ticket area");
static_assert(kMaxSeqs * sizeof(pa::BatchEntry) <= 256, "batch area");

// In host code this name is only a handle for cudaGetSymbolAddress; it is not
// a device address and must never be handed to a kernel as one.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct DeviceSetup {
  bool done = false;
  unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on this device
  int sm_count = 0;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

}  // namespace

namespace pa {
void set_last_error(const char* msg);  // capi.cu: the text pa_last_error() returns
}

extern "C" {

// First call on a device resolves the device address of the scratch array
// (cudaGetSymbolAddress, with that device current) and reads the SM count.
// It allocates nothing.  No call may be made while `stream` is being captured:
// the batch descriptor is copied from this function's stack and the split plan
// is derived from the host array kv_lens, so a replay would read a dead address
// and a frozen plan; a capturing stream is refused with PA_ERR_STATE.
int pa_decode_noalloc(const void* cache_layer, int num_blocks, int kv_heads,
                      const int32_t* block_tables, int table_stride, const int32_t* kv_lens,
                      int n_seqs, const void* q, void* out, int64_t out_stride, float* lse,
                      float scale, void* stream) {
  char g_msg[384];
  auto fail = [&](int code, const char* what) {
    snprintf(g_msg, sizeof(g_msg), "pa_decode_noalloc: %s", what);
    pa::set_last_error(g_msg);
    return code;
  };
  if (!cache_layer || !block_tables || !kv_lens || !q || !out) return fail(PA_ERR_INVALID_ARG, "NULL argument");
  if (kv_heads != 1 && kv_heads != 2 && kv_heads != 4 && kv_heads != 8)
    return fail(PA_ERR_UNSUPPORTED, "kv_heads must be 1, 2, 4 or 8");
  if (n_seqs < 1) return fail(PA_ERR_INVALID_ARG, "n_seqs must be at least 1");
  if (n_seqs > kMaxSeqs) {
    snprintf(g_msg, sizeof(g_msg),
             "pa_decode_noalloc: %d sequences exceed the fixed scratch (PA_NOALLOC_MAX_SEQS = %d); "
             "split the batch or use a pool with pa_decode", n_seqs, kMaxSeqs);
    pa::set_last_error(g_msg);
    return PA_ERR_UNSUPPORTED;
  }
  if (num_blocks < 1 || table_stride < 1) return fail(PA_ERR_INVALID_ARG, "num_blocks and table_stride must be positive");
  if (out_stride < (int64_t)kv_heads * pa::kGroup * pa::kHeadDim) return fail(PA_ERR_INVALID_ARG, "out_stride shorter than a row");

  {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing((cudaStream_t)stream, &cap) != cudaSuccess) {
      cudaGetLastError();
      return fail(PA_ERR_CUDA, "cannot query the stream");
    }
    if (cap != cudaStreamCaptureStatusNone) return fail(PA_ERR_STATE, "the stream is being captured; this entry cannot be recorded in a graph");
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(PA_ERR_CUDA, "no current device");
  DeviceSetup* su = &g_setup[dev];
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!su->done) {
      void* ptr = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (e != cudaSuccess || !ptr) {
        snprintf(g_msg, sizeof(g_msg), "pa_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        pa::set_last_error(g_msg);
        return PA_ERR_CUDA;
      }
      e = cudaDeviceGetAttribute(&su->sm_count, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return fail(PA_ERR_CUDA, "cannot read the SM count");
      su->scratch = static_cast<unsigned char*>(ptr);
      su->done = true;
    }
  }

  pa::BatchEntry entries[kMaxSeqs];
  int max_blocks = 0;
  for (int i = 0; i < n_seqs; i++) {
    const int len = kv_lens[i];
    const int nb = (len + pa::kBlockTok - 1) / pa::kBlockTok;
    if (len < 0 || nb > table_stride) {
      snprintf(g_msg, sizeof(g_msg), "pa_decode_noalloc: sequence %d has %d tokens but its table row holds %d blocks",
               i, len, table_stride);
      pa::set_last_error(g_msg);
      return PA_ERR_INVALID_ARG;
    }
    entries[i] = {i, len, 0, 0, 1, i, 0, 0};
    if (nb > max_blocks) max_blocks = nb;
  }

  // One wave of 8-warp CTAs (one per SM), at most kMaxItems partials: the
  // smallest chunk that satisfies both.
  const int cta_limit = su->sm_count < kMaxItems ? su->sm_count : kMaxItems;
  auto ctas = [&](int cb) {
    long long n = 0;
    for (int i = 0; i < n_seqs; i++) {
      const int nb = (entries[i].kv_len + pa::kBlockTok - 1) / pa::kBlockTok;
      n += nb > 0 ? (nb + cb - 1) / cb : 1;
    }
    return n * kv_heads;
  };
  // partials are indexed [sequence][KV head][chunk of the longest sequence]
  auto fits = [&](int cb) {
    const long long mc = max_blocks > 0 ? (max_blocks + cb - 1) / cb : 1;
    return ctas(cb) <= cta_limit && mc * kv_heads * n_seqs <= kMaxItems;
  };
  int lo = 1, hi = max_blocks > 1 ? max_blocks : 1;
  while (lo < hi) {
    const int mid = lo + (hi - lo) / 2;
    if (fits(mid)) hi = mid; else lo = mid + 1;
  }
  const int cb = lo;
  int max_chunks = (max_blocks + cb - 1) / cb;
  if (max_chunks < 1) max_chunks = 1;
  if ((long long)max_chunks * kv_heads * n_seqs > kMaxItems) return fail(PA_ERR_UNSUPPORTED, "batch does not fit the fixed scratch");

  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* s = su->scratch;
  // Every call shares the array and finds the previous call's contents in it:
  // tickets must start at zero, the descriptor is rewritten.  The status word
  // is left alone: it keeps what a kernel recorded until
  // pa_decode_noalloc_check reads and clears it.
  cudaError_t e = cudaMemsetAsync(s + kOffCount, 0, kOffStatus - kOffCount, st);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(s + kOffBatch, entries, (size_t)n_seqs * sizeof(pa::BatchEntry), cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) {
    snprintf(g_msg, sizeof(g_msg), "pa_decode_noalloc: preparing the scratch failed: %s", cudaGetErrorString(e));
    pa::set_last_error(g_msg);
    return PA_ERR_CUDA;
  }

  pa::DecodeParams d;
  d.q = (const __nv_bfloat16*)q;
  d.out = (__nv_bfloat16*)out;
  d.out_f32 = nullptr;
  d.lse = lse;
  d.storage = (const char*)cache_layer;
  d.tables = block_tables;
  d.batch = reinterpret_cast<const pa::BatchEntry*>(s + kOffBatch);
  d.ws_acc = reinterpret_cast<float*>(s + kOffAcc);
  d.ws_ml = reinterpret_cast<float*>(s + kOffMl);
  d.ws_count = reinterpret_cast<unsigned int*>(s + kOffCount);
  d.status = reinterpret_cast<int*>(s + kOffStatus);
  d.out_stride = out_stride;
  d.scale_log2 = scale * pa::kLog2e;
  d.kv_heads = kv_heads;
  d.num_blocks = num_blocks;
  d.max_blocks_per_seq = table_stride;
  d.chunk_blocks = cb;
  d.max_chunks = max_chunks;
  e = pa::launch_decode(d, n_seqs, 8, 4, st);
  if (e != cudaSuccess) {
    snprintf(g_msg, sizeof(g_msg), "pa_decode_noalloc: launch failed: %s", cudaGetErrorString(e));
    pa::set_last_error(g_msg);
    return PA_ERR_CUDA;
  }
  return PA_OK;
}

// Reads and clears the status word the kernels of pa_decode_noalloc record in
// the scratch array (this entry's callers have no pool, so pa_pool_check cannot
// serve them).  Synchronises `stream`; allocates nothing.
int pa_decode_noalloc_check(void* stream) {
  char g_msg[256];
  auto fail = [&](int code, const char* what) {
    snprintf(g_msg, sizeof(g_msg), "pa_decode_noalloc_check: %s", what);
    pa::set_last_error(g_msg);
    return code;
  };
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(PA_ERR_CUDA, "no current device");
  unsigned char* s = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_setup[dev].done) s = g_setup[dev].scratch;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (!s) {  // pa_decode_noalloc never ran on this device
    if (cudaStreamSynchronize(st) != cudaSuccess) return fail(PA_ERR_CUDA, "stream synchronisation failed");
    return PA_OK;
  }
  int word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, s + kOffStatus, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(PA_ERR_CUDA, cudaGetErrorString(e));
  if (word == 0) return PA_OK;
  e = cudaMemsetAsync(s + kOffStatus, 0, sizeof(int), st);
  if (e != cudaSuccess) return fail(PA_ERR_CUDA, cudaGetErrorString(e));
  if (word == pa::kStatusTimeout) return fail(PA_ERR_TIMEOUT, "a kernel gave up waiting for a bulk copy");
  return fail(PA_ERR_INVALID_ARG, "a kernel met a block id outside the cache (num_blocks); the rows of that call are not valid");
}

}  // extern "C"
