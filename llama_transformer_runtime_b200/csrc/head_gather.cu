// All-gather of head outputs for KV-head sharded decode, one process per GPU.
// The reference is single-GPU; this is the collective batched decode needs once
// the 8 KV heads are spread over n pools: every rank must end up with the full
// [sequences, 2048] attention rows that the output projection consumes.
//
// It is fused into the decode kernel: the CTA that finishes a (sequence, KV
// head) group stores its bf16 rows into the same column slice of EVERY rank's
// row buffer (plain peer stores over NVLink) and adds one arrival to every
// rank's counter for (source rank, layer).  Nothing is loaded from a peer and
// nothing is multicast.  One small kernel at the end of the step waits —
// bounded, PA_ERR_TIMEOUT in the pool's status word otherwise — until all
// counters of the step have reached their target; there is no per-layer
// collective at all.  Two row buffers alternate by step, so a fast rank can
// already write step s+1 while a slow one still reads step s.
#include <cstdio>
#include <cstring>
#include <new>

#include "../../include/paged_attention.h"
#include "kernels.cuh"

namespace pa {
void set_last_error(const char* msg);
}

struct pa_gather {
  int device = 0, rank = 0, world = 1, n_seqs = 0, layers = 0, kv_heads = 0;
  size_t slot_bytes = 0, data_bytes = 0, bytes = 0;
  unsigned char* local = nullptr;
  unsigned char* peer[8] = {};
  bool opened[8] = {};
  bool connected = false;
  unsigned int seq = 0;
};

namespace {

int gfail(int code, const char* fmt, const char* arg = "") {
  char msg[384];
  snprintf(msg, sizeof(msg), fmt, arg);
  pa::set_last_error(msg);
  return code;
}

__global__ void __launch_bounds__(256)
gather_wait_kernel(const unsigned int* counters, int n_counters, unsigned int target, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  for (int i = threadIdx.x; i < n_counters; i += blockDim.x) {
    pa::SpinDeadline dl;
    for (;;) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counters + i) : "memory");
      if ((int)(v - target) >= 0) break;
      if (dl.expired()) {
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok && threadIdx.x == 0) atomicExch(status, pa::kStatusTimeout);
}

size_t row_elems(const pa_gather* g) { return (size_t)g->world * g->kv_heads * pa::kGroup * pa::kHeadDim; }

}  // namespace

namespace pa {
// capi.cu: start a step / describe one layer's destination / finish a step.
bool gather_begin(pa_gather* g) {
  if (!g || !g->connected) return false;
  g->seq++;
  return true;
}
bool gather_fill(pa_gather* g, int layer, int n_seqs, int kv_heads, DecodeParams& d) {
  if (!g || !g->connected || g->seq == 0 || layer < 0 || layer >= g->layers || n_seqs != g->n_seqs ||
      kv_heads != g->kv_heads)
    return false;
  const size_t slot = (size_t)(g->seq & 1u) * g->slot_bytes;
  const size_t layer_off = (size_t)layer * g->n_seqs * row_elems(g) * sizeof(__nv_bfloat16);
  for (int r = 0; r < g->world; r++) {
    d.hs_rows[r] = reinterpret_cast<__nv_bfloat16*>(g->peer[r] + slot + layer_off);
    d.hs_counter[r] =
        reinterpret_cast<unsigned int*>(g->peer[r] + g->data_bytes) + (size_t)g->rank * g->layers + layer;
  }
  d.hs_world = g->world;
  d.hs_col0 = g->rank * g->kv_heads * kGroup * kHeadDim;
  d.hs_stride = (long long)row_elems(g);
  return true;
}
cudaError_t gather_wait(pa_gather* g, int* status, cudaStream_t stream, void** rows) {
  const unsigned int target = g->seq * (unsigned int)(g->n_seqs * g->kv_heads);
  gather_wait_kernel<<<1, 256, 0, stream>>>(reinterpret_cast<const unsigned int*>(g->local + g->data_bytes),
                                            g->world * g->layers, target, status);
  if (rows) *rows = g->local + (size_t)(g->seq & 1u) * g->slot_bytes;
  return cudaGetLastError();
}
int gather_layers(const pa_gather* g) { return g ? g->layers : 0; }
}  // namespace pa

extern "C" {

int pa_gather_create(pa_gather** out, int device, int rank, int world, int n_seqs, int layers, int kv_heads) {
  if (!out) return gfail(PA_ERR_INVALID_ARG, "pa_gather_create: out is NULL");
  *out = nullptr;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || n_seqs < 1 || layers < 1 || kv_heads < 1 ||
      kv_heads * world > 8)
    return gfail(PA_ERR_INVALID_ARG, "pa_gather_create: world 1..8, rank < world, kv_heads * world <= 8");
  pa_gather* g = new (std::nothrow) pa_gather();
  if (!g) return gfail(PA_ERR_INVALID_ARG, "pa_gather_create: out of host memory");
  g->device = device;
  g->rank = rank;
  g->world = world;
  g->n_seqs = n_seqs;
  g->layers = layers;
  g->kv_heads = kv_heads;
  g->slot_bytes = ((size_t)layers * n_seqs * row_elems(g) * sizeof(__nv_bfloat16) + 255) & ~(size_t)255;
  g->data_bytes = 2 * g->slot_bytes;
  g->bytes = g->data_bytes + (((size_t)world * layers * sizeof(unsigned int) + 255) & ~(size_t)255);
  int prev = -1;
  cudaGetDevice(&prev);
  cudaError_t e = cudaSetDevice(device);
  if (e == cudaSuccess) e = cudaMalloc((void**)&g->local, g->bytes);
  if (e == cudaSuccess) e = cudaMemset(g->local, 0, g->bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) {
    int code = gfail(PA_ERR_CUDA, "pa_gather_create: %s", cudaGetErrorString(e));
    delete g;
    return code;
  }
  g->peer[rank] = g->local;
  if (world == 1) g->connected = true;
  *out = g;
  return PA_OK;
}

int pa_gather_buffer(pa_gather* g, void** dev_ptr, uint64_t* bytes) {
  if (!g) return gfail(PA_ERR_INVALID_ARG, "pa_gather_buffer: NULL argument");
  if (dev_ptr) *dev_ptr = g->local;
  if (bytes) *bytes = g->bytes;
  return PA_OK;
}

int pa_gather_connect_ptrs(pa_gather* g, void* const* peer_buffers) {
  if (!g || !peer_buffers) return gfail(PA_ERR_INVALID_ARG, "pa_gather_connect_ptrs: NULL argument");
  for (int r = 0; r < g->world; r++) {
    if (r == g->rank) continue;
    if (!peer_buffers[r]) return gfail(PA_ERR_INVALID_ARG, "pa_gather_connect_ptrs: NULL peer buffer");
    g->peer[r] = static_cast<unsigned char*>(peer_buffers[r]);
  }
  g->connected = true;
  return PA_OK;
}

int pa_gather_handle(pa_gather* g, void* handle64) {
  if (!g || !handle64) return gfail(PA_ERR_INVALID_ARG, "pa_gather_handle: NULL argument");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, g->local);
  if (e != cudaSuccess) return gfail(PA_ERR_CUDA, "pa_gather_handle: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  memcpy(handle64, &h, sizeof(h));
  return PA_OK;
}

int pa_gather_connect(pa_gather* g, const void* handles) {
  if (!g || !handles) return gfail(PA_ERR_INVALID_ARG, "pa_gather_connect: NULL argument");
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(g->device);
  int rc = PA_OK;
  for (int r = 0; r < g->world && rc == PA_OK; r++) {
    if (r == g->rank || g->opened[r]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const unsigned char*)handles + (size_t)r * sizeof(h), sizeof(h));
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      rc = gfail(PA_ERR_CUDA, "pa_gather_connect: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
      cudaGetLastError();
      break;
    }
    g->peer[r] = static_cast<unsigned char*>(ptr);
    g->opened[r] = true;
  }
  if (prev >= 0) cudaSetDevice(prev);
  if (rc == PA_OK) g->connected = true;
  return rc;
}

// The caller makes sure no rank still has work in flight that targets this
// buffer (a host-level barrier after a device synchronisation).
int pa_gather_destroy(pa_gather* g) {
  if (!g) return PA_OK;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(g->device);
  for (int r = 0; r < g->world; r++)
    if (g->opened[r]) cudaIpcCloseMemHandle(g->peer[r]);
  cudaFree(g->local);
  if (prev >= 0) cudaSetDevice(prev);
  delete g;
  return PA_OK;
}

}  // extern "C"
