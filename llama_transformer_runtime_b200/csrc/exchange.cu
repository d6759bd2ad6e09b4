// Cross-GPU log-sum-exp exchange for sequence-range sharded decode, one process
// per GPU.  The reference is single-GPU (no collective anywhere in it); this is
// the exchange step that long-context decode needs once a sequence's cache is
// split by token range over several B200s.
//
// Instead of a library all-gather (a ~8 KiB message, where launch and protocol
// latency dominate), the decode kernel's combine epilogue stores this rank's
// partial (normalised O, LSE) straight into every rank's receive buffer with
// plain peer stores over NVLink.  Two protocols share the buffer:
//  * merge inside the decode kernel (pa_decode_step_sharded): every value
//    travels as one 8-byte word {value, step number}; the combining CTA of a
//    (sequence, KV head) polls its own memory until each word it needs carries
//    the step number (bounded to about a second, then PA_ERR_TIMEOUT in the
//    pool's status word) and merges.  No fence and no flag: a system-scope
//    fence in that CTA cost about 7 us while the next layer was streaming.
//  * push + separate merge kernel (pa_decode_push, pa_exchange_merge): fp32
//    rows, then the step number in a flag (st.release.sys); the merge kernel
//    waits for the flags of all ranks (ld.acquire.sys, bounded likewise).
// Either way a rank reads only its OWN memory.  Nothing is ever loaded
// from a peer, nothing is multicast.  Two slots alternate by step: a rank can
// run at most one step ahead of the slowest one, because its own merge needs
// everybody's partial.
//
// Buffers are cudaMalloc'ed here and shared through CUDA IPC handles, which the
// host exchanges with whatever it has (torch.distributed in the bench).
#include <cstdio>
#include <cstring>
#include <new>

#include "../../include/paged_attention.h"
#include "kernels.cuh"

namespace pa {
void set_last_error(const char* msg);
}

struct pa_exchange {
  int device = 0, rank = 0, world = 1, rows = 0, groups = 0;
  size_t data_bytes = 0, ll_offset = 0, bytes = 0;
  unsigned char* local = nullptr;      // receive buffer of this rank
  unsigned char* peer[8] = {};         // every rank's buffer as mapped here (peer[rank] == local)
  bool opened[8] = {};
  bool connected = false;
  unsigned int seq = 0;
};

namespace {

int xfail(int code, const char* fmt, const char* arg = "") {
  char msg[384];
  snprintf(msg, sizeof(msg), fmt, arg);
  pa::set_last_error(msg);
  return code;
}

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256)
exchange_merge_kernel(pa::ExchangeMergeParams p) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // one waiter per flag, all flags in parallel
  for (int f = threadIdx.x; f < p.world * p.groups; f += blockDim.x) {
    const unsigned int* flag = p.flags + f;
    pa::SpinDeadline dl;
    // flags only grow; a later step's value also means this step has landed
    while ((int)(ld_acquire_sys(flag) - p.seq) < 0) {
      if (dl.expired()) {
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0) atomicExch(p.status, pa::kStatusTimeout);
    return;
  }
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.rows * pa::kHeadDim) return;
  const int row = idx >> 6, d = idx & 63;
  const float* base = p.data + (size_t)p.slot * p.world * p.rows * pa::kXchgRowFloats;
  float M = -INFINITY;
  for (int g = 0; g < p.world; g++)
    M = fmaxf(M, __ldcg(base + ((size_t)g * p.rows + row) * pa::kXchgRowFloats + pa::kHeadDim));
  float L = 0.f, O = 0.f;
  if (M > -INFINITY) {
    for (int g = 0; g < p.world; g++) {
      const float* rowp = base + ((size_t)g * p.rows + row) * pa::kXchgRowFloats;
      const float lse = __ldcg(rowp + pa::kHeadDim);
      const float w = lse == -INFINITY ? 0.f : __expf(lse - M);
      L += w;
      O += w * __ldcg(rowp + d);
    }
  }
  const int z = row / p.q_heads, head = row - z * p.q_heads;
  p.out[(size_t)z * p.out_stride + head * pa::kHeadDim + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
}

}  // namespace

namespace pa {
cudaError_t launch_exchange_merge(const ExchangeMergeParams& p, cudaStream_t stream) {
  const int total = p.rows * kHeadDim;
  exchange_merge_kernel<<<(total + 255) / 256, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

// Used by capi.cu: start the next exchange step (fills the decode launch
// descriptor) and describe the matching merge.
bool exchange_fill(pa_exchange* x, DecodeParams& d, ExchangeMergeParams& m) {
  if (!x || !x->connected) return false;
  x->seq++;
  const int slot = (int)(x->seq & 1u);
  for (int g = 0; g < x->world; g++) {
    d.xchg_peer[g] = reinterpret_cast<float*>(x->peer[g]);
    d.xchg_flag[g] = reinterpret_cast<unsigned int*>(x->peer[g] + x->data_bytes);
    d.xchg_ll[g] = reinterpret_cast<unsigned long long*>(x->peer[g] + x->ll_offset);
  }
  d.xchg_world = x->world;
  d.xchg_rank = x->rank;
  d.xchg_rows = x->rows;
  d.xchg_groups = x->groups;
  d.xchg_slot = slot;
  d.xchg_seq = x->seq;
  m.data = reinterpret_cast<const float*>(x->local);
  m.flags = reinterpret_cast<const unsigned int*>(x->local + x->data_bytes);
  m.world = x->world;
  m.rows = x->rows;
  m.groups = x->groups;
  m.slot = slot;
  m.seq = x->seq;
  return true;
}
// A multi-layer step launched as one kernel uses `steps` more step numbers.
void exchange_advance(pa_exchange* x, int steps) {
  if (x && steps > 0) x->seq += (unsigned)steps;
}
// Take back the step number handed out by the last exchange_fill (nothing was launched).
void exchange_unfill(pa_exchange* x) {
  if (x && x->seq > 0) x->seq--;
}
// The merge of the step most recently started with exchange_fill.
bool exchange_current(pa_exchange* x, ExchangeMergeParams& m) {
  if (!x || !x->connected || x->seq == 0) return false;
  m.data = reinterpret_cast<const float*>(x->local);
  m.flags = reinterpret_cast<const unsigned int*>(x->local + x->data_bytes);
  m.world = x->world;
  m.rows = x->rows;
  m.groups = x->groups;
  m.slot = (int)(x->seq & 1u);
  m.seq = x->seq;
  return true;
}
int exchange_rows(const pa_exchange* x) { return x ? x->rows : 0; }
int exchange_groups(const pa_exchange* x) { return x ? x->groups : 0; }
}  // namespace pa

extern "C" {

int pa_exchange_create(pa_exchange** out, int device, int rank, int world, int n_seqs, int kv_heads) {
  if (!out) return xfail(PA_ERR_INVALID_ARG, "pa_exchange_create: out is NULL");
  *out = nullptr;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || n_seqs < 1 || kv_heads < 1 || kv_heads > 8)
    return xfail(PA_ERR_INVALID_ARG, "pa_exchange_create: world 1..8, rank < world, n_seqs >= 1, kv_heads 1..8");
  pa_exchange* x = new (std::nothrow) pa_exchange();
  if (!x) return xfail(PA_ERR_INVALID_ARG, "pa_exchange_create: out of host memory");
  x->device = device;
  x->rank = rank;
  x->world = world;
  x->rows = n_seqs * kv_heads * pa::kGroup;
  x->groups = n_seqs * kv_heads;
  x->data_bytes = ((size_t)2 * world * x->rows * pa::kXchgRowFloats * sizeof(float) + 255) & ~(size_t)255;
  // [data | flags | words]: the first two serve the push + separate merge
  // kernel, the third the merge inside the decode kernel
  x->ll_offset = x->data_bytes + (((size_t)world * x->groups * sizeof(unsigned int) + 255) & ~(size_t)255);
  // kXchgWordSlots slots of words: up to four combining CTAs per (sequence, head) work on
  // alternate layers, so a peer may already be that many steps ahead of a slot a rank still polls
  x->bytes = x->ll_offset + (size_t)pa::kXchgWordSlots * world * x->rows * pa::kXchgRowFloats * sizeof(unsigned long long);
  int prev = -1;
  cudaGetDevice(&prev);
  cudaError_t e = cudaSetDevice(device);
  if (e == cudaSuccess) e = cudaMalloc((void**)&x->local, x->bytes);
  if (e == cudaSuccess) e = cudaMemset(x->local, 0, x->bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) {
    int code = xfail(PA_ERR_CUDA, "pa_exchange_create: %s", cudaGetErrorString(e));
    delete x;
    return code;
  }
  x->peer[rank] = x->local;
  if (world == 1) x->connected = true;
  *out = x;
  return PA_OK;
}

int pa_exchange_buffer(pa_exchange* x, void** dev_ptr, uint64_t* bytes) {
  if (!x) return xfail(PA_ERR_INVALID_ARG, "pa_exchange_buffer: NULL argument");
  if (dev_ptr) *dev_ptr = x->local;
  if (bytes) *bytes = x->bytes;
  return PA_OK;
}

// For hosts that drive several GPUs from one process (peer access enabled by
// the caller) and for single-GPU tests: the ranks' buffers as plain pointers.
int pa_exchange_connect_ptrs(pa_exchange* x, void* const* peer_buffers) {
  if (!x || !peer_buffers) return xfail(PA_ERR_INVALID_ARG, "pa_exchange_connect_ptrs: NULL argument");
  for (int g = 0; g < x->world; g++) {
    if (g == x->rank) continue;
    if (!peer_buffers[g]) return xfail(PA_ERR_INVALID_ARG, "pa_exchange_connect_ptrs: NULL peer buffer");
    x->peer[g] = static_cast<unsigned char*>(peer_buffers[g]);
  }
  x->connected = true;
  return PA_OK;
}

int pa_exchange_handle(pa_exchange* x, void* handle64) {
  if (!x || !handle64) return xfail(PA_ERR_INVALID_ARG, "pa_exchange_handle: NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == PA_EXCHANGE_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, x->local);
  if (e != cudaSuccess) return xfail(PA_ERR_CUDA, "pa_exchange_handle: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  memcpy(handle64, &h, sizeof(h));
  return PA_OK;
}

int pa_exchange_connect(pa_exchange* x, const void* handles) {
  if (!x || !handles) return xfail(PA_ERR_INVALID_ARG, "pa_exchange_connect: NULL argument");
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(x->device);
  int rc = PA_OK;
  for (int g = 0; g < x->world && rc == PA_OK; g++) {
    if (g == x->rank || x->opened[g]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const unsigned char*)handles + (size_t)g * sizeof(h), sizeof(h));
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      rc = xfail(PA_ERR_CUDA, "pa_exchange_connect: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
      cudaGetLastError();
      break;
    }
    x->peer[g] = static_cast<unsigned char*>(ptr);
    x->opened[g] = true;
  }
  if (prev >= 0) cudaSetDevice(prev);
  if (rc == PA_OK) x->connected = true;
  return rc;
}

// The caller makes sure no rank still has work in flight that targets this
// buffer (a host-level barrier after a device synchronisation).
int pa_exchange_destroy(pa_exchange* x) {
  if (!x) return PA_OK;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(x->device);
  for (int g = 0; g < x->world; g++)
    if (x->opened[g]) cudaIpcCloseMemHandle(x->peer[g]);
  cudaFree(x->local);
  if (prev >= 0) cudaSetDevice(prev);
  delete x;
  return PA_OK;
}

}  // extern "C"
