// Greedy sampling of a decode step: the index of the largest logit of every row.
//
// Replaces launch_argmax (src/kernels/sampling/argmax_128256.cu:43-101: one CTA of 256 threads over
// the 128256 bf16 logits, thread t scanning t, t + 256, ... with a strict ">" and the lanes and warps
// combined by shuffle-down, again with a strict ">"), which the reference's decode loop calls after
// the language-model head (src/runtime/llama_runtime.cu:907-930, with a cudaMalloc, a blocking copy
// and a cudaFree per token around it).  Its tie rule follows from that structure and is restated
// here as a total order, so that any reduction tree gives the reference's answer: a thread keeps
// its smallest index; a shuffle-down reduction is a tree whose left operand wins a tie and whose
// leaves, left to right, are the lanes in bit-reversed order; the warps are combined the same way.
// So among equal largest values the winner has the smallest (bit-reversed warp number,
// bit-reversed lane number, index), with thread = index mod 256.
//
// A cluster of eight CTAs of 1024 threads per row, 16-byte loads (8 logits), best candidate per
// thread, lanes by shuffle, warps through shared memory, CTAs through distributed shared memory.
#include <cfloat>

#include "../../include/paged_attention.h"
#include "kernels.cuh"

namespace pa {
void set_last_error(const char* msg);
}

namespace {

constexpr int kArgmaxThreads = 1024;
constexpr int kArgmaxCluster = 8;

struct Cand {
  float v;
  int i;
};
// 10-bit tie key of an index: bit-reversed warp number (5 bits) above bit-reversed lane number
__device__ __forceinline__ unsigned tie_key(int i) {
  const unsigned t = (unsigned)i & 255u;
  return ((__brev(t >> 5) >> 27) << 5) | (__brev(t & 31u) >> 27);
}
// true when b beats a: larger value; among equal values the smaller (tie key, index)
__device__ __forceinline__ bool beats(const Cand& b, const Cand& a) {
  if (b.v != a.v) return b.v > a.v;
  if (a.i < 0 || b.i < 0) return a.i < 0 && b.i >= 0;
  const unsigned ka = tie_key(a.i), kb = tie_key(b.i);
  return kb != ka ? kb < ka : b.i < a.i;
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_meet() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ Cand ld_peer_cand(const Cand* local, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  Cand c;
  asm volatile("ld.shared::cluster.v2.b32 {%0, %1}, [%2];" : "=f"(c.v), "=r"(c.i) : "r"(a) : "memory");
  return c;
}

// A cluster of kArgmaxCluster CTAs per row (blockIdx.y): CTA r scans the r-th part of the row's 16-byte
// chunks, the last one also a tail shorter than a chunk; the parts' winners meet in the first CTA
// through distributed shared memory.  One CTA alone needs 16 dependent rounds of loads for a
// 128256-entry row (about 12 us); eight need two.
__global__ void __cluster_dims__(kArgmaxCluster, 1, 1) __launch_bounds__(kArgmaxThreads)
    argmax_rows_kernel(const __nv_bfloat16* logits, int* tokens, int vocab, int pdl) {
  __shared__ Cand s_best[kArgmaxThreads / 32];
  __shared__ __align__(8) Cand s_part;
  if (pdl) {  // behind the language-model head of the same step: the logits are its output
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  const uint32_t rank = cluster_rank();
  const __nv_bfloat16* row = logits + (size_t)blockIdx.y * vocab;
  Cand best{-FLT_MAX, -1};
  const int chunks = vocab / 8;
  const int c_begin = (int)((long long)chunks * rank / kArgmaxCluster), c_end = (int)((long long)chunks * (rank + 1) / kArgmaxCluster);
  for (int c = c_begin + threadIdx.x; c < c_end; c += kArgmaxThreads) {
    const uint4 d = reinterpret_cast<const uint4*>(row)[c];
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 f = __bfloat1622float2(h2[j]);
      const Cand a{f.x, c * 8 + 2 * j}, b{f.y, c * 8 + 2 * j + 1};
      if (beats(a, best)) best = a;
      if (beats(b, best)) best = b;
    }
  }
  if (rank == kArgmaxCluster - 1)
    for (int i = chunks * 8 + threadIdx.x; i < vocab; i += kArgmaxThreads) {  // a tail shorter than one chunk
      const Cand a{__bfloat162float(row[i]), i};
      if (beats(a, best)) best = a;
    }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const Cand o{__shfl_xor_sync(0xffffffffu, best.v, off), __shfl_xor_sync(0xffffffffu, best.i, off)};
    if (beats(o, best)) best = o;
  }
  if ((threadIdx.x & 31) == 0) s_best[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = s_best[threadIdx.x];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const Cand o{__shfl_xor_sync(0xffffffffu, best.v, off), __shfl_xor_sync(0xffffffffu, best.i, off)};
      if (beats(o, best)) best = o;
    }
    if (threadIdx.x == 0) s_part = best;
  }
  cluster_meet();  // every CTA's winner is in its shared memory
  if (rank == 0 && threadIdx.x < 32) {
    best = threadIdx.x < kArgmaxCluster ? ld_peer_cand(&s_part, threadIdx.x) : Cand{-FLT_MAX, -1};
#pragma unroll
    for (int off = kArgmaxCluster / 2; off > 0; off >>= 1) {
      const Cand o{__shfl_xor_sync(0xffffffffu, best.v, off), __shfl_xor_sync(0xffffffffu, best.i, off)};
      if (beats(o, best)) best = o;
    }
    if (threadIdx.x == 0) tokens[blockIdx.y] = best.i;
  }
  cluster_meet();  // no CTA leaves while the first one reads its shared memory
}

}  // namespace

namespace pa {
int argmax_impl(const void* logits, int32_t* tokens, int rows, int vocab, int pdl, void* stream) {
  if (!logits || !tokens) {
    set_last_error("pa_argmax: NULL argument");
    return PA_ERR_INVALID_ARG;
  }
  if (rows < 1) return PA_OK;
  if (rows > 65535) {
    set_last_error("pa_argmax: at most 65535 rows per call");
    return PA_ERR_UNSUPPORTED;
  }
  if (vocab < 1 || (vocab % 8 != 0 && rows > 1) || (reinterpret_cast<uintptr_t>(logits) & 15u) != 0) {
    set_last_error("pa_argmax: logits must be 16-byte aligned and, for several rows, vocab a multiple of 8");
    return PA_ERR_INVALID_ARG;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kArgmaxCluster, rows);
  cfg.blockDim = dim3(kArgmaxThreads);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, argmax_rows_kernel, (const __nv_bfloat16*)logits, (int*)tokens, vocab, pdl);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return PA_ERR_CUDA;
  }
  return PA_OK;
}
}  // namespace pa

extern "C" int pa_argmax(const void* logits, int32_t* tokens, int rows, int vocab, void* stream) {
  return pa::argmax_impl(logits, tokens, rows, vocab, 0, stream);
}
