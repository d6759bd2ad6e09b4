// Token embedding lookup: out[r, :] = table[tokens[r], :], bf16 rows of `hidden` elements.
//
// Replaces launch_embedding (src/kernels/embedding/embedding.cu:31-95: one CTA of 256 threads per
// token, bf16x2 copies), which the reference's decode loop calls after a blocking copy of the token
// id to the device (src/runtime/llama_runtime.cu:831-854) and its prefill with the prompt's ids
// (llama_runtime.cu:967-984).  Here the ids are read on the device, so the token a step produced
// feeds the next step without a host round trip.  The reference does not check the ids; a token
// outside [0, vocab) here gives a row of zeros and, where a status word is given, records
// PA_ERR_INVALID_ARG in it — it never reads outside the table.
//
// One CTA of 256 threads per row, 16-byte copies (a 2048-element row is one copy per thread).
#include <cstdint>

#include "../../include/paged_attention.h"
#include "kernels.cuh"

namespace pa {
void set_last_error(const char* msg);
}

namespace {

constexpr int kEmbedThreads = 256;

__global__ void __launch_bounds__(kEmbedThreads) embedding_rows_kernel(const int32_t* __restrict__ tokens,
                                                                      const uint4* __restrict__ table, uint4* __restrict__ out,
                                                                      int chunks, int vocab, int* status, int pdl) {
  // behind another kernel of a generation loop the ids are that kernel's output
  if (pdl) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  const int tok = tokens[blockIdx.x];
  const bool ok = tok >= 0 && tok < vocab;
  if (!ok && status && threadIdx.x == 0) atomicCAS(status, 0, PA_ERR_INVALID_ARG);
  const uint4* src = table + (size_t)(ok ? tok : 0) * chunks;
  uint4* dst = out + (size_t)blockIdx.x * chunks;
  for (int c = threadIdx.x; c < chunks; c += kEmbedThreads) dst[c] = ok ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
}

}  // namespace

namespace pa {
int embedding_impl(const int32_t* tokens, const void* table, void* out, int rows, int hidden, int vocab, int* status,
                   int pdl, void* stream) {
  if (!tokens || !table || !out) {
    set_last_error("pa_embedding: NULL argument");
    return PA_ERR_INVALID_ARG;
  }
  if (rows < 1) return PA_OK;
  if (hidden < 8 || hidden % 8 != 0 || vocab < 1 ||
      ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) & 15u) != 0) {
    set_last_error("pa_embedding: hidden must be a multiple of 8, vocab positive, table and out 16-byte aligned");
    return PA_ERR_INVALID_ARG;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(kEmbedThreads);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, embedding_rows_kernel, tokens, (const uint4*)table, (uint4*)out,
                                           hidden / 8, vocab, status, pdl);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return PA_ERR_CUDA;
  }
  return PA_OK;
}
}  // namespace pa

extern "C" int pa_embedding(const int32_t* tokens, const void* table, void* out, int rows, int hidden, int vocab,
                            void* stream) {
  return pa::embedding_impl(tokens, table, out, rows, hidden, vocab, nullptr, 0, stream);
}
