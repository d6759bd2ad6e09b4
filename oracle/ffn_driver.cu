// TEST INFRASTRUCTURE — not part of the product.
//
// A caller of the reference's runtime::FeedForward (src/runtime/ffn.hpp:8-36), built twice: against
// the reference's own ffn.cu and kernels (oracle/Makefile, `callers`), and — with -DPA_SHIM_CLASS —
// against include/ffn.hpp of the product, the drop-in class over libpaged_attention.so.  Tests
// compare what the two programs write.
//
// It runs forward() for 1, 3 and 40 rows with seeded weights and writes the three outputs as raw bf16.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <initializer_list>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "ffn.hpp"
#ifdef PA_SHIM_CLASS
namespace runtime {
struct Tensor {  // a minimal stand-in for the reference's Tensor (src/runtime/tensor.hpp:9-41)
  explicit Tensor(std::initializer_list<long> shape) {
    n = 1;
    for (long d : shape) n *= d;
    if (cudaMalloc(&p, (size_t)n * sizeof(__nv_bfloat16)) != cudaSuccess) exit(2);
  }
  ~Tensor() { cudaFree(p); }
  __nv_bfloat16* data_bf16() { return p; }
  __nv_bfloat16* p = nullptr;
  long n = 0;
};
}  // namespace runtime
#define FORWARD(ffn, in, out, len) (ffn).forward((in).data_bf16(), (out).data_bf16(), len)
#else
#include "tensor.hpp"
#define FORWARD(ffn, in, out, len) (ffn).forward(in, out, len)
#endif

namespace {

uint64_t g_state = 0xD1B54A32D192ED03ull;
float uniform() {  // (-1, 1), a 64-bit LCG's upper bits
  g_state = g_state * 6364136223846793005ull + 1442695040888963407ull;
  return (float)((g_state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;
}

__nv_bfloat16* device_bf16(size_t n, float scale, float offset) {
  std::vector<__nv_bfloat16> h(n);
  for (size_t i = 0; i < n; i++) h[i] = __float2bfloat16(offset + scale * uniform());
  __nv_bfloat16* d = nullptr;
  if (cudaMalloc(&d, n * sizeof(__nv_bfloat16)) != cudaSuccess) exit(2);
  cudaMemcpy(d, h.data(), n * sizeof(__nv_bfloat16), cudaMemcpyHostToDevice);
  return d;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) {
    fprintf(stderr, "usage: %s <output file>\n", argv[0]);
    return 2;
  }
  const int H = 2048, I = 8192;
  __nv_bfloat16* norm = device_bf16(H, 0.5f, 1.0f);
  __nv_bfloat16* gate = device_bf16((size_t)H * I, 0.05f, 0.f);
  __nv_bfloat16* up = device_bf16((size_t)H * I, 0.05f, 0.f);
  __nv_bfloat16* down = device_bf16((size_t)I * H, 0.03f, 0.f);
  runtime::FeedForward ffn(norm, gate, up, down);
  FILE* f = fopen(argv[1], "wb");
  if (!f) return 2;
  for (int rows : {1, 3, 40}) {
    runtime::Tensor in({rows, H}), out({rows, H});
    std::vector<__nv_bfloat16> h((size_t)rows * H);
    for (auto& v : h) v = __float2bfloat16(1.5f * uniform());
    cudaMemcpy(in.data_bf16(), h.data(), h.size() * sizeof(__nv_bfloat16), cudaMemcpyHostToDevice);
    cudaMemset(out.data_bf16(), 0, h.size() * sizeof(__nv_bfloat16));
    FORWARD(ffn, in, out, rows);
    if (cudaDeviceSynchronize() != cudaSuccess) return 3;
    cudaMemcpy(h.data(), out.data_bf16(), h.size() * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost);
    fwrite(h.data(), sizeof(__nv_bfloat16), h.size(), f);
  }
  fclose(f);
  printf("feed-forward GPU time %.3f ms\n", runtime::FeedForward::get_accumulated_ffn_ms());
  return 0;
}
