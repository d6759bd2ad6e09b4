// TEST INFRASTRUCTURE — not part of the product.
//
// A caller of the reference's runtime::Attention (src/runtime/attention.hpp:9-35), used to prove
// at run time that the reference's own Attention::forward (src/runtime/attention.cu:99-390,
// compiled unchanged) works when its three kernel launchers — launch_rope_qkv,
// transformer::launch_flash_attention, launch_flash_output_layout — come from
// libpaged_attention.so instead of the reference's rope.cu, flashattention.cu and layout.cu.
// oracle/Makefile links this file twice, once each way; tests compare what the two programs write.
//
// It runs one prompt of 37 tokens and two single-token steps through one Attention layer with
// seeded weights and writes: the three output tensors and rows 0..38 of both caches, as raw bf16.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <initializer_list>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "attention.hpp"
#ifdef PA_SHIM_CLASS
// Built against include/attention.hpp of the product (raw pointers instead of Tensor): the same
// run through the drop-in runtime::Attention class.  A minimal stand-in for the reference's Tensor.
namespace runtime {
struct Tensor {
  explicit Tensor(std::initializer_list<long> shape) {
    n = 1;
    for (long d : shape) n *= d;
    if (cudaMalloc(&p, (size_t)n * sizeof(__nv_bfloat16)) != cudaSuccess) exit(2);
  }
  ~Tensor() { cudaFree(p); }
  __nv_bfloat16* data_bf16() { return p; }
  long numel() const { return n; }
  __nv_bfloat16* p = nullptr;
  long n = 0;
};
}  // namespace runtime
#define FORWARD(att, in, out, pos, len) (att).forward((in).data_bf16(), (out).data_bf16(), pos, len)
#else
#include "tensor.hpp"
#define FORWARD(att, in, out, pos, len) (att).forward(in, out, pos, len)
#endif

namespace {

uint64_t g_state = 0x9E3779B97F4A7C15ull;
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

void fill(runtime::Tensor& t, float scale) {
  std::vector<__nv_bfloat16> h((size_t)t.numel());
  for (auto& v : h) v = __float2bfloat16(scale * uniform());
  cudaMemcpy(t.data_bf16(), h.data(), h.size() * sizeof(__nv_bfloat16), cudaMemcpyHostToDevice);
}

void dump(FILE* f, const __nv_bfloat16* dev, size_t n) {
  std::vector<__nv_bfloat16> h(n);
  cudaMemcpy(h.data(), dev, n * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost);
  fwrite(h.data(), sizeof(__nv_bfloat16), n, f);
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) return 1;
  const int max_seq = 128, prompt = 37;
  cudaSetDevice(0);
  __nv_bfloat16* norm = device_bf16(2048, 0.1f, 1.0f);
  __nv_bfloat16* wq = device_bf16((size_t)2048 * 2048, 0.05f, 0.f);
  __nv_bfloat16* wk = device_bf16((size_t)2048 * 512, 0.05f, 0.f);
  __nv_bfloat16* wv = device_bf16((size_t)2048 * 512, 0.05f, 0.f);
  __nv_bfloat16* wo = device_bf16((size_t)2048 * 2048, 0.05f, 0.f);
  std::vector<float> hc((size_t)max_seq * 32), hs((size_t)max_seq * 32);
  for (int p = 0; p < max_seq; p++)
    for (int i = 0; i < 32; i++) {
      const float inv = 1.0f / powf(500000.0f, (float)(2 * i) / 64.0f);
      hc[(size_t)p * 32 + i] = cosf((float)p * inv);
      hs[(size_t)p * 32 + i] = sinf((float)p * inv);
    }
  float *cos_t = nullptr, *sin_t = nullptr;
  cudaMalloc(&cos_t, hc.size() * 4);
  cudaMalloc(&sin_t, hs.size() * 4);
  cudaMemcpy(cos_t, hc.data(), hc.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(sin_t, hs.data(), hs.size() * 4, cudaMemcpyHostToDevice);

  runtime::Attention att(norm, wq, wk, wv, wo, cos_t, sin_t, max_seq, 0);
  FILE* f = fopen(argv[1], "wb");
  if (!f) return 3;
  {
    runtime::Tensor in({prompt, 2048}), out({prompt, 2048});
    fill(in, 1.7f);
    FORWARD(att, in, out, 0, prompt);
    cudaDeviceSynchronize();
    dump(f, out.data_bf16(), (size_t)prompt * 2048);
  }
  for (int step = 0; step < 2; step++) {
    runtime::Tensor in({1, 2048}), out({1, 2048});
    fill(in, 1.7f);
    FORWARD(att, in, out, prompt + step, 1);
    cudaDeviceSynchronize();
    dump(f, out.data_bf16(), 2048);
  }
  for (int h = 0; h < 8; h++) dump(f, att.get_key_cache() + (size_t)h * max_seq * 64, (size_t)(prompt + 2) * 64);
  for (int h = 0; h < 8; h++) dump(f, att.get_value_cache() + (size_t)h * max_seq * 64, (size_t)(prompt + 2) * 64);
  fclose(f);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "CUDA error: %s\n", cudaGetErrorString(e));
    return 4;
  }
  printf("attention ms %.3f\n", runtime::Attention::get_accumulated_attention_ms());
  return 0;
}
