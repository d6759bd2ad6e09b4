// TEST INFRASTRUCTURE — not part of the product.
//
// The reference's whole decode step, run both ways on the same seeded model.  oracle/Makefile builds
// this file into _ref/token_forward_ref with the reference's own runtime::Transformer
// (src/runtime/transformer.cu, transformer_block.cu, attention.cu, ffn.cu, tensor.cu, compiled
// unchanged, with all of the reference's kernels) and the calls its LlamaRuntime::decode_forward makes
// around it (src/runtime/llama_runtime.cu:822-945: launch_embedding, Transformer::forward,
// rmsnorm_launch<2048>, launch_gemm_2048x128256, launch_argmax — LlamaRuntime itself needs a
// tokenizer and a weight file, so its body is restated here call for call, and forward_prefill's,
// llama_runtime.cu:947-1075, for the prompt).  The test builds the same file twice against
// libpaged_attention.so: with -DPA_SHIM_CLASS the same calls on the drop-in classes and entry points
// (include/transformer.hpp's runtime::Transformer, pa_embedding, pa_lm_head, pa_argmax), with -DPA_SHIM
// every token, the prompt's too, as one pa_decode_token step.
//
// All programs fill the Llama-3.2-1B-shaped weights (3 GB) on the device from the same hash, start
// with an empty cache, run a prompt of 21 fixed ids (one forward of 21 rows; single-token steps with
// -DPA_SHIM) and then feed twelve fixed ids one per step (not the generated ones, so that the runs stay on
// the same inputs).  They write the logits row (128256 bf16) and the greedy token after the prompt and
// after every step.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <initializer_list>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#if defined(PA_SHIM)
#include "paged_attention.h"
#elif defined(PA_SHIM_CLASS)
#include "transformer.hpp"
namespace runtime {
// A minimal stand-in for the reference's Tensor (the drop-in classes take raw pointers).
struct Tensor {
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
#define FORWARD(t, in, out, pos, len) (t).forward((in).data_bf16(), (out).data_bf16(), pos, len)
#define PA(call)                                         \
  do {                                                   \
    if ((call) != PA_OK) {                               \
      fprintf(stderr, "%s: %s\n", #call, pa_last_error()); \
      exit(5);                                           \
    }                                                    \
  } while (0)
#else
#include "argmax_128256.hpp"
#include "embedding.hpp"
#include "gemm_2048x128256.hpp"
#include "rmsnorm.hpp"
#include "transformer.hpp"
#define FORWARD(t, in, out, pos, len) (t).forward(in, out, pos, len)
#endif

namespace {

constexpr int kLayers = 16, kHidden = 2048, kInter = 8192, kVocab = 128256, kQ = 2048, kKv = 512;
constexpr int kSteps = 12, kPrompt = 21, kMaxSeq = 64;

#define CK(call)                                                                        \
  do {                                                                                  \
    cudaError_t e_ = (call);                                                            \
    if (e_ != cudaSuccess) {                                                            \
      fprintf(stderr, "%s: %s (line %d)\n", #call, cudaGetErrorString(e_), __LINE__);   \
      exit(2);                                                                          \
    }                                                                                   \
  } while (0)

// element i of stream `seed`: offset + scale * u, u uniform in (-1, 1) from a 64-bit mix of (seed, i);
// with hot_cols > 0 the matrix has hot_cols columns and every 64th of them is 16 times larger (a head
// whose largest logits stand out, so that the greedy token is not decided by the last bit)
__global__ void fill_kernel(__nv_bfloat16* p, size_t n, uint64_t seed, float scale, float offset, int hot_cols) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + i + 1;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    const float u = (float)(z >> 40) / 8388608.0f - 1.0f;
    const float hot = hot_cols > 0 && (i % (size_t)hot_cols) % 64 == 0 ? 16.0f : 1.0f;
    p[i] = __float2bfloat16(offset + hot * scale * u);
  }
}

__nv_bfloat16* device_fill(size_t n, uint64_t seed, float scale, float offset, int hot_cols = 0) {
  __nv_bfloat16* d = nullptr;
  CK(cudaMalloc(&d, n * sizeof(__nv_bfloat16)));
  fill_kernel<<<1184, 256>>>(d, n, seed, scale, offset, hot_cols);
  CK(cudaGetLastError());
  return d;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) return 1;
  CK(cudaSetDevice(0));
  // per-kind buffers with the layers stacked, so that one layout serves both builds
  __nv_bfloat16* in_norm = device_fill((size_t)kLayers * kHidden, 1, 0.1f, 1.0f);
  __nv_bfloat16* wq = device_fill((size_t)kLayers * kHidden * kQ, 2, 0.05f, 0.f);
  __nv_bfloat16* wk = device_fill((size_t)kLayers * kHidden * kKv, 3, 0.05f, 0.f);
  __nv_bfloat16* wv = device_fill((size_t)kLayers * kHidden * kKv, 4, 0.05f, 0.f);
  __nv_bfloat16* wo = device_fill((size_t)kLayers * kQ * kHidden, 5, 0.05f, 0.f);
  __nv_bfloat16* post_norm = device_fill((size_t)kLayers * kHidden, 6, 0.1f, 1.0f);
  __nv_bfloat16* wg = device_fill((size_t)kLayers * kHidden * kInter, 7, 0.05f, 0.f);
  __nv_bfloat16* wu = device_fill((size_t)kLayers * kHidden * kInter, 8, 0.05f, 0.f);
  __nv_bfloat16* wd = device_fill((size_t)kLayers * kInter * kHidden, 9, 0.025f, 0.f);
  __nv_bfloat16* embed = device_fill((size_t)kVocab * kHidden, 10, 1.7f, 0.f);
  __nv_bfloat16* final_norm = device_fill((size_t)kHidden, 11, 0.1f, 1.0f);
  __nv_bfloat16* lm_head = device_fill((size_t)kHidden * kVocab, 12, 0.01f, 0.f, kVocab);
  CK(cudaDeviceSynchronize());

  std::vector<float> hc((size_t)kMaxSeq * 32), hs((size_t)kMaxSeq * 32);
  for (int p = 0; p < kMaxSeq; p++)
    for (int i = 0; i < 32; i++) {
      const float inv = 1.0f / powf(500000.0f, (float)(2 * i) / 64.0f);
      hc[(size_t)p * 32 + i] = cosf((float)p * inv);
      hs[(size_t)p * 32 + i] = sinf((float)p * inv);
    }
  float *cos_t = nullptr, *sin_t = nullptr;
  CK(cudaMalloc(&cos_t, hc.size() * 4));
  CK(cudaMalloc(&sin_t, hs.size() * 4));
  CK(cudaMemcpy(cos_t, hc.data(), hc.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(sin_t, hs.data(), hs.size() * 4, cudaMemcpyHostToDevice));

  const int fed[kSteps] = {128000, 9906, 1917, 0, 128255, 31415, 27182, 8128, 496, 65536, 100000, 7};
  int prompt[kPrompt];
  for (int i = 0; i < kPrompt; i++) prompt[i] = (int)((1000003ull * (unsigned)(i + 1) + 12345) % kVocab);
  int* d_tok = nullptr;
  int* d_next = nullptr;
  __nv_bfloat16* logits = nullptr;
  CK(cudaMalloc(&d_tok, kPrompt * sizeof(int)));
  CK(cudaMalloc(&d_next, sizeof(int)));
  CK(cudaMalloc(&logits, (size_t)kVocab * sizeof(__nv_bfloat16)));
  FILE* f = fopen(argv[1], "wb");
  if (!f) return 3;
  std::vector<__nv_bfloat16> h_logits(kVocab);
  auto record = [&](const char* what, int fed_id) {
    CK(cudaDeviceSynchronize());
    int next = -1;
    CK(cudaMemcpy(&next, d_next, sizeof(int), cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(h_logits.data(), logits, (size_t)kVocab * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost));
    fwrite(h_logits.data(), sizeof(__nv_bfloat16), kVocab, f);
    fwrite(&next, sizeof(int), 1, f);
    printf("%s: fed %d -> %d\n", what, fed_id, next);
  };

#if defined(PA_SHIM)
  pa_pool* pool = nullptr;
  if (pa_pool_create(&pool, 0, kLayers, 16, 8, 1, 8) != PA_OK) {
    fprintf(stderr, "%s\n", pa_last_error());
    return 4;
  }
  int seq = -1;
  pa_seq_create(pool, &seq);
  pa_attention_weights aw = {};
  aw.input_norm = in_norm;
  aw.wq = wq;
  aw.wk = wk;
  aw.wv = wv;
  aw.wo = wo;
  aw.norm_layer_stride = kHidden;
  aw.wq_layer_stride = (int64_t)kHidden * kQ;
  aw.wkv_layer_stride = (int64_t)kHidden * kKv;
  aw.wo_layer_stride = (int64_t)kQ * kHidden;
  aw.rms_eps = 1e-5f;
  aw.hidden = kHidden;
  pa_ffn_weights fw = {};
  fw.ffn_norm = post_norm;
  fw.gate = wg;
  fw.up = wu;
  fw.down = wd;
  fw.norm_layer_stride = kHidden;
  fw.gate_layer_stride = fw.up_layer_stride = fw.down_layer_stride = (int64_t)kHidden * kInter;
  fw.rms_eps = 1e-5f;
  fw.hidden = kHidden;
  fw.inter = kInter;
  pa_model_weights model = {embed, &aw, &fw, final_norm, lm_head, kVocab, 1e-5f};
  auto token_step = [&](int id, int position) {
    const int one = 1;
    CK(cudaMemcpy(d_tok, &id, sizeof(int), cudaMemcpyHostToDevice));
    int rc = pa_seq_reserve(pool, seq, position + 1);
    if (rc == PA_OK) rc = pa_batch_set(pool, &seq, &one, 1, nullptr);
    if (rc == PA_OK) rc = pa_decode_token(pool, &model, d_tok, d_next, logits, cos_t, sin_t, 0.125f, 0, nullptr);
    if (rc == PA_OK) rc = pa_pool_check(pool, nullptr);
    if (rc != PA_OK) {
      fprintf(stderr, "position %d: %s\n", position, pa_last_error());
      exit(5);
    }
  };
  for (int i = 0; i < kPrompt; i++) token_step(prompt[i], i);
  record("prompt", prompt[kPrompt - 1]);
  for (int step = 0; step < kSteps; step++) {
    token_step(fed[step], kPrompt + step);
    record("step", fed[step]);
  }
#else
  llama::LlamaWeights weights;
  for (int l = 0; l < kLayers; l++) {
    auto& w = weights.layers[l];
    w.input_layernorm = in_norm + (size_t)l * kHidden;
    w.q_proj = wq + (size_t)l * kHidden * kQ;
    w.k_proj = wk + (size_t)l * kHidden * kKv;
    w.v_proj = wv + (size_t)l * kHidden * kKv;
    w.o_proj = wo + (size_t)l * kQ * kHidden;
    w.post_attention_layernorm = post_norm + (size_t)l * kHidden;
    w.gate_proj = wg + (size_t)l * kHidden * kInter;
    w.up_proj = wu + (size_t)l * kHidden * kInter;
    w.down_proj = wd + (size_t)l * kInter * kHidden;
  }
  weights.embed_tokens = embed;
  weights.final_norm = final_norm;
  weights.lm_head = lm_head;
  runtime::Transformer transformer(weights, cos_t, sin_t, kMaxSeq);
  runtime::Tensor last_hidden_state({1, kHidden}), final_norm_output({1, kHidden});
  // the end of both forward_prefill and decode_forward: final norm, head, greedy token
  auto head = [&](const __nv_bfloat16* row) {
#ifdef PA_SHIM_CLASS
    PA(pa_lm_head(row, weights.final_norm, 1e-5f, weights.lm_head, logits, 1, kHidden, kVocab, nullptr));
    PA(pa_argmax(logits, d_next, 1, kVocab, nullptr));
#else
    rmsnorm_launch<llama::HIDDEN_SIZE>(row, weights.final_norm, final_norm_output.data_bf16(), 1, 1e-5f);
    cudaDeviceSynchronize();
    launch_gemm_2048x128256(final_norm_output.data_bf16(), weights.lm_head, logits, 1, llama::VOCAB_SIZE,
                            llama::HIDDEN_SIZE);
    cudaDeviceSynchronize();
    launch_argmax(logits, d_next, 0);
#endif
  };
  auto embed_rows = [&](int n, __nv_bfloat16* out) {
#ifdef PA_SHIM_CLASS
    PA(pa_embedding(d_tok, weights.embed_tokens, out, n, kHidden, kVocab, nullptr));
#else
    launch_embedding(d_tok, weights.embed_tokens, out, n);
#endif
    cudaDeviceSynchronize();
  };
  {  // forward_prefill
    runtime::Tensor hidden_states({kPrompt, kHidden}), transformer_output({kPrompt, kHidden});
    CK(cudaMemcpy(d_tok, prompt, kPrompt * sizeof(int), cudaMemcpyHostToDevice));
    embed_rows(kPrompt, hidden_states.data_bf16());
    FORWARD(transformer, hidden_states, transformer_output, 0, kPrompt);
    cudaDeviceSynchronize();
    CK(cudaMemcpy(last_hidden_state.data_bf16(), transformer_output.data_bf16() + (size_t)(kPrompt - 1) * kHidden,
                  kHidden * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice));
    head(last_hidden_state.data_bf16());
    record("prompt", prompt[kPrompt - 1]);
  }
  runtime::Tensor hidden_states({1, kHidden}), transformer_output({1, kHidden});
  for (int step = 0; step < kSteps; step++) {  // decode_forward
    CK(cudaMemcpy(d_tok, &fed[step], sizeof(int), cudaMemcpyHostToDevice));
    embed_rows(1, hidden_states.data_bf16());
    FORWARD(transformer, hidden_states, transformer_output, kPrompt + step, 1);
    cudaDeviceSynchronize();
    head(transformer_output.data_bf16());
    record("step", fed[step]);
  }
#endif
  fclose(f);
  CK(cudaGetLastError());
  return 0;
}
