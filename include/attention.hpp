#pragma once
// runtime::Attention over the paged library: the reference's per-layer attention object
// (src/runtime/attention.hpp:9-57, src/runtime/attention.cu:54-390) with the same constructor
// arguments, the same forward(input, output, position, seq_len) and the same cache and timing
// accessors, taking raw device pointers where the reference takes its Tensor (a move-only RAII
// device buffer, src/runtime/tensor.hpp:9-41, whose data_bf16() is what a caller passes here).
//
// What forward() runs, for the reference's steps 1-8:
//   seq_len == 1   pa_attention_step: RMSNorm + Q/K/V projections, RoPE + append + paged decode
//                  attention, output projection — three launches, no per-call allocation.
//   seq_len  > 1   pa_rmsnorm, pa_qkv_project_append (tensor-core GEMM with RoPE and the cache
//                  append as its epilogue), pa_prefill (tcgen05 attention), pa_out_project_rows.
// Like the reference's forward() it returns with `output` complete (it synchronises on an event;
// the reference synchronises the device after every step) and adds its GPU time to a process-wide
// accumulator.  Errors print and exit, as the reference's CUDA_CHECK does.
//
// Ownership: the object owns one pool of ceil(max_seq_len / 16) blocks for its layer (the
// reference owns two [8, max_seq_len, 64] tensors), packed copies of the four weight matrices for
// the tensor-core path, and the rows between its kernels; it borrows the weights and RoPE tables.
// position must equal the number of tokens already cached; position == 0 starts a new sequence.
#include <atomic>
#include <cstdio>
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "paged_attention.h"

namespace runtime {

class Attention {
 public:
  Attention(__nv_bfloat16* input_norm, __nv_bfloat16* q_proj, __nv_bfloat16* k_proj, __nv_bfloat16* v_proj,
            __nv_bfloat16* o_proj, float* cos_table, float* sin_table, int max_seq_len, int layer_idx)
      : cos_table_(cos_table), sin_table_(sin_table), max_seq_len_(max_seq_len), layer_idx_(layer_idx) {
    w_.input_norm = input_norm;
    w_.wq = q_proj;
    w_.wk = k_proj;
    w_.wv = v_proj;
    w_.wo = o_proj;
    w_.norm_layer_stride = w_.wq_layer_stride = w_.wkv_layer_stride = w_.wo_layer_stride = 0;
    w_.rms_eps = 1e-5f;
    w_.hidden = kHidden;
    int dev = 0;
    cuda(cudaGetDevice(&dev));
    const int blocks = (max_seq_len + PA_BLOCK_TOKENS - 1) / PA_BLOCK_TOKENS;
    pa(pa_pool_create(&pool_, dev, 1, blocks, 8, 1, blocks));
    pa(pa_seq_create(pool_, &seq_));
    const size_t big = (size_t)kHidden * kHidden * sizeof(__nv_bfloat16), small = (size_t)kHidden * 512 * sizeof(__nv_bfloat16);
    cuda(cudaMalloc(&packed_q_, big));
    cuda(cudaMalloc(&packed_k_, small));
    cuda(cudaMalloc(&packed_v_, small));
    cuda(cudaMalloc(&packed_o_, big));
    pa(pa_pack_projection_weights(q_proj, packed_q_, kHidden, kHidden, nullptr));
    pa(pa_pack_projection_weights(k_proj, packed_k_, kHidden, 512, nullptr));
    pa(pa_pack_projection_weights(v_proj, packed_v_, kHidden, 512, nullptr));
    pa(pa_pack_projection_weights(o_proj, packed_o_, kHidden, kHidden, nullptr));
    const size_t rows = (size_t)max_seq_len * kHidden * sizeof(__nv_bfloat16);
    cuda(cudaMalloc(&normalized_, rows));
    cuda(cudaMalloc(&q_rot_, rows));
    cuda(cudaMalloc(&attn_, rows));
    const size_t cache = (size_t)8 * max_seq_len * 64 * sizeof(__nv_bfloat16);
    cuda(cudaMalloc(&key_view_, cache));
    cuda(cudaMalloc(&value_view_, cache));
    cuda(cudaMemset(key_view_, 0, cache));
    cuda(cudaMemset(value_view_, 0, cache));
    cuda(cudaEventCreate(&start_));
    cuda(cudaEventCreate(&stop_));
    cuda(cudaDeviceSynchronize());
  }
  Attention(const Attention&) = delete;
  Attention& operator=(const Attention&) = delete;
  ~Attention() {
    cudaDeviceSynchronize();
    pa_pool_destroy(pool_);
    cudaFree(packed_q_);
    cudaFree(packed_k_);
    cudaFree(packed_v_);
    cudaFree(packed_o_);
    cudaFree(normalized_);
    cudaFree(q_rot_);
    cudaFree(attn_);
    cudaFree(key_view_);
    cudaFree(value_view_);
    cudaEventDestroy(start_);
    cudaEventDestroy(stop_);
  }

  // input, output: [seq_len, 2048] bf16 on the device (the reference's Tensor::data_bf16())
  void forward(const __nv_bfloat16* input, __nv_bfloat16* output, int position, int seq_len) {
    const int tokens = seq_len;
    if (tokens < 1 || position < 0 || position + tokens > max_seq_len_) die("forward: position/seq_len outside the cache");
    int cached = 0;
    pa(pa_seq_length(pool_, seq_, &cached));
    if (position == 0 && cached > 0) {  // a new conversation: hand the blocks back and start over
      pa(pa_seq_free(pool_, seq_));
      pa(pa_seq_create(pool_, &seq_));
      cached = 0;
    }
    if (position != cached) die("forward: position must equal the number of cached tokens");
    cuda(cudaEventRecord(start_, nullptr));
    pa(pa_seq_reserve(pool_, seq_, position + tokens));
    const int32_t id = seq_, n_new = tokens;
    pa(pa_batch_set(pool_, &id, &n_new, 1, nullptr));
    const float scale = 0.125f;  // 1 / sqrt(64), src/runtime/attention.cu:318
    if (tokens == 1) {
      pa(pa_attention_step(pool_, nullptr, 0, 1, &w_, input, output, /*add_residual=*/0, cos_table_, sin_table_, scale,
                           nullptr));
    } else {
      pa(pa_rmsnorm(input, w_.input_norm, normalized_, tokens, kHidden, w_.rms_eps, nullptr));
      pa(pa_qkv_project_append(pool_, 0, normalized_, packed_q_, packed_k_, packed_v_, cos_table_, sin_table_, q_rot_,
                               kHidden, nullptr));
      pa(pa_prefill(pool_, 0, q_rot_, attn_, nullptr, scale, nullptr));
      pa(pa_out_project_rows(pool_, attn_, packed_o_, nullptr, output, tokens, kHidden, kHidden, nullptr));
    }
    cuda(cudaEventRecord(stop_, nullptr));
    cuda(cudaEventSynchronize(stop_));
    float ms = 0.f;
    cuda(cudaEventElapsedTime(&ms, start_, stop_));
    double old = accumulated().load(std::memory_order_relaxed);
    while (!accumulated().compare_exchange_weak(old, old + (double)ms, std::memory_order_relaxed)) {
    }
    pa(pa_pool_check(pool_, nullptr));
  }

  // [8, max_seq_len, 64], the view the reference keeps as its cache (rows beyond the cached
  // tokens are zero); refreshed from the paged cache on every call.
  const __nv_bfloat16* get_key_cache() const {
    refresh_views();
    return key_view_;
  }
  const __nv_bfloat16* get_value_cache() const {
    refresh_views();
    return value_view_;
  }

  static void reset_attention_timing() { accumulated().store(0.0); }
  static double get_accumulated_attention_ms() { return accumulated().load(); }

 private:
  static constexpr int kHidden = 2048;
  static std::atomic<double>& accumulated() {
    static std::atomic<double> ms{0.0};
    return ms;
  }
  static void die(const char* what) {
    fprintf(stderr, "runtime::Attention: %s\n", what);
    exit(EXIT_FAILURE);
  }
  static void pa(int rc) {
    if (rc != PA_OK) die(pa_last_error());
  }
  static void cuda(cudaError_t e) {
    if (e != cudaSuccess) die(cudaGetErrorString(e));
  }
  void refresh_views() const {
    int cached = 0;
    pa(pa_seq_length(pool_, seq_, &cached));
    if (cached > 0) pa(pa_gather_kv(pool_, 0, seq_, key_view_, value_view_, max_seq_len_, nullptr));
    cuda(cudaStreamSynchronize(nullptr));
  }

  pa_attention_weights w_;
  float* cos_table_;
  float* sin_table_;
  int max_seq_len_;
  int layer_idx_;
  pa_pool* pool_ = nullptr;
  int seq_ = -1;
  __nv_bfloat16 *packed_q_ = nullptr, *packed_k_ = nullptr, *packed_v_ = nullptr, *packed_o_ = nullptr;
  __nv_bfloat16 *normalized_ = nullptr, *q_rot_ = nullptr, *attn_ = nullptr;
  __nv_bfloat16 *key_view_ = nullptr, *value_view_ = nullptr;
  cudaEvent_t start_ = nullptr, stop_ = nullptr;
};

}  // namespace runtime
