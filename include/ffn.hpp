#pragma once
// runtime::FeedForward over the library: the reference's per-layer feed-forward object
// (src/runtime/ffn.hpp:8-36, src/runtime/ffn.cu:13-145) with the same constructor arguments, the same
// forward(input, output, seq_len) and the same timing accessors, taking raw device pointers where
// the reference takes its Tensor (src/runtime/tensor.hpp:9-41; data_bf16() is what a caller passes).
//
// What forward() runs:
//   seq_len <= 8   pa_ffn: RMSNorm + gate and up projections + SiLU(gate) * up in one weight-streaming
//                  launch, the down projection in a second one; no per-call allocation.
//   seq_len  > 8   pa_ffn_rows: RMSNorm kernel, two tensor-core GEMM launches on packed copies of
//                  the weights (gate and up as one, SiLU * up in its epilogue; down).  The packed copies (100 MB) and the scratch rows
//                  are made on the first such call and kept; call reserve(max_rows) at set-up to keep
//                  forward() free of allocations.
// Like the reference's forward() it writes FeedForward(input) WITHOUT the residual (the block adds
// it, src/runtime/transformer_block.cu:76-81), returns with `output` complete and adds its GPU time
// to a process-wide accumulator.  Errors print and exit, as the reference's CUDA_CHECK does.
#include <atomic>
#include <cstdio>
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "paged_attention.h"

namespace runtime {

class FeedForward {
 public:
  FeedForward(__nv_bfloat16* ffn_norm, __nv_bfloat16* gate_proj, __nv_bfloat16* up_proj, __nv_bfloat16* down_proj) {
    w_ = {};
    w_.ffn_norm = ffn_norm;
    w_.gate = gate_proj;
    w_.up = up_proj;
    w_.down = down_proj;
    w_.rms_eps = 1e-5f;
    w_.hidden = kHidden;
    w_.inter = kInter;
    cuda(cudaMalloc(&h_, (size_t)8 * kInter * sizeof(__nv_bfloat16)));
    cuda(cudaEventCreate(&start_));
    cuda(cudaEventCreate(&stop_));
  }
  FeedForward(const FeedForward&) = delete;
  FeedForward& operator=(const FeedForward&) = delete;
  ~FeedForward() {
    cudaDeviceSynchronize();
    if (pool_) pa_pool_destroy(pool_);
    cudaFree(h_);
    cudaFree(packed_gate_);
    cudaFree(packed_up_);
    cudaFree(packed_down_);
    cudaFree(scratch_);
    cudaEventDestroy(start_);
    cudaEventDestroy(stop_);
  }

  // Set-up call for prompt chunks of up to max_rows rows: packed weight copies and scratch rows.
  void reserve(int max_rows) const {
    if (max_rows <= 8) return;
    if (!pool_) {
      int dev = 0;
      cuda(cudaGetDevice(&dev));
      pa(pa_pool_create(&pool_, dev, 1, 1, 8, 1, 1));  // carries the device status word of the GEMM launches
      const size_t bytes = (size_t)kHidden * kInter * sizeof(__nv_bfloat16);
      cuda(cudaMalloc(&packed_gate_, bytes));
      cuda(cudaMalloc(&packed_up_, bytes));
      cuda(cudaMalloc(&packed_down_, bytes));
      pa(pa_pack_projection_weights(w_.gate, packed_gate_, kHidden, kInter, nullptr));
      pa(pa_pack_projection_weights(w_.up, packed_up_, kHidden, kInter, nullptr));
      pa(pa_pack_projection_weights(w_.down, packed_down_, kInter, kHidden, nullptr));
      wp_ = w_;
      wp_.gate = packed_gate_;
      wp_.up = packed_up_;
      wp_.down = packed_down_;
    }
    if (max_rows > scratch_rows_) {
      cuda(cudaDeviceSynchronize());
      cudaFree(scratch_);
      cuda(cudaMalloc(&scratch_, (size_t)max_rows * (kHidden + kInter) * sizeof(__nv_bfloat16)));
      scratch_rows_ = max_rows;
    }
  }

  // input, output: [seq_len, 2048] bf16 on the device (the reference's Tensor::data_bf16())
  void forward(const __nv_bfloat16* input, __nv_bfloat16* output, int seq_len) const {
    if (seq_len < 1) die("forward: seq_len must be positive");
    cuda(cudaEventRecord(start_, nullptr));
    if (seq_len <= 8) {
      pa(pa_ffn(&w_, 0, input, h_, output, seq_len, /*add_residual=*/0, nullptr));
    } else {
      reserve(seq_len);
      pa(pa_ffn_rows(pool_, &wp_, 0, input, scratch_, output, seq_len, /*add_residual=*/0, nullptr));
    }
    cuda(cudaEventRecord(stop_, nullptr));
    cuda(cudaEventSynchronize(stop_));
    float ms = 0.f;
    cuda(cudaEventElapsedTime(&ms, start_, stop_));
    double old = accumulated().load(std::memory_order_relaxed);
    while (!accumulated().compare_exchange_weak(old, old + (double)ms, std::memory_order_relaxed)) {
    }
    if (pool_) pa(pa_pool_check(pool_, nullptr));
  }

  static void reset_ffn_timing() { accumulated().store(0.0); }
  static double get_accumulated_ffn_ms() { return accumulated().load(); }

 private:
  static constexpr int kHidden = 2048, kInter = 8192;
  static std::atomic<double>& accumulated() {
    static std::atomic<double> ms{0.0};
    return ms;
  }
  static void die(const char* what) {
    fprintf(stderr, "runtime::FeedForward: %s\n", what);
    exit(EXIT_FAILURE);
  }
  static void pa(int rc) {
    if (rc != PA_OK) die(pa_last_error());
  }
  static void cuda(cudaError_t e) {
    if (e != cudaSuccess) die(cudaGetErrorString(e));
  }

  pa_ffn_weights w_;
  mutable pa_ffn_weights wp_ = {};
  mutable pa_pool* pool_ = nullptr;
  __nv_bfloat16* h_ = nullptr;
  mutable __nv_bfloat16 *packed_gate_ = nullptr, *packed_up_ = nullptr, *packed_down_ = nullptr, *scratch_ = nullptr;
  mutable int scratch_rows_ = 0;
  cudaEvent_t start_ = nullptr, stop_ = nullptr;
};

}  // namespace runtime
