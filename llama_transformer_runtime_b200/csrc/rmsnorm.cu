// RMSNorm over the rows of a prompt chunk: y = bf16((x * rsqrt(mean(x^2) + eps)) * w).
//
// The step in front of the Q/K/V projections in the reference's Attention::forward
// (src/runtime/attention.cu:118-131 calling rmsnorm_launch<2048>,
// src/kernels/rmsnorm/rmsnorm.cu:51-148: one block of 256 threads per row, uint4 loads, warp and
// block reduction, the row read twice).  For decode shapes the same arithmetic runs as the prologue
// of the projection kernel (qkv_project.cu); this kernel serves chunks of many rows, whose
// projections run on the tensor cores.  HBM-bound: rows x hidden x 2 bytes read and written once —
// the row stays in registers between the two passes, a warp owns a row, so there is no block-wide
// barrier and no shared memory.
//
// The sum of squares is formed in the reference's order (a thread's 8-element chunks in sequence
// with fused multiply-adds, lanes by shuffle-down 16..1, then the 8 groups of 32 chunks the same
// way), so the result equals the reference kernel's bit for bit for hidden = 2048.
#include <cstdio>

#include "../../include/paged_attention.h"
#include "pa_common.cuh"

namespace pa {
void set_last_error(const char* msg);
}

namespace {

constexpr int kRowsPerCta = 4;  // one warp per row
constexpr int kMaxChunksPerLane = 8;  // hidden <= 2048: 256 chunks of 8 elements, 8 per lane

// The reference's thread t (of 256) owns chunk t; its warp w = t / 32 sums chunks 32w..32w+31 by
// shuffle-down, and warp 0 then sums the 8 warp totals by shuffle-down over lanes 0..7.  Here one
// warp does the work of all 8: lane l holds chunks l, 32 + l, ..., and reproduces both levels.
__global__ void __launch_bounds__(kRowsPerCta * 32)
rmsnorm_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                    __nv_bfloat16* __restrict__ y, int rows, int hidden, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kRowsPerCta + warp;
  if (row >= rows) return;
  const int chunks = hidden / 8, groups = chunks / 32;  // groups = the reference's warps
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * hidden);
  uint4 data[kMaxChunksPerLane];
  float part[kMaxChunksPerLane];
#pragma unroll
  for (int g = 0; g < kMaxChunksPerLane; g++)
    if (g < groups) data[g] = xr[g * 32 + lane];
#pragma unroll
  for (int g = 0; g < kMaxChunksPerLane; g++) {
    if (g >= groups) continue;
    const __nv_bfloat162* bf = reinterpret_cast<const __nv_bfloat162*>(&data[g]);
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 v = __bfloat1622float2(bf[j]);
      s = __fmaf_rn(v.x, v.x, s);
      s = __fmaf_rn(v.y, v.y, s);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
    part[g] = __shfl_sync(0xffffffffu, s, 0);  // total of group g, on every lane
  }
  // second level: lanes 0..groups-1 hold the group totals, the rest zero, shuffle-down again
  float tot = 0.0f;
#pragma unroll
  for (int g = 0; g < kMaxChunksPerLane; g++)
    if (g < groups && lane == g) tot = part[g];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) tot += __shfl_down_sync(0xffffffffu, tot, off);
  tot = __shfl_sync(0xffffffffu, tot, 0);
  const float rms_recip = rsqrtf(tot / static_cast<float>(hidden) + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * hidden);
#pragma unroll
  for (int g = 0; g < kMaxChunksPerLane; g++) {
    if (g >= groups) continue;
    const uint4 wd = wr[g * 32 + lane];
    const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&data[g]);
    const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wd);
    uint4 yd;
    __nv_bfloat162* yb = reinterpret_cast<__nv_bfloat162*>(&yd);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 xf = __bfloat1622float2(xb[j]);
      const float2 wf = __bfloat1622float2(wb[j]);
      yb[j] = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(xf.x, rms_recip), wf.x),
                                    __fmul_rn(__fmul_rn(xf.y, rms_recip), wf.y));
    }
    yr[g * 32 + lane] = yd;
  }
}

}  // namespace

extern "C" int pa_rmsnorm(const void* x, const void* weight, void* y, int rows, int hidden, float eps, void* stream) {
  if (!x || !weight || !y) {
    pa::set_last_error("pa_rmsnorm: NULL argument");
    return PA_ERR_INVALID_ARG;
  }
  if (rows < 1) return PA_OK;
  if (hidden < 256 || hidden > 2048 || hidden % 256 != 0) {
    pa::set_last_error("pa_rmsnorm: hidden must be a multiple of 256, at most 2048");
    return PA_ERR_UNSUPPORTED;
  }
  rmsnorm_rows_kernel<<<(rows + kRowsPerCta - 1) / kRowsPerCta, kRowsPerCta * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)weight, (__nv_bfloat16*)y, rows, hidden, eps);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "pa_rmsnorm: %s", cudaGetErrorString(e));
    pa::set_last_error(msg);
    return PA_ERR_CUDA;
  }
  return PA_OK;
}
