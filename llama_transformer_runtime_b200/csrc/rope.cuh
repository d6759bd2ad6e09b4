// Half-split RoPE arithmetic shared by the append kernel and the legacy
// launch_rope_qkv entry.
#pragma once
#include "pa_common.cuh"

namespace pa {

// y0 = x0*c - x1*s,  y1 = x0*s + x1*c  in fp32, rounded to bf16 (nearest even).
// The grouping of roundings is what the reference's compiled kernel does
// (src/kernels/rope/rope.cu:90-98, built for sm_100a): y1 is a fused
// multiply-add onto the rounded product x1*c, and so is y0 (VARIANT 1:
// fma(x0, c, -(x1*s)); measured equal to the reference on 8.4 M random values,
// the other two groupings are kept for the test that pins this).
template <int VARIANT>
__device__ __forceinline__ void rope_pair(float x0, float x1, float c, float s, float& y0,
                                          float& y1) {
  if (VARIANT == 0) {
    y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
  } else if (VARIANT == 1) {
    y0 = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
  } else {
    y0 = __fmaf_rn(-x1, s, __fmul_rn(x0, c));
  }
  y1 = __fmaf_rn(x0, s, __fmul_rn(x1, c));
}

// One thread's share of a 64-wide head: chunk `lo` (elements 8c..8c+7) and its
// partner `hi` (elements 32+8c..), with the 8 cos/sin values of pairs 8c..8c+7.
template <int VARIANT>
__device__ __forceinline__ void rope_chunks(const uint4& lo, const uint4& hi, const float* c8,
                                            const float* s8, uint4& out_lo, uint4& out_hi) {
  const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(&lo);
  const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&hi);
  __nv_bfloat16* ya = reinterpret_cast<__nv_bfloat16*>(&out_lo);
  __nv_bfloat16* yb = reinterpret_cast<__nv_bfloat16*>(&out_hi);
#pragma unroll
  for (int i = 0; i < 8; i++) {
    float y0, y1;
    rope_pair<VARIANT>(__bfloat162float(a[i]), __bfloat162float(b[i]), c8[i], s8[i], y0, y1);
    ya[i] = __float2bfloat16_rn(y0);
    yb[i] = __float2bfloat16_rn(y1);
  }
}

}  // namespace pa
