// Q/K/V projections of a decode step as one weight stream.
//
// The producer on the input side of the attention path: the reference computes
// q = x Wq, k = x Wk, v = x Wv with three tensor-core GEMM launches per layer
// (src/runtime/attention.cu:138-191 calling launch_gemm_2048x2048 and
// launch_gemm_2048x512, src/kernels/gemm/gemm_2048x2048.cu, gemm_2048x512.cu:
// A [M, K] row-major, B [K, N] row-major, fp32 accumulation, bf16 result), each
// followed by a device synchronisation.  In decode M is the number of sequences
// (1 to a few), so the work is reading the weights once: 12.6 MB per layer for
// Llama-3.2-1B shapes.  This kernel streams them at HBM rate for all layers of
// a step in one launch; RoPE and the cache append stay where they already are,
// inside the decode kernel that consumes q, k, v.
//
// Grid (column tile, layer): a CTA owns 32 adjacent output columns (64 bytes of
// every weight row) of the concatenated [q | k | v] output and walks all K rows:
// warp w, lane (kr, c) reads the 16-byte chunk c of rows 64 j + 8 w + kr, a
// rolling window of 16 independent loads in flight per thread (64 KiB per CTA),
// the first of them issued before x is staged.  x sits in shared
// memory as bf16.  Partial sums are reduced over the 8 row lanes by shuffles
// and over the 8 warps through shared memory in a fixed order, so the result
// does not depend on scheduling.
#include <cstdio>

#include "../../include/paged_attention.h"
#include "kernels.cuh"

namespace pa {
void set_last_error(const char* msg);
}

namespace {

constexpr int kColsPerCta = 32;
constexpr int kThreads = 256;
constexpr int kMaxHidden = 2048;

struct QkvParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* w[3];   // Wq, Wk, Wv: [hidden, n] row-major
  __nv_bfloat16* out[3];       // q, k, v: [rows, n]
  long long x_layer_stride, w_layer_stride[3], out_layer_stride[3];  // elements
  int n[3];                    // columns of q, k, v
  int tiles_q, tiles_qk;       // column tiles before k, before v
  int rows, hidden;
};

template <int ROWS>
__global__ void __launch_bounds__(kThreads) qkv_project_kernel(QkvParams p) {
  __shared__ __align__(16) __nv_bfloat16 sx[ROWS][kMaxHidden];
  __shared__ float red[8][ROWS][kColsPerCta];
  const int t = blockIdx.x, layer = blockIdx.y;
  const int which = t < p.tiles_q ? 0 : (t < p.tiles_qk ? 1 : 2);
  const int col0 = (t - (which == 0 ? 0 : (which == 1 ? p.tiles_q : p.tiles_qk))) * kColsPerCta;
  const int n = p.n[which];
  const __nv_bfloat16* w = p.w[which] + (size_t)layer * p.w_layer_stride[which];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kr = lane >> 2, c = lane & 3;

  // the first 16 weight loads go out before anything else: they do not depend on x
  const uint4* wp = reinterpret_cast<const uint4*>(w + (size_t)(warp * 8 + kr) * n + col0) + c;
  const size_t step = (size_t)64 * n / 8;  // 64 rows further, in 16-byte units
  const int n_steps = p.hidden / 64;
  uint4 wv[16];
#pragma unroll
  for (int u = 0; u < 16; u++)
    if (u < n_steps) wv[u] = __ldg(wp + (size_t)u * step);

  // x rows of this layer -> shared memory (rows beyond p.rows are zero)
  const __nv_bfloat16* x = p.x + (size_t)layer * p.x_layer_stride;
  for (int i = threadIdx.x; i < ROWS * (p.hidden / 8); i += kThreads) {
    const int r = i / (p.hidden / 8), ch = i % (p.hidden / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < p.rows) v = reinterpret_cast<const uint4*>(x + (size_t)r * p.hidden)[ch];
    reinterpret_cast<uint4*>(&sx[r][0])[ch] = v;
  }
  __syncthreads();

  float acc[ROWS][8];
#pragma unroll
  for (int r = 0; r < ROWS; r++)
#pragma unroll
    for (int i = 0; i < 8; i++) acc[r][i] = 0.f;

  // rolling window: as soon as a register's row is consumed, the row 16 steps on is requested
  for (int j0 = 0; j0 < n_steps; j0 += 16) {
#pragma unroll
    for (int u = 0; u < 16; u++) {
      if (j0 + u >= n_steps) break;
      const int k = (j0 + u) * 64 + warp * 8 + kr;
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&wv[u]);
      float wf[8];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(h2[i]);
        wf[2 * i] = f.x;
        wf[2 * i + 1] = f.y;
      }
      if (j0 + u + 16 < n_steps) wv[u] = __ldg(wp + (size_t)(j0 + u + 16) * step);
#pragma unroll
      for (int r = 0; r < ROWS; r++) {
        const float xv = __bfloat162float(sx[r][k]);
#pragma unroll
        for (int i = 0; i < 8; i++) acc[r][i] = fmaf(xv, wf[i], acc[r][i]);
      }
    }
  }
  // over the 8 row lanes of the warp
#pragma unroll
  for (int r = 0; r < ROWS; r++)
#pragma unroll
    for (int i = 0; i < 8; i++) {
      float v = acc[r][i];
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      acc[r][i] = v;
    }
  if (kr == 0) {
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
      for (int i = 0; i < 8; i++) red[warp][r][c * 8 + i] = acc[r][i];
  }
  __syncthreads();
  // over the 8 warps, in warp order
  __nv_bfloat16* out = p.out[which] + (size_t)layer * p.out_layer_stride[which];
  for (int i = threadIdx.x; i < ROWS * kColsPerCta; i += kThreads) {
    const int r = i / kColsPerCta, cc = i % kColsPerCta;
    if (r >= p.rows) continue;
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; wi++) s += red[wi][r][cc];
    out[(size_t)r * n + col0 + cc] = __float2bfloat16_rn(s);
  }
}

int qfail(int code, const char* msg) {
  pa::set_last_error(msg);
  return code;
}

}  // namespace

extern "C" int pa_qkv_project(const void* x, const void* wq, const void* wk, const void* wv, void* q, void* k,
                              void* v, int rows, int layers, int hidden, int q_cols, int kv_cols,
                              int64_t x_layer_stride, int64_t wq_layer_stride, int64_t wkv_layer_stride,
                              int64_t q_layer_stride, int64_t kv_layer_stride, void* stream) {
  if (!x || !wq || !wk || !wv || !q || !k || !v) return qfail(PA_ERR_INVALID_ARG, "pa_qkv_project: NULL argument");
  if (rows < 1 || layers < 1) return qfail(PA_ERR_INVALID_ARG, "pa_qkv_project: rows and layers must be >= 1");
  if (rows > 8)
    return qfail(PA_ERR_UNSUPPORTED, "pa_qkv_project: at most 8 rows per call (decode shapes; prefill needs a tensor-core GEMM)");
  if (hidden < 64 || hidden > kMaxHidden || hidden % 64 != 0)
    return qfail(PA_ERR_UNSUPPORTED, "pa_qkv_project: hidden must be a multiple of 64, at most 2048");
  if (q_cols < kColsPerCta || kv_cols < kColsPerCta || q_cols % kColsPerCta != 0 || kv_cols % kColsPerCta != 0)
    return qfail(PA_ERR_UNSUPPORTED, "pa_qkv_project: q_cols and kv_cols must be multiples of 32");
  if (layers > 65535) return qfail(PA_ERR_INVALID_ARG, "pa_qkv_project: too many layers");
  QkvParams p;
  p.x = (const __nv_bfloat16*)x;
  p.w[0] = (const __nv_bfloat16*)wq;
  p.w[1] = (const __nv_bfloat16*)wk;
  p.w[2] = (const __nv_bfloat16*)wv;
  p.out[0] = (__nv_bfloat16*)q;
  p.out[1] = (__nv_bfloat16*)k;
  p.out[2] = (__nv_bfloat16*)v;
  p.x_layer_stride = x_layer_stride;
  p.w_layer_stride[0] = wq_layer_stride;
  p.w_layer_stride[1] = p.w_layer_stride[2] = wkv_layer_stride;
  p.out_layer_stride[0] = q_layer_stride;
  p.out_layer_stride[1] = p.out_layer_stride[2] = kv_layer_stride;
  p.n[0] = q_cols;
  p.n[1] = p.n[2] = kv_cols;
  p.tiles_q = q_cols / kColsPerCta;
  p.tiles_qk = p.tiles_q + kv_cols / kColsPerCta;
  p.rows = rows;
  p.hidden = hidden;
  const dim3 grid(p.tiles_qk + kv_cols / kColsPerCta, layers);
  cudaStream_t st = (cudaStream_t)stream;
  if (rows == 1)
    qkv_project_kernel<1><<<grid, kThreads, 0, st>>>(p);
  else if (rows == 2)
    qkv_project_kernel<2><<<grid, kThreads, 0, st>>>(p);
  else if (rows <= 4)
    qkv_project_kernel<4><<<grid, kThreads, 0, st>>>(p);
  else
    qkv_project_kernel<8><<<grid, kThreads, 0, st>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "pa_qkv_project: %s", cudaGetErrorString(e));
    return qfail(PA_ERR_CUDA, msg);
  }
  return PA_OK;
}
