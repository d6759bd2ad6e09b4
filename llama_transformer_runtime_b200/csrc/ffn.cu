// The feed-forward block of a decode step as two weight streams.
//
// The component after the attention path in the reference's TransformerBlock
// (src/runtime/ffn.cu:34-145): RMSNorm (rmsnorm_launch<2048>), gate = x Wg and up = x Wu
// (launch_gemm_2048x8192, twice), h = SiLU(gate) * up (launch_silu_mul,
// src/kernels/silu/silu_8192.cu:55-100), y = h Wd (launch_gemm_8192x2048), each on the default
// stream with per-call temporaries; the block adds y to its input afterwards
// (src/runtime/transformer_block.cu:76-81).  In decode the rows are the sequences of the step (1 to
// a few), so the work is reading the weights once: 2 x 33.5 MB + 33.5 MB per layer for
// Llama-3.2-1B shapes, eight times the attention block's weights.
//
// Numerics follow the reference chain: the normalised row is bf16 (arithmetic and summation order of
// the reference's RMSNorm kernel); gate and up are fp32 sums rounded to bf16 (the GEMMs' outputs);
// h = bf16((g * (1 / (1 + __expf(-g)))) * u) in fp32 on those bf16 values; y is an fp32 sum rounded
// to bf16; with a residual, out = bf16(residual + y) as residual_add does.
//
// ffn_gate_up_mma_kernel: a CTA owns 32 adjacent columns of BOTH Wg and Wu and walks all rows in steps
// of 128: warp w copies rows 16 w .. 16 w + 15 of a step (64 bytes of each matrix per row) into its own
// slot of a shared-memory ring with cp.async, five steps ahead, the first of them before x is staged,
// and multiplies them on the tensor cores (mma.sync m16n8k16, ldmatrix.trans).
// ffn_down_mma_kernel: a cluster of four CTAs owns 32 adjacent columns of Wd; CTA s of the cluster walks
// rows [s K/4, (s+1) K/4) (64 column tiles alone would leave half of the SMs idle); the four partial
// sums are added in rank order by the cluster's first CTA, which reads its peers' shared memory, so
// the result does not depend on scheduling.
#include <cstdio>

#include "../../include/paged_attention.h"
#include "kernels.cuh"
#include "mma_stream.cuh"

namespace pa {
void set_last_error(const char* msg);
}

namespace {

using namespace pa;
constexpr int kColsPerCta = kStreamCols;
constexpr int kThreads = kStreamThreads;
constexpr int kSlice = kStreamRowLen;   // rows of a weight matrix one CTA walks = elements of x it stages
constexpr int kDownSplit = 4;  // CTAs of a cluster of the down projection

struct FfnParams {
  const __nv_bfloat16* x;       // gate/up: [rows, hidden]; down: h [rows, inter]
  const __nv_bfloat16* w0;      // gate/up: Wg [hidden, inter]; down: Wd [inter, hidden]
  const __nv_bfloat16* w1;      // gate/up: Wu
  __nv_bfloat16* out;           // gate/up: h [rows, inter]; down: [rows, hidden]
  const __nv_bfloat16* residual;  // down: [rows, hidden], nullable
  const __nv_bfloat16* norm_w;    // gate/up: [hidden], nullable
  int rows, k, n;               // k: rows of the weight matrix, n: its columns
  float eps;
  int pdl;
};

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float ld_peer_shared(const float* local, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(pa::smem_u32(local)), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
  return v;
}

// ROWS rows of `len` (<= kSlice) elements -> shared memory; rows beyond `rows` are zero.
template <int ROWS>
__device__ __forceinline__ void stage_rows(__nv_bfloat16 (*sx)[kSlice], const __nv_bfloat16* x, size_t row_pitch,
                                           int rows, int len) {
  for (int i = threadIdx.x; i < ROWS * (len / 8); i += kThreads) {
    const int r = i / (len / 8), ch = i % (len / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) v = reinterpret_cast<const uint4*>(x + (size_t)r * row_pitch)[ch];
    reinterpret_cast<uint4*>(&sx[r][0])[ch] = v;
  }
}

// RMSNorm of the staged rows, in place, with the arithmetic AND the summation order of the
// reference's kernel (src/kernels/rmsnorm/rmsnorm.cu:51-110, launched with 256 threads): a thread
// sums the squares of its 8-element chunks in order, lanes combine by shuffle-down (16, 8, 4, 2, 1),
// warp sums combine the same way in warp 0; y = bf16((x * r) * w).
template <int ROWS>
__device__ __forceinline__ void rmsnorm_rows(__nv_bfloat16 (*sx)[kSlice], const __nv_bfloat16* norm_w, int rows,
                                             int hidden, float eps, float* scratch /* 9 floats */) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint4* nw = reinterpret_cast<const uint4*>(norm_w);
#pragma unroll
  for (int r = 0; r < ROWS; r++) {
    if (r >= rows) break;  // uniform
    float sum_sq = 0.0f;
    for (int i = threadIdx.x; i < hidden / 8; i += kThreads) {
      const uint4 data = reinterpret_cast<const uint4*>(&sx[r][0])[i];
      const __nv_bfloat162* bf = reinterpret_cast<const __nv_bfloat162*>(&data);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 v = __bfloat1622float2(bf[j]);
        sum_sq = __fmaf_rn(v.x, v.x, sum_sq);
        sum_sq = __fmaf_rn(v.y, v.y, sum_sq);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum_sq += __shfl_down_sync(0xffffffffu, sum_sq, off);
    if (lane == 0) scratch[warp] = sum_sq;
    __syncthreads();
    float tot = lane < kThreads / 32 ? scratch[lane] : 0.0f;
    if (warp == 0) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) tot += __shfl_down_sync(0xffffffffu, tot, off);
      if (lane == 0) scratch[8] = tot;
    }
    __syncthreads();
    const float rms_recip = rsqrtf(scratch[8] / static_cast<float>(hidden) + eps);
    for (int i = threadIdx.x; i < hidden / 8; i += kThreads) {
      const uint4 xd = reinterpret_cast<const uint4*>(&sx[r][0])[i];
      const uint4 wd = nw[i];
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xd);
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
      reinterpret_cast<uint4*>(&sx[r][0])[i] = yd;  // a thread rewrites only chunks it alone read
    }
    __syncthreads();  // scratch is reused by the next row
  }
}

// Ring depths, measured in the block chain at 1 row (us per layer; gate/up x down): 3 x 8 38.9, 4 x 8 39.0,
// 5 x 4 38.7, 5 x 8 36.7, 5 x 12 36.3, 5 x 16 40.3, 6 x 12 36.2.  Two CTAs per SM must fit: 12 steps of
// the down projection only up to 4 rows.
constexpr int kGateUpStages = 5;
template <int ROWS>
constexpr int kDownStages = ROWS <= 4 ? 12 : 8;
template <int ROWS>
constexpr int gate_up_smem() { return kGateUpStages * 2 * kMmaStepBytes + ROWS * kSlice * 2; }
template <int ROWS>
constexpr int down_smem() { return kDownStages<ROWS> * kMmaStepBytes + ROWS * kSlice * 2; }

template <int ROWS>
__global__ void __launch_bounds__(kThreads, 2) ffn_gate_up_mma_kernel(FfnParams p) {
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ float nscratch[16];
  auto sx = reinterpret_cast<__nv_bfloat16(*)[kSlice]>(dyn + kGateUpStages * 2 * kMmaStepBytes);
  const int col0 = blockIdx.x * kColsPerCta;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  MmaStream<2, kGateUpStages> st;
  st.w[0] = p.w0 + col0;
  st.w[1] = p.w1 + col0;
  st.n = (size_t)p.n;
  st.ring = pa::smem_u32(dyn);
  st.n_steps = p.k / kMmaStepRows;
  st.warp = warp;
  st.lane = lane;
  st.k_total = p.k;
  st.prologue();  // the weights do not depend on the kernel in front; x does
  uint4 nw8[ROWS >= 4 ? 8 : 1];   // nor do this lane's chunks of the norm weight (kernels of 4 and 8 rows)
  if constexpr (ROWS >= 4) {
    if (p.norm_w) {
#pragma unroll
      for (int g = 0; g < 8; g++) nw8[g] = __ldg(reinterpret_cast<const uint4*>(p.norm_w) + g * 32 + lane);
    }
  }
  if (p.pdl) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  stage_rows<ROWS>(sx, p.x, (size_t)p.k, p.rows, p.k);
  __syncthreads();
  // the reference kernel's arithmetic and summation order either way: with more than 2 rows one warp
  // per row side by side, else the whole CTA on a row (a warp alone needs 1 us longer for one row)
  if constexpr (ROWS >= 4) {
    if (p.norm_w) {
      if (warp < ROWS && warp < p.rows) rmsnorm_row_by_warp(&sx[warp][0], nw8, p.k, p.eps, lane);
      __syncthreads();
    }
  } else {
    if (p.norm_w) rmsnorm_rows<ROWS>(sx, p.norm_w, p.rows, p.k, p.eps, nscratch);
  }
  float acc[2][4][4];
  st.template run<ROWS>(sx, acc);
  __syncthreads();  // every warp is done with the ring
  float* red = reinterpret_cast<float*>(dyn);
  store_partials<2, ROWS>(red, acc, warp, lane);
  __syncthreads();
  // over the 8 warps, in warp order; then SiLU(gate) * up on the two bf16 GEMM outputs
  for (int i = threadIdx.x; i < ROWS * kColsPerCta; i += kThreads) {
    const int r = i / kColsPerCta, cc = i % kColsPerCta;
    if (r >= p.rows) continue;
    float sg = 0.f, su = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; wi++) {
      sg += red[(((size_t)wi * ROWS + r) * 2 + 0) * kColsPerCta + cc];
      su += red[(((size_t)wi * ROWS + r) * 2 + 1) * kColsPerCta + cc];
    }
    const float g = __bfloat162float(__float2bfloat16_rn(sg));
    const float u = __bfloat162float(__float2bfloat16_rn(su));
    const float s = __fmul_rn(g, 1.0f / (1.0f + __expf(-g)));
    p.out[(size_t)r * p.n + col0 + cc] = __float2bfloat16_rn(__fmul_rn(s, u));
  }
}

template <int ROWS>
__global__ void __cluster_dims__(kDownSplit, 1, 1) __launch_bounds__(kThreads, 2) ffn_down_mma_kernel(FfnParams p) {
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ float part[ROWS][kColsPerCta];
  auto sx = reinterpret_cast<__nv_bfloat16(*)[kSlice]>(dyn + kDownStages<ROWS> * kMmaStepBytes);
  const uint32_t split = cluster_ctarank();
  const int col0 = (int)(blockIdx.x / kDownSplit) * kColsPerCta;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = p.n;
  const int k_slice = p.k / kDownSplit;  // rows of Wd this CTA walks
  const int k0 = (int)split * k_slice;
  MmaStream<1, kDownStages<ROWS>> st;
  st.w[0] = p.w0 + (size_t)k0 * n + col0;
  st.n = (size_t)n;
  st.ring = pa::smem_u32(dyn);
  st.n_steps = k_slice / kMmaStepRows;
  st.warp = warp;
  st.lane = lane;
  st.k_total = k_slice;
  st.prologue();
  if (p.pdl) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  stage_rows<ROWS>(sx, p.x + k0, (size_t)p.k, p.rows, k_slice);
  __syncthreads();
  float acc[1][4][4];
  st.template run<ROWS>(sx, acc);
  __syncthreads();
  float* red = reinterpret_cast<float*>(dyn);
  store_partials<1, ROWS>(red, acc, warp, lane);
  __syncthreads();
  for (int i = threadIdx.x; i < ROWS * kColsPerCta; i += kThreads) {
    const int r = i / kColsPerCta, cc = i % kColsPerCta;
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; wi++) s += red[((size_t)wi * ROWS + r) * kColsPerCta + cc];
    part[r][cc] = s;
  }
  cluster_sync_all();  // every CTA's partial is in its shared memory
  if (split == 0) {
    for (int i = threadIdx.x; i < ROWS * kColsPerCta; i += kThreads) {
      const int r = i / kColsPerCta, cc = i % kColsPerCta;
      if (r >= p.rows) continue;
      float s = part[r][cc];
#pragma unroll
      for (uint32_t q = 1; q < kDownSplit; q++) s += ld_peer_shared(&part[r][cc], q);
      __nv_bfloat16 y = __float2bfloat16_rn(s);  // the GEMM's bf16 output
      if (p.residual)
        y = __float2bfloat16_rn(__bfloat162float(p.residual[(size_t)r * n + col0 + cc]) + __bfloat162float(y));
      p.out[(size_t)r * n + col0 + cc] = y;
    }
  }
  cluster_sync_all();  // the peers' shared memory stays until the first CTA has read it
}

template <auto Kern>
cudaError_t launch_dyn(int ctas, int smem, const FfnParams& p, cudaStream_t st) {
  static bool configured[64] = {};  // per kernel (the template argument) and device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, Kern, p);
}

int ffail(int code, const char* msg) {
  pa::set_last_error(msg);
  return code;
}

}  // namespace

namespace pa {

// One layer's feed-forward block for `rows` <= 8 rows: two launches; pdl != 0 chains the first
// behind the kernel in front by programmatic dependent launch (the second always is).
int ffn_impl(const void* x, const void* norm_w, float eps, const void* wg, const void* wu, const void* wd,
             const void* residual, void* h, void* out, int rows, int hidden, int inter, int pdl, void* stream) {
  if (!x || !wg || !wu || !wd || !h || !out) return ffail(PA_ERR_INVALID_ARG, "pa_ffn: NULL argument");
  if (rows < 1 || rows > 8) return ffail(PA_ERR_UNSUPPORTED, "pa_ffn: 1 to 8 rows");
  if (hidden != kSlice || inter != kDownSplit * kSlice)
    return ffail(PA_ERR_UNSUPPORTED, "pa_ffn: built for hidden 2048 and intermediate 8192");
  cudaStream_t st = (cudaStream_t)stream;
  FfnParams a = {};
  a.x = (const __nv_bfloat16*)x;
  a.w0 = (const __nv_bfloat16*)wg;
  a.w1 = (const __nv_bfloat16*)wu;
  a.out = (__nv_bfloat16*)h;
  a.norm_w = (const __nv_bfloat16*)norm_w;
  a.rows = rows;
  a.k = hidden;
  a.n = inter;
  a.eps = eps;
  a.pdl = pdl;
  FfnParams b = {};
  b.x = (const __nv_bfloat16*)h;
  b.w0 = (const __nv_bfloat16*)wd;
  b.out = (__nv_bfloat16*)out;
  b.residual = (const __nv_bfloat16*)residual;
  b.rows = rows;
  b.k = inter;
  b.n = hidden;
  b.pdl = 1;
  const int ctas_a = inter / kColsPerCta, ctas_b = kDownSplit * (hidden / kColsPerCta);
  cudaError_t e;
  if (rows == 1) {
    e = launch_dyn<ffn_gate_up_mma_kernel<1>>(ctas_a, gate_up_smem<1>(), a, st);
    if (e == cudaSuccess) e = launch_dyn<ffn_down_mma_kernel<1>>(ctas_b, down_smem<1>(), b, st);
  } else if (rows == 2) {
    e = launch_dyn<ffn_gate_up_mma_kernel<2>>(ctas_a, gate_up_smem<2>(), a, st);
    if (e == cudaSuccess) e = launch_dyn<ffn_down_mma_kernel<2>>(ctas_b, down_smem<2>(), b, st);
  } else if (rows <= 4) {
    e = launch_dyn<ffn_gate_up_mma_kernel<4>>(ctas_a, gate_up_smem<4>(), a, st);
    if (e == cudaSuccess) e = launch_dyn<ffn_down_mma_kernel<4>>(ctas_b, down_smem<4>(), b, st);
  } else {
    e = launch_dyn<ffn_gate_up_mma_kernel<8>>(ctas_a, gate_up_smem<8>(), a, st);
    if (e == cudaSuccess) e = launch_dyn<ffn_down_mma_kernel<8>>(ctas_b, down_smem<8>(), b, st);
  }
  if (e != cudaSuccess) return ffail(PA_ERR_CUDA, cudaGetErrorString(e));
  return PA_OK;
}

}  // namespace pa

extern "C" {

int pa_ffn(const pa_ffn_weights* w, int layer, const void* x, void* h_scratch, void* out, int rows, int add_residual,
           void* stream) {
  if (!w) return ffail(PA_ERR_INVALID_ARG, "pa_ffn: NULL weights");
  if (layer < 0) return ffail(PA_ERR_INVALID_ARG, "pa_ffn: negative layer");
  const __nv_bfloat16* norm = w->ffn_norm ? (const __nv_bfloat16*)w->ffn_norm + (size_t)layer * w->norm_layer_stride : nullptr;
  const __nv_bfloat16* wg = w->gate ? (const __nv_bfloat16*)w->gate + (size_t)layer * w->gate_layer_stride : nullptr;
  const __nv_bfloat16* wu = w->up ? (const __nv_bfloat16*)w->up + (size_t)layer * w->up_layer_stride : nullptr;
  const __nv_bfloat16* wd = w->down ? (const __nv_bfloat16*)w->down + (size_t)layer * w->down_layer_stride : nullptr;
  return pa::ffn_impl(x, norm, w->rms_eps, wg, wu, wd, add_residual ? x : nullptr, h_scratch, out, rows, w->hidden,
                      w->inter, 0, stream);
}

}  // extern "C"
