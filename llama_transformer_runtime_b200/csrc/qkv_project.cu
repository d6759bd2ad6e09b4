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
// every weight row) of the concatenated [q | k | v] output and walks all K rows in
// steps of 128: warp w copies rows 16 w .. 16 w + 15 of a step into its own slot of
// a shared-memory ring with cp.async, the first steps before x is staged, and
// multiplies them on the tensor cores (mma_stream.cuh: mma.sync m16n8k16 on up to
// 8 rows of x, ldmatrix.trans for the weight blocks).  x sits in shared memory as
// bf16.  Partial sums are added over the 8 warps through shared memory in a fixed
// order, so the result does not depend on scheduling.
#include <cstdio>

#include "../../include/paged_attention.h"
#include "kernels.cuh"
#include "mma_stream.cuh"

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
  int* status = nullptr;       // packed kernel: a wait that ran out is recorded here (nullable: then only the loop ends)
  // optional residual of output 0 (the output projection): out = bf16(residual + bf16(x W)), same strides as out[0]
  const __nv_bfloat16* residual = nullptr;
  long long residual_layer_stride = 0;
  // optional RMSNorm in front of the projections: x <- bf16(x * rsqrt(mean(x^2) + eps) * norm_w)
  const __nv_bfloat16* norm_w = nullptr;  // [layers][hidden]
  long long norm_layer_stride = 0;
  float eps = 0.f;
  // launched with programmatic stream serialization: x (and the residual) come from the kernel in
  // front, the weights do not; see the two griddepcontrol points in the kernel
  int pdl = 0;
  // column tiles of the launch; a grid with fewer CTAs in x than this walks them in turn (x is staged
  // and normalised once per CTA, not once per tile); 0: one tile per CTA
  int total_tiles = 0;
};

// STAGES = 16 (one layer behind another kernel, launched with programmatic stream serialization): the
// ring holds the CTA's whole weight slab (2048 rows x 64 bytes = 128 KiB), copied while the kernel in
// front is still running, so that nothing is left to stream once x is there.  STAGES = 8: the
// streaming form for launches over many layers or column tiles, where several CTAs per SM keep the
// stream going (4, 6, 10 and 12 steps measured 1-4 % slower on the language-model head, 10 and 12
// 10-20 % slower on the 16-layer Q/K/V and output launches).  The arithmetic and its order are the same in both (the results are bit-equal).
template <int ROWS, int STAGES>
constexpr int rows_smem() { return STAGES * pa::kMmaStepBytes + ROWS * kMaxHidden * 2; }

template <int ROWS, int STAGES>
__global__ void __launch_bounds__(kThreads, STAGES == 16 ? 1 : 2) qkv_project_kernel(QkvParams p) {
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ float nscratch[16];
  auto sx = reinterpret_cast<__nv_bfloat16(*)[kMaxHidden]>(dyn + STAGES * pa::kMmaStepBytes);
  const int layer = blockIdx.y;
  const int n_tiles = p.total_tiles > 0 ? p.total_tiles : (int)gridDim.x;
  int t = blockIdx.x;
  int which = t < p.tiles_q ? 0 : (t < p.tiles_qk ? 1 : 2);
  int col0 = (t - (which == 0 ? 0 : (which == 1 ? p.tiles_q : p.tiles_qk))) * kColsPerCta;
  int n = p.n[which];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // the first weight copies go out before anything else: they do not depend on x
  pa::MmaStream<1, STAGES> st;
  st.w[0] = p.w[which] + (size_t)layer * p.w_layer_stride[which] + col0;
  st.n = (size_t)n;
  st.ring = pa::smem_u32(dyn);
  st.n_steps = (p.hidden + pa::kMmaStepRows - 1) / pa::kMmaStepRows;
  st.warp = warp;
  st.lane = lane;
  st.k_total = p.hidden;
  st.prologue();

  // The weight copies above are all this kernel may do before the kernel in front has finished:
  // x is its output.  The kernel behind may start its own weight copies from here on.
  // The norm weights do not depend on the kernel in front either: this thread's chunks of them are
  // loaded here (one chunk per thread at hidden = 2048), not after the wait behind x.
  // More than 2 rows of a hidden size that is a multiple of 256 (the model's): one warp per row side by
  // side (rmsnorm_row_by_warp), every lane with its 8 chunks of the norm weight; else the CTA-wide form
  // below, a chunk per thread.  Both give the reference kernel's bits.
  // (decided per instantiation: the kernels of 1 and 2 rows carry none of the other form's code)
  const bool norm_by_warp = ROWS >= 4 && p.hidden % 256 == 0;  // a warp alone needs 1 us longer for one row
  uint4 nw_pre[kMaxHidden / 8 / kThreads];
  uint4 nw8[ROWS >= 4 ? 8 : 1];
  if (p.norm_w) {
    const uint4* nwp = reinterpret_cast<const uint4*>(p.norm_w + (size_t)layer * p.norm_layer_stride);
    if constexpr (ROWS >= 4) {
      if (norm_by_warp) {
#pragma unroll
        for (int g = 0; g < 8; g++)
          if (g < p.hidden / 256) nw8[g] = __ldg(nwp + g * 32 + lane);
      }
    }
    if (!norm_by_warp) {
#pragma unroll
      for (int i = 0; i < kMaxHidden / 8 / kThreads; i++)
        if ((int)threadIdx.x + i * kThreads < p.hidden / 8) nw_pre[i] = __ldg(nwp + threadIdx.x + i * kThreads);
    }
  }
  if (p.pdl) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }

  // x rows of this layer -> shared memory (rows beyond p.rows and elements beyond hidden are zero)
  const __nv_bfloat16* x = p.x + (size_t)layer * p.x_layer_stride;
  for (int i = threadIdx.x; i < ROWS * (kMaxHidden / 8); i += kThreads) {
    const int r = i / (kMaxHidden / 8), ch = i % (kMaxHidden / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < p.rows && ch < p.hidden / 8) v = reinterpret_cast<const uint4*>(x + (size_t)r * p.hidden)[ch];
    reinterpret_cast<uint4*>(&sx[r][0])[ch] = v;
  }
  __syncthreads();
  if (p.norm_w && norm_by_warp) {
    if constexpr (ROWS >= 4) {
      if (warp < ROWS && warp < p.rows) pa::rmsnorm_row_by_warp(&sx[warp][0], nw8, p.hidden, p.eps, lane);
      __syncthreads();
    }
  } else if (p.norm_w) {
    // RMSNorm of the staged rows, in place, with the arithmetic AND the summation order of the
    // reference's kernel (src/kernels/rmsnorm/rmsnorm.cu:51-110, launched with 256 threads): a
    // thread sums the squares of its 8-element chunks in order, lanes combine by shuffle-down
    // (16, 8, 4, 2, 1), warp sums combine the same way in warp 0; y = bf16((x * r) * w).
#pragma unroll
    for (int r = 0; r < ROWS; r++) {
      if (r >= p.rows) break;  // uniform
      float sum_sq = 0.0f;
      for (int i = threadIdx.x; i < p.hidden / 8; i += kThreads) {
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
      if (lane == 0) nscratch[warp] = sum_sq;
      __syncthreads();
      float tot = lane < kThreads / 32 ? nscratch[lane] : 0.0f;
      if (warp == 0) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) tot += __shfl_down_sync(0xffffffffu, tot, off);
        if (lane == 0) nscratch[8] = tot;
      }
      __syncthreads();
      const float rms_recip = rsqrtf(nscratch[8] / static_cast<float>(p.hidden) + p.eps);
      for (int i = threadIdx.x, ii = 0; i < p.hidden / 8; i += kThreads, ii++) {
        const uint4 xd = reinterpret_cast<const uint4*>(&sx[r][0])[i];
        const uint4 wd = nw_pre[ii];
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
      __syncthreads();  // the scratch is reused by the next row; the last one publishes the rows
    }
  }

  for (;;) {
  float acc[1][4][4];
  st.template run<ROWS>(sx, acc);
  __syncthreads();  // every warp is done with the ring
  float* red = reinterpret_cast<float*>(dyn);
  pa::store_partials<1, ROWS>(red, acc, warp, lane);
  __syncthreads();
  // over the 8 warps, in warp order
  __nv_bfloat16* out = p.out[which] + (size_t)layer * p.out_layer_stride[which];
  for (int i = threadIdx.x; i < ROWS * kColsPerCta; i += kThreads) {
    const int r = i / kColsPerCta, cc = i % kColsPerCta;
    if (r >= p.rows) continue;
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; wi++) s += red[((size_t)wi * ROWS + r) * kColsPerCta + cc];
    __nv_bfloat16 y = __float2bfloat16_rn(s);  // the GEMM's bf16 output
    if (which == 0 && p.residual) {
      // the reference adds the residual in a second kernel on the bf16 GEMM output
      // (src/kernels/residual_add/residual_add.cu:14-38): fp32 sum of two bf16, rounded once
      const __nv_bfloat16 rv = p.residual[(size_t)layer * p.residual_layer_stride + (size_t)r * n + col0 + cc];
      y = __float2bfloat16_rn(__bfloat162float(rv) + __bfloat162float(y));
    }
    out[(size_t)r * n + col0 + cc] = y;
  }
  // the next column tile of this CTA (a launch of more tiles than CTAs): the staged rows stay
  t += gridDim.x;
  if (t >= n_tiles) break;
  which = t < p.tiles_q ? 0 : (t < p.tiles_qk ? 1 : 2);
  col0 = (t - (which == 0 ? 0 : (which == 1 ? p.tiles_q : p.tiles_qk))) * kColsPerCta;
  n = p.n[which];
  st.w[0] = p.w[which] + (size_t)layer * p.w_layer_stride[which] + col0;
  st.n = (size_t)n;
  __syncthreads();  // the partial sums in the ring have been read
  st.prologue();
  }
}

// ---- the same projections from PACKED weights (the tile images of pa_pack_projection_weights) --
// One weight format then serves decode and prefill, and the stream becomes 8 KiB contiguous
// bursts: a CTA owns one head (64 output columns) and pulls its 32 blocks (64 k-rows x 128 bytes,
// chunks XOR-swizzled) through an 8-stage ring with bulk (TMA) copies on mbarriers, as the decode
// attention kernel does; warp w takes rows 16w..16w+15 of every block, lane (rsub, c) the 16-byte
// chunk c of rows rsub + 4j.  Sums are reduced over lanes and warps in a fixed order.
constexpr int kPkStages = 8;
constexpr int kPkBlock = 64 * 128;  // 8 KiB
constexpr int kPkThreads = 128;

template <int ROWS>
__global__ void __launch_bounds__(kPkThreads) qkv_project_packed_kernel(QkvParams p) {
  extern __shared__ __align__(128) unsigned char pk_smem[];
  unsigned char* ring = pk_smem;
  __nv_bfloat16* sx = reinterpret_cast<__nv_bfloat16*>(pk_smem + kPkStages * kPkBlock);  // [ROWS][hidden]
  float* red = reinterpret_cast<float*>(pk_smem + kPkStages * kPkBlock + ROWS * kMaxHidden * 2);  // [4][ROWS][64]
  __shared__ __align__(8) unsigned long long bars[2 * kPkStages];
  const uint32_t bar_full = pa::smem_u32(bars), bar_empty = bar_full + 8 * kPkStages;
  const uint32_t ring_u32 = pa::smem_u32(ring);

  const int t = blockIdx.x, layer = blockIdx.y;
  const int hq = p.n[0] / 64, hkv = p.n[1] / 64;
  const int which = t < hq ? 0 : (t < hq + hkv ? 1 : 2);
  const int head = t - (which == 0 ? 0 : (which == 1 ? hq : hq + hkv));
  const int n = p.n[which];
  const char* w = reinterpret_cast<const char*>(p.w[which] + (size_t)layer * p.w_layer_stride[which]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_kb = p.hidden / 64;
  auto block_src = [&](int kb) { return w + ((size_t)kb * (n / 64) + head) * kPkBlock; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPkStages; s++) {
      pa::mbar_init(bar_full + 8 * s, 1);
      pa::mbar_init(bar_empty + 8 * s, kPkThreads / 32);
    }
    pa::mbar_fence_init();
    pa::fence_proxy_async_smem();
    for (int kb = 0; kb < kPkStages && kb < n_kb; kb++) {  // fill the ring: the copies do not depend on x
      pa::mbar_expect_tx(bar_full + 8 * kb, kPkBlock);
      pa::bulk_g2s(ring_u32 + kb * kPkBlock, block_src(kb), kPkBlock, bar_full + 8 * kb);
    }
  }
  const __nv_bfloat16* x = p.x + (size_t)layer * p.x_layer_stride;
  for (int i = threadIdx.x; i < ROWS * (p.hidden / 8); i += kPkThreads) {
    const int r = i / (p.hidden / 8), ch = i % (p.hidden / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < p.rows) v = reinterpret_cast<const uint4*>(x + (size_t)r * p.hidden)[ch];
    reinterpret_cast<uint4*>(sx + (size_t)r * kMaxHidden)[ch] = v;
  }
  __syncthreads();

  float acc[ROWS][8];
#pragma unroll
  for (int r = 0; r < ROWS; r++)
#pragma unroll
    for (int i = 0; i < 8; i++) acc[r][i] = 0.f;
  const int c = lane & 7, rsub = lane >> 3;
  bool ok = true;
  for (int kb = 0; kb < n_kb; kb++) {
    const int st = kb % kPkStages;
    if (!__all_sync(0xffffffffu, pa::mbar_wait(bar_full + 8 * st, (uint32_t)((kb / kPkStages) & 1)))) {
      ok = false;
      break;
    }
    const unsigned char* blk = ring + st * kPkBlock;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int r = warp * 16 + rsub + 4 * j;
      const uint4 wv = *reinterpret_cast<const uint4*>(blk + r * 128 + ((c ^ (r & 7)) << 4));
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
      float wf[8];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(h2[i]);
        wf[2 * i] = f.x;
        wf[2 * i + 1] = f.y;
      }
      const int k = kb * 64 + r;
#pragma unroll
      for (int rr = 0; rr < ROWS; rr++) {
        const float xv = __bfloat162float(sx[(size_t)rr * kMaxHidden + k]);
#pragma unroll
        for (int i = 0; i < 8; i++) acc[rr][i] = fmaf(xv, wf[i], acc[rr][i]);
      }
    }
    __syncwarp();
    if (lane == 0) pa::mbar_arrive(bar_empty + 8 * st);
    // the thread that owns the ring refills this stage once every warp has left it
    if (threadIdx.x == 0 && kb + kPkStages < n_kb) {
      if (!pa::mbar_wait(bar_empty + 8 * st, (uint32_t)((kb / kPkStages) & 1))) {
        ok = false;
      } else {
        pa::mbar_expect_tx(bar_full + 8 * st, kPkBlock);
        pa::bulk_g2s(ring_u32 + st * kPkBlock, block_src(kb + kPkStages), kPkBlock, bar_full + 8 * st);
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
  }
  if (!ok && lane == 0) atomicExch(p.status, pa::kStatusTimeout);
  // over the 4 row groups of the warp, then over the warps in warp order
#pragma unroll
  for (int r = 0; r < ROWS; r++)
#pragma unroll
    for (int i = 0; i < 8; i++) {
      float v = acc[r][i];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      acc[r][i] = v;
    }
  if (rsub == 0) {
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
      for (int i = 0; i < 8; i++) red[(warp * ROWS + r) * 64 + c * 8 + i] = acc[r][i];
  }
  __syncthreads();
  __nv_bfloat16* out = p.out[which] + (size_t)layer * p.out_layer_stride[which];
  for (int i = threadIdx.x; i < ROWS * 64; i += kPkThreads) {
    const int r = i / 64, cc = i % 64;
    if (r >= p.rows) continue;
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < kPkThreads / 32; wi++) s += red[(wi * ROWS + r) * 64 + cc];
    out[(size_t)r * n + head * 64 + cc] = __float2bfloat16_rn(s);
  }
}

template <int ROWS>
cudaError_t launch_packed(const QkvParams& p, int layers, cudaStream_t st) {
  const int smem = kPkStages * kPkBlock + ROWS * kMaxHidden * 2 + 4 * ROWS * 64 * 4;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(qkv_project_packed_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const dim3 grid((p.n[0] + 2 * p.n[1]) / 64, layers);
  qkv_project_packed_kernel<ROWS><<<grid, kPkThreads, smem, st>>>(p);
  return cudaGetLastError();
}

int qfail(int code, const char* msg) {
  pa::set_last_error(msg);
  return code;
}

// Launch of the row-major projection kernel for 1..8 rows, with programmatic stream serialization
// when p.pdl is set (the kernel then waits for the kernel in front before it reads x).
template <auto Kern>
cudaError_t launch_one(int smem, const QkvParams& p, dim3 grid, cudaStream_t st) {
  static bool configured[64] = {};  // per kernel (the template argument) and device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
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
template <int STAGES>
cudaError_t launch_stages(const QkvParams& p, dim3 grid, cudaStream_t st) {
  if (p.rows == 1) return launch_one<qkv_project_kernel<1, STAGES>>(rows_smem<1, STAGES>(), p, grid, st);
  if (p.rows == 2) return launch_one<qkv_project_kernel<2, STAGES>>(rows_smem<2, STAGES>(), p, grid, st);
  if (p.rows <= 4) return launch_one<qkv_project_kernel<4, STAGES>>(rows_smem<4, STAGES>(), p, grid, st);
  return launch_one<qkv_project_kernel<8, STAGES>>(rows_smem<8, STAGES>(), p, grid, st);
}
cudaError_t launch_rows(const QkvParams& p, dim3 grid, cudaStream_t st) {
  // one layer behind another kernel: the form that holds its weight slab in shared memory
  // (a grid of many waves, the language-model head, streams: its CTAs overlap one another)
  const bool resident = p.pdl && grid.y == 1 && p.hidden <= kMaxHidden && grid.x <= 512;
  if (resident) return launch_stages<16>(p, grid, st);
  // many waves of column tiles (the language-model head): as many CTAs as are resident at once walk
  // the tiles, so that x is staged and normalised once per CTA (with 8 rows that prologue took
  // longer than a tile's stream: 190 us for the head against 87 us with one row; with one row the
  // walk is 3 us slower than a CTA per tile, whose successors start while it drains)
  if (grid.y == 1 && grid.x > 1024 && p.rows > 2) {
    QkvParams q = p;
    q.total_tiles = (int)grid.x;
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int per_sm = p.rows <= 4 ? 3 : 2;  // what shared memory admits (64 KiB of ring + the staged rows)
    return launch_stages<8>(q, dim3(sms * per_sm, 1), st);
  }
  return launch_stages<8>(p, grid, st);
}

}  // namespace

namespace pa {
int out_project_impl(const void* attn, const void* wo, const void* residual, void* out, int rows, int layers,
                     int hidden, int cols, int64_t attn_layer_stride, int64_t wo_layer_stride,
                     int64_t residual_layer_stride, int64_t out_layer_stride, int pdl, void* stream);

int qkv_project_impl(const void* x, const void* norm_weight, int64_t norm_layer_stride, float eps, const void* wq,
                     const void* wk, const void* wv, void* q, void* k, void* v, int rows, int layers, int hidden,
                     int q_cols, int kv_cols, int64_t x_layer_stride, int64_t wq_layer_stride,
                     int64_t wkv_layer_stride, int64_t q_layer_stride, int64_t kv_layer_stride, int pdl,
                     void* stream) {
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
  p.norm_w = (const __nv_bfloat16*)norm_weight;
  p.norm_layer_stride = norm_layer_stride;
  p.eps = eps;
  p.pdl = pdl;
  const dim3 grid(p.tiles_qk + kv_cols / kColsPerCta, layers);
  const cudaError_t e = launch_rows(p, grid, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "pa_qkv_project: %s", cudaGetErrorString(e));
    return qfail(PA_ERR_CUDA, msg);
  }
  return PA_OK;
}
}  // namespace pa

extern "C" int pa_qkv_project(const void* x, const void* wq, const void* wk, const void* wv, void* q, void* k,
                              void* v, int rows, int layers, int hidden, int q_cols, int kv_cols,
                              int64_t x_layer_stride, int64_t wq_layer_stride, int64_t wkv_layer_stride,
                              int64_t q_layer_stride, int64_t kv_layer_stride, void* stream) {
  return pa::qkv_project_impl(x, nullptr, 0, 0.f, wq, wk, wv, q, k, v, rows, layers, hidden, q_cols, kv_cols,
                              x_layer_stride, wq_layer_stride, wkv_layer_stride, q_layer_stride, kv_layer_stride, 0,
                              stream);
}

extern "C" int pa_rmsnorm_qkv_project(const void* x, const void* norm_weight, int64_t norm_layer_stride, float eps,
                                      const void* wq, const void* wk, const void* wv, void* q, void* k, void* v,
                                      int rows, int layers, int hidden, int q_cols, int kv_cols,
                                      int64_t x_layer_stride, int64_t wq_layer_stride, int64_t wkv_layer_stride,
                                      int64_t q_layer_stride, int64_t kv_layer_stride, void* stream) {
  if (!norm_weight) return qfail(PA_ERR_INVALID_ARG, "pa_rmsnorm_qkv_project: NULL norm weight");
  return pa::qkv_project_impl(x, norm_weight, norm_layer_stride, eps, wq, wk, wv, q, k, v, rows, layers, hidden,
                              q_cols, kv_cols, x_layer_stride, wq_layer_stride, wkv_layer_stride, q_layer_stride,
                              kv_layer_stride, 0, stream);
}

extern "C" int pa_qkv_project_packed(const void* x, const void* wq_packed, const void* wk_packed,
                                     const void* wv_packed, void* q, void* k, void* v, int rows, int layers,
                                     int hidden, int q_cols, int kv_cols, int64_t x_layer_stride,
                                     int64_t wq_layer_stride, int64_t wkv_layer_stride, int64_t q_layer_stride,
                                     int64_t kv_layer_stride, int* status_word, void* stream) {
  if (!x || !wq_packed || !wk_packed || !wv_packed || !q || !k || !v || !status_word)
    return qfail(PA_ERR_INVALID_ARG, "pa_qkv_project_packed: NULL argument");
  if (rows < 1 || layers < 1 || layers > 65535) return qfail(PA_ERR_INVALID_ARG, "pa_qkv_project_packed: rows >= 1, 1 <= layers <= 65535");
  if (rows > 8) return qfail(PA_ERR_UNSUPPORTED, "pa_qkv_project_packed: at most 8 rows per call (decode shapes)");
  if (hidden < 64 || hidden > kMaxHidden || hidden % 64 != 0)
    return qfail(PA_ERR_UNSUPPORTED, "pa_qkv_project_packed: hidden must be a multiple of 64, at most 2048");
  if (q_cols < 64 || kv_cols < 64 || q_cols % 64 != 0 || kv_cols % 64 != 0)
    return qfail(PA_ERR_UNSUPPORTED, "pa_qkv_project_packed: q_cols and kv_cols must be multiples of 64");
  QkvParams p;
  p.x = (const __nv_bfloat16*)x;
  p.w[0] = (const __nv_bfloat16*)wq_packed;
  p.w[1] = (const __nv_bfloat16*)wk_packed;
  p.w[2] = (const __nv_bfloat16*)wv_packed;
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
  p.tiles_q = p.tiles_qk = 0;
  p.rows = rows;
  p.hidden = hidden;
  p.status = status_word;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (rows == 1)
    e = launch_packed<1>(p, layers, st);
  else if (rows == 2)
    e = launch_packed<2>(p, layers, st);
  else if (rows <= 4)
    e = launch_packed<4>(p, layers, st);
  else
    e = launch_packed<8>(p, layers, st);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "pa_qkv_project_packed: %s", cudaGetErrorString(e));
    return qfail(PA_ERR_CUDA, msg);
  }
  return PA_OK;
}

// Output projection of a decode step with the attention residual folded in: out = bf16(residual +
// bf16(attn W_o)).  Replaces launch_gemm_2048x2048 (src/runtime/attention.cu:367-375) and
// transformer::residual_add (src/runtime/transformer_block.cu:76-81) for decode shapes.
extern "C" int pa_out_project(const void* attn, const void* wo, const void* residual, void* out, int rows,
                              int layers, int hidden, int cols, int64_t attn_layer_stride,
                              int64_t wo_layer_stride, int64_t out_layer_stride, void* stream) {
  return pa::out_project_impl(attn, wo, residual, out, rows, layers, hidden, cols, attn_layer_stride, wo_layer_stride,
                              out_layer_stride, out_layer_stride, 0, stream);
}

int pa::out_project_impl(const void* attn, const void* wo, const void* residual, void* out, int rows, int layers,
                         int hidden, int cols, int64_t attn_layer_stride, int64_t wo_layer_stride,
                         int64_t residual_layer_stride, int64_t out_layer_stride, int pdl, void* stream) {
  if (!attn || !wo || !out) return qfail(PA_ERR_INVALID_ARG, "pa_out_project: NULL argument");
  if (rows < 1 || layers < 1 || layers > 65535) return qfail(PA_ERR_INVALID_ARG, "pa_out_project: rows >= 1, 1 <= layers <= 65535");
  if (rows > 8) return qfail(PA_ERR_UNSUPPORTED, "pa_out_project: at most 8 rows per call (decode shapes)");
  if (hidden < 64 || hidden > kMaxHidden || hidden % 64 != 0)
    return qfail(PA_ERR_UNSUPPORTED, "pa_out_project: hidden must be a multiple of 64, at most 2048");
  if (cols < kColsPerCta || cols % kColsPerCta != 0) return qfail(PA_ERR_UNSUPPORTED, "pa_out_project: cols must be a multiple of 32");
  QkvParams p;
  p.x = (const __nv_bfloat16*)attn;
  p.w[0] = p.w[1] = p.w[2] = (const __nv_bfloat16*)wo;
  p.out[0] = p.out[1] = p.out[2] = (__nv_bfloat16*)out;
  p.x_layer_stride = attn_layer_stride;
  p.w_layer_stride[0] = p.w_layer_stride[1] = p.w_layer_stride[2] = wo_layer_stride;
  p.out_layer_stride[0] = p.out_layer_stride[1] = p.out_layer_stride[2] = out_layer_stride;
  p.n[0] = p.n[1] = p.n[2] = cols;
  p.tiles_q = p.tiles_qk = cols / kColsPerCta;  // every tile belongs to output 0
  p.rows = rows;
  p.hidden = hidden;
  p.residual = (const __nv_bfloat16*)residual;
  p.residual_layer_stride = residual_layer_stride;
  p.pdl = pdl;
  const dim3 grid(p.tiles_q, layers);
  const cudaError_t e = launch_rows(p, grid, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "pa_out_project: %s", cudaGetErrorString(e));
    return qfail(PA_ERR_CUDA, msg);
  }
  return PA_OK;
}

// The language-model head of a decode step: logits = RMSNorm(x, final_norm) W_lm, bf16, as the
// reference computes them with rmsnorm_launch<2048> and launch_gemm_2048x128256
// (src/runtime/llama_runtime.cu:880-905; the weight [hidden, vocab] row-major).  The same
// weight-streaming kernel as the projections: 525 MB per token for the 128256-entry vocabulary,
// 4008 column tiles of 32.
namespace pa {
int lm_head_impl(const void* x, const void* final_norm, float eps, const void* w_lm, void* logits, int rows, int hidden,
                 int vocab, int pdl, void* stream) {
  if (!x || !w_lm || !logits) return qfail(PA_ERR_INVALID_ARG, "pa_lm_head: NULL argument");
  if (rows < 1) return qfail(PA_ERR_INVALID_ARG, "pa_lm_head: rows must be >= 1");
  if (rows > 8) return qfail(PA_ERR_UNSUPPORTED, "pa_lm_head: at most 8 rows per call (decode shapes)");
  if (hidden < 64 || hidden > kMaxHidden || hidden % 64 != 0)
    return qfail(PA_ERR_UNSUPPORTED, "pa_lm_head: hidden must be a multiple of 64, at most 2048");
  if (vocab < kColsPerCta || vocab % kColsPerCta != 0) return qfail(PA_ERR_UNSUPPORTED, "pa_lm_head: vocab must be a multiple of 32");
  QkvParams p;
  p.x = (const __nv_bfloat16*)x;
  p.w[0] = p.w[1] = p.w[2] = (const __nv_bfloat16*)w_lm;
  p.out[0] = p.out[1] = p.out[2] = (__nv_bfloat16*)logits;
  p.x_layer_stride = 0;
  p.w_layer_stride[0] = p.w_layer_stride[1] = p.w_layer_stride[2] = 0;
  p.out_layer_stride[0] = p.out_layer_stride[1] = p.out_layer_stride[2] = 0;
  p.n[0] = p.n[1] = p.n[2] = vocab;
  p.tiles_q = p.tiles_qk = vocab / kColsPerCta;  // every tile belongs to output 0
  p.rows = rows;
  p.hidden = hidden;
  p.norm_w = (const __nv_bfloat16*)final_norm;
  p.norm_layer_stride = 0;
  p.eps = eps;
  p.pdl = pdl;
  const dim3 grid(p.tiles_q, 1);
  const cudaError_t e = launch_rows(p, grid, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "pa_lm_head: %s", cudaGetErrorString(e));
    return qfail(PA_ERR_CUDA, msg);
  }
  return PA_OK;
}
}  // namespace pa

extern "C" int pa_lm_head(const void* x, const void* final_norm, float eps, const void* w_lm, void* logits, int rows,
                          int hidden, int vocab, void* stream) {
  return pa::lm_head_impl(x, final_norm, eps, w_lm, logits, rows, hidden, vocab, 0, stream);
}
