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
// ffn_gate_up_kernel: a CTA owns 32 adjacent columns of BOTH Wg and Wu and walks all rows: warp
// w, lane (kr, c) reads the 16-byte chunk c of rows 64 j + 8 w + kr of each matrix, a rolling window
// of 8 + 8 independent loads in flight per thread, the first of them issued before x is staged.
// ffn_down_kernel: a cluster of four CTAs owns 32 adjacent columns of Wd; CTA s of the cluster walks
// rows [s K/4, (s+1) K/4) (64 column tiles alone would leave half of the SMs idle); the four partial
// sums are added in rank order by the cluster's first CTA, which reads its peers' shared memory, so
// the result does not depend on scheduling.
#include <cstdio>
#include <cstdlib>

#include "../../include/paged_attention.h"
#include "kernels.cuh"

namespace pa {
void set_last_error(const char* msg);
}

namespace {

constexpr int kColsPerCta = 32;
constexpr int kThreads = 256;
constexpr int kSlice = 2048;   // rows of a weight matrix one CTA walks = elements of x it stages
constexpr int kDownSplit = 4;  // CTAs of a cluster of the down projection
constexpr int kRowGroup = 4;   // rows one CTA carries; more rows form a second group of CTAs

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

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 t = __bfloat1622float2(h2[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// h[r][col] = bf16(silu(bf16(x_r . Wg[:, col])) * bf16(x_r . Wu[:, col])), x normalised first.
// Rows beyond the first kRowGroup are a second group of CTAs (blockIdx.y = 1): with more than 4 rows per
// thread the accumulators alone push the kernel to one CTA per SM and 256 CTAs into two waves; the
// second group's weight reads hit L2 behind the first's.
template <int ROWS, int WIN>
__global__ void __launch_bounds__(kThreads, 2) ffn_gate_up_kernel(FfnParams p) {
  __shared__ __align__(16) __nv_bfloat16 sx[ROWS][kSlice];
  __shared__ float red[8][ROWS][2][kColsPerCta];
  p.x += (size_t)blockIdx.y * kRowGroup * p.k;
  p.out += (size_t)blockIdx.y * kRowGroup * p.n;
  p.rows = min(p.rows - (int)blockIdx.y * kRowGroup, kRowGroup);
  const int col0 = blockIdx.x * kColsPerCta;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kr = lane >> 2, c = lane & 3;
  const int n = p.n;

  // the first weight loads go out before anything else: they do not depend on x
  const size_t first = (size_t)(warp * 8 + kr) * n + col0;
  const uint4* gp = reinterpret_cast<const uint4*>(p.w0 + first) + c;
  const uint4* up = reinterpret_cast<const uint4*>(p.w1 + first) + c;
  const size_t step = (size_t)64 * n / 8;  // 64 rows further, in 16-byte units
  const int n_steps = p.k / 64;
  constexpr int kWin = WIN;
  uint4 gv[kWin], uv[kWin];
#pragma unroll
  for (int u = 0; u < kWin; u++)
    if (u < n_steps) {
      gv[u] = __ldg(gp + (size_t)u * step);
      uv[u] = __ldg(up + (size_t)u * step);
    }
  // x comes from the kernel in front, the weights do not.  (Asking the rest of the weight rows into
  // L2 here, as the small projection kernels do, made this block slower — 26.7 against 24.8 us per
  // layer: its 100 MB are bound by DRAM bandwidth, which the prefetches only take from the kernel
  // in front.)
  if (p.pdl) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  stage_rows<ROWS>(sx, p.x, (size_t)p.k, p.rows, p.k);
  __syncthreads();
  if (p.norm_w) rmsnorm_rows<ROWS>(sx, p.norm_w, p.rows, p.k, p.eps, &red[0][0][0][0]);

  float ag[ROWS][8], au[ROWS][8];
#pragma unroll
  for (int r = 0; r < ROWS; r++)
#pragma unroll
    for (int i = 0; i < 8; i++) ag[r][i] = au[r][i] = 0.f;

  for (int j0 = 0; j0 < n_steps; j0 += kWin) {
#pragma unroll
    for (int u = 0; u < kWin; u++) {
      if (j0 + u >= n_steps) break;
      const int k = (j0 + u) * 64 + warp * 8 + kr;
      float gf[8], uf[8];
      unpack8(gv[u], gf);
      unpack8(uv[u], uf);
      if (j0 + u + kWin < n_steps) {
        gv[u] = __ldg(gp + (size_t)(j0 + u + kWin) * step);
        uv[u] = __ldg(up + (size_t)(j0 + u + kWin) * step);
      }
#pragma unroll
      for (int r = 0; r < ROWS; r++) {
        const float xv = __bfloat162float(sx[r][k]);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          ag[r][i] = fmaf(xv, gf[i], ag[r][i]);
          au[r][i] = fmaf(xv, uf[i], au[r][i]);
        }
      }
    }
  }
  // over the 8 row lanes of the warp
#pragma unroll
  for (int r = 0; r < ROWS; r++)
#pragma unroll
    for (int i = 0; i < 8; i++) {
      float a = ag[r][i], b = au[r][i];
      a += __shfl_xor_sync(0xffffffffu, a, 4);
      b += __shfl_xor_sync(0xffffffffu, b, 4);
      a += __shfl_xor_sync(0xffffffffu, a, 8);
      b += __shfl_xor_sync(0xffffffffu, b, 8);
      a += __shfl_xor_sync(0xffffffffu, a, 16);
      b += __shfl_xor_sync(0xffffffffu, b, 16);
      ag[r][i] = a;
      au[r][i] = b;
    }
  __syncthreads();  // red doubles as the RMSNorm scratch
  if (kr == 0) {
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
      for (int i = 0; i < 8; i++) {
        red[warp][r][0][c * 8 + i] = ag[r][i];
        red[warp][r][1][c * 8 + i] = au[r][i];
      }
  }
  __syncthreads();
  // over the 8 warps, in warp order; then SiLU(gate) * up on the two bf16 GEMM outputs
  for (int i = threadIdx.x; i < ROWS * kColsPerCta; i += kThreads) {
    const int r = i / kColsPerCta, cc = i % kColsPerCta;
    if (r >= p.rows) continue;
    float sg = 0.f, su = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; wi++) {
      sg += red[wi][r][0][cc];
      su += red[wi][r][1][cc];
    }
    const float g = __bfloat162float(__float2bfloat16_rn(sg));
    const float u = __bfloat162float(__float2bfloat16_rn(su));
    const float s = __fmul_rn(g, 1.0f / (1.0f + __expf(-g)));
    p.out[(size_t)r * n + col0 + cc] = __float2bfloat16_rn(__fmul_rn(s, u));
  }
}

// out[r][col] = bf16(residual + bf16(h_r . Wd[:, col])), K split over the four CTAs of a cluster.
template <int ROWS>
__global__ void __cluster_dims__(kDownSplit, 1, 1) __launch_bounds__(kThreads, 2) ffn_down_kernel(FfnParams p) {
  __shared__ __align__(16) __nv_bfloat16 sx[ROWS][kSlice];
  __shared__ float red[8][ROWS][kColsPerCta];
  __shared__ float part[ROWS][kColsPerCta];
  p.x += (size_t)blockIdx.y * kRowGroup * p.k;
  p.out += (size_t)blockIdx.y * kRowGroup * p.n;
  if (p.residual) p.residual += (size_t)blockIdx.y * kRowGroup * p.n;
  p.rows = min(p.rows - (int)blockIdx.y * kRowGroup, kRowGroup);
  const uint32_t split = cluster_ctarank();
  const int col0 = (int)(blockIdx.x / kDownSplit) * kColsPerCta;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kr = lane >> 2, c = lane & 3;
  const int n = p.n;
  const int k_slice = p.k / kDownSplit;  // rows of Wd this CTA walks
  const int k0 = (int)split * k_slice;

  const uint4* wp = reinterpret_cast<const uint4*>(p.w0 + (size_t)(k0 + warp * 8 + kr) * n + col0) + c;
  const size_t step = (size_t)64 * n / 8;
  const int n_steps = k_slice / 64;
  constexpr int kWin = 16;
  uint4 wv[kWin];
#pragma unroll
  for (int u = 0; u < kWin; u++)
    if (u < n_steps) wv[u] = __ldg(wp + (size_t)u * step);
  if (p.pdl) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  stage_rows<ROWS>(sx, p.x + k0, (size_t)p.k, p.rows, k_slice);
  __syncthreads();

  float acc[ROWS][8];
#pragma unroll
  for (int r = 0; r < ROWS; r++)
#pragma unroll
    for (int i = 0; i < 8; i++) acc[r][i] = 0.f;
  for (int j0 = 0; j0 < n_steps; j0 += kWin) {
#pragma unroll
    for (int u = 0; u < kWin; u++) {
      if (j0 + u >= n_steps) break;
      const int k = (j0 + u) * 64 + warp * 8 + kr;
      float wf[8];
      unpack8(wv[u], wf);
      if (j0 + u + kWin < n_steps) wv[u] = __ldg(wp + (size_t)(j0 + u + kWin) * step);
#pragma unroll
      for (int r = 0; r < ROWS; r++) {
        const float xv = __bfloat162float(sx[r][k]);
#pragma unroll
        for (int i = 0; i < 8; i++) acc[r][i] = fmaf(xv, wf[i], acc[r][i]);
      }
    }
  }
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
  for (int i = threadIdx.x; i < ROWS * kColsPerCta; i += kThreads) {
    const int r = i / kColsPerCta, cc = i % kColsPerCta;
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; wi++) s += red[wi][r][cc];
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

// ---- the same two kernels on the tensor cores ---------------------------------------------------
// With fused multiply-adds a thread spends about 50 instructions on every 16 bytes of weights
// (unpacking, 8 x rows multiply-adds, addresses), and the stream slows down with every row: 25, 27.5,
// 35 and 60 us per layer for 1, 2, 4 and 8 rows.  Here a warp copies its 16 weight rows of a step
// (64 bytes each, per matrix) into its own slot of a shared-memory ring with cp.async — no registers
// held by loads in flight, no CTA-wide barrier in the loop — and multiplies them with
// mma.sync.m16n8k16: A = the step's x values of up to 8 rows (rows 8..15 of the tile are zero), B =
// the 16 x 8 weight blocks fetched with ldmatrix.trans (16-byte chunks XOR-swizzled by row pair, so
// that the 8 rows of a matrix fetch hit 8 different bank groups), fp32 accumulators.  Two ldmatrix.x4
// and four MMAs per matrix and step replace 2 x 50 instructions per lane.  Sums over the 8 warps in
// warp order, so results do not depend on scheduling; they differ from the multiply-add form in
// the order of the fp32 additions inside a warp's 16 rows.
constexpr int kMmaStepRows = 128;            // weight rows per step: 16 per warp
constexpr int kMmaWarpTile = 16 * 64;        // a warp's rows of one matrix in one step: 1 KiB
constexpr int kMmaStepBytes = 8 * kMmaWarpTile;  // one matrix, one step: 8 KiB

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&d)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(addr));
}
// c += A B with A's rows 8..15 zero: a0 = (row lane/4, k 2(lane%4), +1), a2 = the same row at k + 8
__device__ __forceinline__ void mma_rows8(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// The stream of NM matrices (1: down, 2: gate and up) over `n_steps` steps of 128 rows starting at row
// k_first, columns col0 .. col0 + 31, against the rows staged in sx: acc[m][ng] = this warp's partial
// sums (its 16 rows of every step) for the 8 columns of group ng, rows lane / 4.
template <int NM, int STAGES>
struct MmaStream {
  const __nv_bfloat16* w[NM];
  size_t n;        // row pitch of the matrices in elements
  uint32_t ring;   // shared-memory address of STAGES x NM x 8 KiB
  int n_steps, warp, lane;

  __device__ __forceinline__ void issue(int j) const {
    if (j < n_steps) {
      const int slot = j % STAGES;
#pragma unroll
      for (int m = 0; m < NM; m++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int q = lane + 32 * h, r = q >> 2, c = q & 3;
          cp_async16(ring + (slot * NM + m) * kMmaStepBytes + warp * kMmaWarpTile + r * 64 + ((c ^ ((r >> 1) & 3)) << 4),
                     w[m] + (size_t)(j * kMmaStepRows + warp * 16 + r) * n + c * 8);
        }
    }
    cp_async_commit();  // an empty group past the end keeps the count of groups in flight uniform
  }
  __device__ __forceinline__ void prologue() const {
#pragma unroll
    for (int j = 0; j < STAGES; j++) issue(j);
  }
  template <int ROWS>
  __device__ __forceinline__ void run(const __nv_bfloat16 (*sx)[kSlice], float (&acc)[NM][4][4]) const {
#pragma unroll
    for (int m = 0; m < NM; m++)
#pragma unroll
      for (int g = 0; g < 4; g++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[m][g][i] = 0.f;
    const int row = lane >> 2;
    const int lr = (lane & 7) + ((lane >> 3) & 1) * 8;  // the row of the 16 x 64-byte tile whose address this lane gives
    const uint32_t lm_off = lr * 64, lm_sw = (lr >> 1) & 3, lm_chunk = lane >> 4;
    for (int j = 0; j < n_steps; j++) {
      cp_async_wait<STAGES - 1>();
      __syncwarp();
      const int kbase = j * kMmaStepRows + warp * 16 + 2 * (lane & 3);
      uint32_t a0 = 0, a2 = 0;
      if (row < ROWS) {
        a0 = *reinterpret_cast<const uint32_t*>(&sx[row][kbase]);
        a2 = *reinterpret_cast<const uint32_t*>(&sx[row][kbase + 8]);
      }
      const int slot = j % STAGES;
#pragma unroll
      for (int m = 0; m < NM; m++) {
        const uint32_t tile = ring + (slot * NM + m) * kMmaStepBytes + warp * kMmaWarpTile + lm_off;
#pragma unroll
        for (int g0 = 0; g0 < 4; g0 += 2) {
          uint32_t d[4];
          ldmatrix_x4_trans(tile + (((g0 + lm_chunk) ^ lm_sw) << 4), d);
          mma_rows8(acc[m][g0], a0, a2, d[0], d[1]);
          mma_rows8(acc[m][g0 + 1], a0, a2, d[2], d[3]);
        }
      }
      __syncwarp();  // every lane has read the slot
      issue(j + STAGES);
    }
    cp_async_wait<0>();
  }
};

// Partial sums of the 8 warps -> red[warp][row][m][col] (red may lie in the ring: the stream is over).
template <int NM, int ROWS>
__device__ __forceinline__ void store_partials(float* red, const float (&acc)[NM][4][4], int warp, int lane) {
  const int row = lane >> 2, cq = 2 * (lane & 3);
  if (row < ROWS) {
#pragma unroll
    for (int m = 0; m < NM; m++)
#pragma unroll
      for (int g = 0; g < 4; g++) {
        float* at = red + (((size_t)warp * ROWS + row) * NM + m) * kColsPerCta + g * 8 + cq;
        at[0] = acc[m][g][0];
        at[1] = acc[m][g][1];
      }
  }
}

constexpr int kGateUpStages = 5, kDownStages = 8;
template <int ROWS>
constexpr int gate_up_smem() { return kGateUpStages * 2 * kMmaStepBytes + ROWS * kSlice * 2; }
template <int ROWS>
constexpr int down_smem() { return kDownStages * kMmaStepBytes + ROWS * kSlice * 2; }

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
  st.prologue();  // the weights do not depend on the kernel in front; x does
  if (p.pdl) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  stage_rows<ROWS>(sx, p.x, (size_t)p.k, p.rows, p.k);
  __syncthreads();
  if (p.norm_w) rmsnorm_rows<ROWS>(sx, p.norm_w, p.rows, p.k, p.eps, nscratch);
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
  auto sx = reinterpret_cast<__nv_bfloat16(*)[kSlice]>(dyn + kDownStages * kMmaStepBytes);
  const uint32_t split = cluster_ctarank();
  const int col0 = (int)(blockIdx.x / kDownSplit) * kColsPerCta;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = p.n;
  const int k_slice = p.k / kDownSplit;  // rows of Wd this CTA walks
  const int k0 = (int)split * k_slice;
  MmaStream<1, kDownStages> st;
  st.w[0] = p.w0 + (size_t)k0 * n + col0;
  st.n = (size_t)n;
  st.ring = pa::smem_u32(dyn);
  st.n_steps = k_slice / kMmaStepRows;
  st.warp = warp;
  st.lane = lane;
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

template <typename K>
cudaError_t launch_dyn(K kern, int ctas, int smem, const FfnParams& p, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
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
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <typename K>
cudaError_t launch(K kern, int ctas, int groups, const FfnParams& p, cudaStream_t st) {
  if (!p.pdl) {
    kern<<<dim3(ctas, groups), kThreads, 0, st>>>(p);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas, groups);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
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
  static const bool fma_form = getenv("PA_FFN_FMA") != nullptr;
  const int groups = (rows + kRowGroup - 1) / kRowGroup;
  if (!fma_form) {
    if (rows == 1) {
      e = launch_dyn(ffn_gate_up_mma_kernel<1>, ctas_a, gate_up_smem<1>(), a, st);
      if (e == cudaSuccess) e = launch_dyn(ffn_down_mma_kernel<1>, ctas_b, down_smem<1>(), b, st);
    } else if (rows == 2) {
      e = launch_dyn(ffn_gate_up_mma_kernel<2>, ctas_a, gate_up_smem<2>(), a, st);
      if (e == cudaSuccess) e = launch_dyn(ffn_down_mma_kernel<2>, ctas_b, down_smem<2>(), b, st);
    } else if (rows <= 4) {
      e = launch_dyn(ffn_gate_up_mma_kernel<4>, ctas_a, gate_up_smem<4>(), a, st);
      if (e == cudaSuccess) e = launch_dyn(ffn_down_mma_kernel<4>, ctas_b, down_smem<4>(), b, st);
    } else {
      e = launch_dyn(ffn_gate_up_mma_kernel<8>, ctas_a, gate_up_smem<8>(), a, st);
      if (e == cudaSuccess) e = launch_dyn(ffn_down_mma_kernel<8>, ctas_b, down_smem<8>(), b, st);
    }
  } else
  if (rows == 1) {
    e = launch(ffn_gate_up_kernel<1, 8>, ctas_a, 1, a, st);
    if (e == cudaSuccess) e = launch(ffn_down_kernel<1>, ctas_b, 1, b, st);
  } else if (rows == 2) {
    e = launch(ffn_gate_up_kernel<2, 8>, ctas_a, 1, a, st);
    if (e == cudaSuccess) e = launch(ffn_down_kernel<2>, ctas_b, 1, b, st);
  } else {
    e = launch(ffn_gate_up_kernel<4, 4>, ctas_a, groups, a, st);
    if (e == cudaSuccess) e = launch(ffn_down_kernel<4>, ctas_b, groups, b, st);
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
