// The weight stream of the decode-shape projections on the tensor cores, shared by the feed-forward
// kernels (ffn.cu) and the Q/K/V, output and language-model-head projections (qkv_project.cu).
#pragma once
#include "pa_common.cuh"

namespace pa {

constexpr int kStreamThreads = 256;    // 8 warps
constexpr int kStreamCols = 32;        // output columns per CTA: 64 bytes of every weight row
constexpr int kStreamRowLen = 2048;    // elements of a staged x row (the most a CTA walks)

// ---- the weight stream on the tensor cores ------------------------------------------------------
// With fused multiply-adds from a rolling window of 16-byte loads a thread spent about 50 instructions
// on every 16 bytes of weights (unpacking, 8 x rows multiply-adds, addresses), and the stream slowed
// down with every row: 25, 27.5, 35 and 60 us per layer for 1, 2, 4 and 8 rows (24.5, 24.9, 26.7 and
// 31.9 now).  Here a warp copies its 16 weight rows of a step
// (64 bytes each, per matrix) into its own slot of a shared-memory ring with cp.async — no registers
// held by loads in flight, no CTA-wide barrier in the loop — and multiplies them with
// mma.sync.m16n8k16: A = the step's x values of up to 8 rows (rows 8..15 of the tile are zero), B =
// the 16 x 8 weight blocks fetched with ldmatrix.trans (16-byte chunks XOR-swizzled by row pair, so
// that the 8 rows of a matrix fetch hit 8 different bank groups), fp32 accumulators.  Two ldmatrix.x4
// and four MMAs per matrix and step replace 2 x 50 instructions per lane.  Sums over the 8 warps in
// warp order, so results do not depend on scheduling.
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
  int k_total;     // weight rows that exist (a last step may be partly past the end: those tile rows are zeros)

  __device__ __forceinline__ void issue(int j) const {
    if (j < n_steps) {
      const int slot = j % STAGES;
#pragma unroll
      for (int m = 0; m < NM; m++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int q = lane + 32 * h, r = q >> 2, c = q & 3;
          const uint32_t dst = ring + (slot * NM + m) * kMmaStepBytes + warp * kMmaWarpTile + r * 64 + ((c ^ ((r >> 1) & 3)) << 4);
          const int k = j * kMmaStepRows + warp * 16 + r;
          if (k < k_total)
            cp_async16(dst, w[m] + (size_t)k * n + c * 8);
          else
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
        }
    }
    cp_async_commit();  // an empty group past the end keeps the count of groups in flight uniform
  }
  __device__ __forceinline__ void prologue() const {
#pragma unroll
    for (int j = 0; j < STAGES; j++) issue(j);
  }
  template <int ROWS>
  __device__ __forceinline__ void run(const __nv_bfloat16 (*sx)[kStreamRowLen], float (&acc)[NM][4][4]) const {
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
        float* at = red + (((size_t)warp * ROWS + row) * NM + m) * kStreamCols + g * 8 + cq;
        at[0] = acc[m][g][0];
        at[1] = acc[m][g][1];
      }
  }
}

// RMSNorm of one staged row by ONE warp, in place: y = bf16((x * rsqrt(mean(x^2) + eps)) * w), with the
// arithmetic AND the summation order of the reference's kernel (src/kernels/rmsnorm/rmsnorm.cu:51-110,
// 256 threads: thread t sums the squares of chunk t with fused multiply-adds, each warp combines its 32
// lanes by shuffle-down 16..1, warp 0 the 8 warp totals the same way).  The warp plays the reference's
// 8 warps in turn (lane l holds chunks l, 32 + l, ...), so the rows of a step are normalised side by
// side, one per warp, without a CTA-wide barrier.  hidden a multiple of 256, at most 2048; nw8 = this
// lane's chunks of the norm weight (chunk 32 g + lane in nw8[g]).
__device__ __forceinline__ void rmsnorm_row_by_warp(__nv_bfloat16* row, const uint4 (&nw8)[8], int hidden, float eps, int lane) {
  const int groups = hidden / 256;  // the reference's warps that hold data
  uint4 data[8];
  float tot = 0.0f;
#pragma unroll
  for (int g = 0; g < 8; g++) {
    if (g >= groups) continue;
    data[g] = reinterpret_cast<const uint4*>(row)[g * 32 + lane];
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
    s = __shfl_sync(0xffffffffu, s, 0);  // total of group g, on every lane
    if (lane == g) tot = s;
  }
  // second level: lanes 0..groups-1 hold the group totals, the rest zero, shuffle-down again
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) tot += __shfl_down_sync(0xffffffffu, tot, off);
  tot = __shfl_sync(0xffffffffu, tot, 0);
  const float rms_recip = rsqrtf(tot / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int g = 0; g < 8; g++) {
    if (g >= groups) continue;
    const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&data[g]);
    const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&nw8[g]);
    uint4 yd;
    __nv_bfloat162* yb = reinterpret_cast<__nv_bfloat162*>(&yd);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 xf = __bfloat1622float2(xb[j]);
      const float2 wf = __bfloat1622float2(wb[j]);
      yb[j] = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(xf.x, rms_recip), wf.x),
                                    __fmul_rn(__fmul_rn(xf.y, rms_recip), wf.y));
    }
    reinterpret_cast<uint4*>(row)[g * 32 + lane] = yd;
  }
}

}  // namespace pa
