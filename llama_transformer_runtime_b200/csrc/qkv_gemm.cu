// Q/K/V projections of a prefill chunk on the 5th-generation tensor cores, with
// RoPE and the paged-cache append as the epilogue.
//
// Replaces, in one launch, what the reference's Attention::forward does between
// the normalised input and the attention kernel (src/runtime/attention.cu:138-262):
// three tensor-core GEMMs (launch_gemm_2048x2048, 2 x launch_gemm_2048x512; A
// [tokens, 2048] row-major, B [2048, N] row-major, fp32 accumulation, bf16 out),
// rope_q_kernel / rope_k_kernel / transpose_v_kernel (src/kernels/rope/rope.cu)
// and the 2*8*tokens 128-byte copies into the cache.  Numerics follow that
// chain: the fp32 accumulator is rounded to bf16 (the GEMM's output), RoPE runs
// in fp32 on those bf16 values with the same rounding as append_kernel, V is
// stored as it comes out.
//
// One CTA computes 256 tokens (two M = 128 halves) x 256 output columns (4 heads
// of one of Wq, Wk, Wv) over K = 2048 in steps of 64.  The tile is that large
// because every byte of it comes through L2: with 128 x 256 tiles (85 flop per
// loaded byte, 295 MB of L2-to-SM traffic per layer) the kernel sat at 96 us per
// layer whatever the load mechanism; 256 x 256 tiles move 197 MB.
//   warp 0      load: per step one 16 KiB bulk (TMA) copy per row half for the A tile (128
//               token rows x 64 k) and ONE 32 KiB bulk copy for the B tile (64 weight rows
//               x 4 heads), 3 stages of 64 KiB.  Both operands are read from tile images of
//               the shared-memory layout the tensor cores want (rows of 128 bytes,
//               16-byte chunks XOR-swizzled; A K-major, B MN-major), the same idea
//               as the KV cache's tile layout: the weights are packed once, at load
//               time (pack_weights_kernel), the activations by a small kernel in
//               front of the GEMM (pack_x_kernel, 8 MB in, 8 MB out per layer).
//               With 16-byte cp.async from the row-major arrays instead the kernel
//               ran at 96 us per layer: lg_throttle and long_scoreboard stalls on
//               the load path, tensor pipe 18 % busy.
//   warps 0-3   epilogue after the last step: thread = token row = TMEM lane.
//   warp 4      issues, per step, row half and 16-wide k-slice, one tcgen05.mma
//               M128 N256 K16 from an elected lane (8 per step) into the half's 256
//               TMEM columns — B spans four 128-byte atoms along N, 8 KiB apart,
//               which is the descriptor's leading byte offset — and frees the
//               stage with tcgen05.commit.
// Every wait is bounded; on expiry the CTA raises its abort flag, the status
// word gets PA_ERR_TIMEOUT and all warps leave through the common exit, where
// tensor memory is released.
#include "kernels.cuh"
#include "rope.cuh"
#include "tc05.cuh"

namespace pa {

namespace {

constexpr int kGM = 128;        // tokens per UMMA (M = 128) and per packed activation tile
constexpr int kGMH = 2;         // row halves per CTA: 256 tokens share every weight tile
constexpr int kGN = 256;        // output columns per CTA (4 heads)
constexpr int kGK = 64;         // k per stage
constexpr int kGStages = 3;
constexpr int kABytes = kGM * 128;            // 16 KiB
constexpr int kBBytes = (kGN / 64) * kGK * 128;  // 4 head blocks x 8 KiB
constexpr int kStageBytes = kGMH * kABytes + kBBytes;  // 64 KiB
constexpr int kGOffBar = kGStages * kStageBytes;
constexpr int kGOffMisc = kGOffBar + (2 * kGStages + 1) * 8;
constexpr int kGSmem = kGOffMisc + 16 + 112;
constexpr int kGemmThreads = 160;  // 4 epilogue warps (warp 0 also loads) + the MMA warp
constexpr uint32_t kGTmemCols = 512;  // 2 row halves x 4 heads x 64 fp32 columns

__global__ void __launch_bounds__(kGemmThreads, 1)
qkv_gemm_kernel(QkvGemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {  // swizzle atoms need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(p.status, kStatusBadBlock);
    return;
  }
  unsigned char* sm = smem_raw;
  const uint32_t bar_full = base + kGOffBar, bar_empty = bar_full + 8 * kGStages;
  const uint32_t bar_acc = bar_empty + 8 * kGStages;
  uint32_t* s_tmem_base = reinterpret_cast<uint32_t*>(sm + kGOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kGOffMisc + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.y * (kGMH * kGM);
  // column tile -> matrix and first column: tiles of Wq, then Wk, then Wv
  const int tq = p.q_cols / kGN, tk = p.kv_cols / kGN;
  const int ct = blockIdx.x;
  // which: 0 Q, 1 K, 2 V (projection with RoPE + append); 3: plain linear layer with residual
  const int which = p.linear ? 3 : (ct < tq ? 0 : (ct < tq + tk ? 1 : 2));
  const int n0 = (ct - ((which == 0 || which == 3) ? 0 : (which == 1 ? tq : tq + tk))) * kGN;
  const int n_cols = (which == 0 || which == 3) ? p.q_cols : p.kv_cols;
  const __nv_bfloat16* w = (which == 0 || which == 3) ? p.wq : (which == 1 ? p.wk : p.wv);
  const int k_steps = p.hidden / kGK;

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kGStages; s++) {
      mbar_init(bar_full + 8 * s, 1);  // one arrival (with the byte count of both bulk copies)
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc, 1);
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(base + kGOffMisc, kGTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem_base;

  if (warp < 4) {
    // ===================== loads ==============================================
    bool ok = true;
    if (warp == 0) {
      const char* a_img = reinterpret_cast<const char*>(p.x) + (size_t)blockIdx.y * kGMH * k_steps * kABytes;
      const int tiles_m = (p.rows + kGM - 1) / kGM;  // packed activation tiles that exist
      const char* b_img = reinterpret_cast<const char*>(w) + (size_t)(n0 / 64) * (kGK * 128);
      for (int ks = 0; ks < k_steps; ks++) {
        const int st = ks % kGStages;
        if (!wait_or_abort(bar_empty + 8 * st, (uint32_t)(((ks / kGStages) & 1) ^ 1), abort_flag)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t sA = base + st * kStageBytes, sB = sA + kGMH * kABytes;
          const bool second = (int)blockIdx.y * kGMH + 1 < tiles_m;  // the last CTA row may have one half only
          mbar_expect_tx(bar_full + 8 * st, (second ? 2 : 1) * kABytes + kBBytes);
          bulk_g2s(sA, a_img + (size_t)ks * kABytes, kABytes, bar_full + 8 * st);
          if (second)
            bulk_g2s(sA + kABytes, a_img + ((size_t)k_steps + ks) * kABytes, kABytes, bar_full + 8 * st);
          // the 4 head blocks of this k-step are adjacent in the packed weights
          bulk_g2s(sB, b_img + (size_t)ks * (n_cols / 64) * (kGK * 128), kBBytes, bar_full + 8 * st);
        }
        __syncwarp();
      }
    }

    // ===================== epilogue ============================================
    if (ok && wait_or_abort(bar_acc, 0, abort_flag)) {
      tc_fence_after();
#pragma unroll 1
      for (int mh = 0; mh < kGMH; mh++) {
      const int row = m0 + mh * kGM + warp * 32 + lane;  // token row; TMEM lane = warp * 32 + lane
      const uint32_t lane_base = ((uint32_t)(warp * 32) << 16) + (uint32_t)(mh * kGN);
      // which sequence and position this row is
      int seq = (which == 3 && row < p.rows) ? 0 : -1, lpos = 0, pos = 0;
      for (int s = 0; which != 3 && s < p.n_seqs; s++) {
        const BatchEntry e = p.batch[s];
        if (row >= e.kv_row_off && row < e.kv_row_off + e.n_new) {
          seq = e.seq;
          lpos = e.kv_len - e.n_new + (row - e.kv_row_off);  // position inside the local cache
          pos = e.kv_pos_off + lpos;                          // RoPE position
        }
      }
      int blk = 0;
      if (seq >= 0 && (which == 1 || which == 2)) {
        blk = p.tables[(size_t)seq * p.max_blocks_per_seq + lpos / kBlockTok];
        if (blk < 0 || blk >= p.num_blocks) {
          atomicExch(p.status, kStatusBadBlock);
          seq = -1;
        }
      }
      const int slot = lpos % kBlockTok;
      // This row's RoPE factors, once per row: 16 vector loads into a private row of the (now
      // idle) stage ring, 65 floats apart so that the 32 lanes of a warp hit 32 banks.  Read per
      // element from global memory instead (scalar, one 128-byte line per lane and load, 4 heads
      // over) they made the epilogue longer than the whole MMA loop.
      float* trow = reinterpret_cast<float*>(sm) + (warp * 32 + lane) * 65;
      if (which < 2 && seq >= 0) {
        const float4* cs4 = reinterpret_cast<const float4*>(p.cos_table + (size_t)pos * 32);
        const float4* sn4 = reinterpret_cast<const float4*>(p.sin_table + (size_t)pos * 32);
        float4 cv[8], sv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
          cv[i] = cs4[i];
          sv[i] = sn4[i];
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
          trow[4 * i] = cv[i].x;
          trow[4 * i + 1] = cv[i].y;
          trow[4 * i + 2] = cv[i].z;
          trow[4 * i + 3] = cv[i].w;
          trow[32 + 4 * i] = sv[i].x;
          trow[32 + 4 * i + 1] = sv[i].y;
          trow[32 + 4 * i + 2] = sv[i].z;
          trow[32 + 4 * i + 3] = sv[i].w;
        }
      }
      __syncwarp();
#pragma unroll 1
      for (int hb = 0; hb < kGN / 64; hb++) {
        uint32_t acc[2][32];
        tmem_ld32(tmem + lane_base + hb * 64, acc[0]);
        tmem_ld32(tmem + lane_base + hb * 64 + 32, acc[1]);
        tmem_wait_ld();
        // rows without a token skip the stores; the warp meets again before the next
        // (warp-wide, aligned) tensor-memory load
        __syncwarp();
        if (seq >= 0) {
        const int head = n0 / 64 + hb;
        // the GEMM's bf16 output, then RoPE on it: element i pairs with i + 32
        uint32_t lo[16], hi[16];  // bf16 pairs of elements 0..31 and 32..63
        if (which == 3) {
          // plain output: bf16 of the accumulator, then (optionally) the residual added in fp32 and
          // rounded once more, as the reference's GEMM and residual_add kernels do in turn
          const size_t at = (size_t)row * p.q_cols + n0 + hb * 64;
          uint4 rl[4], rh[4];
          if (p.residual) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
              rl[c] = reinterpret_cast<const uint4*>(p.residual + at)[c];
              rh[c] = reinterpret_cast<const uint4*>(p.residual + at)[c + 4];
            }
          }
#pragma unroll
          for (int i = 0; i < 16; i++) {
            float a0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[0][2 * i])));
            float a1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[0][2 * i + 1])));
            float b0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[1][2 * i])));
            float b1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[1][2 * i + 1])));
            if (p.residual) {
              const uint32_t ra = reinterpret_cast<const uint32_t*>(rl)[i], rb = reinterpret_cast<const uint32_t*>(rh)[i];
              a0 += __uint_as_float(ra << 16);
              a1 += __uint_as_float(ra & 0xffff0000u);
              b0 += __uint_as_float(rb << 16);
              b1 += __uint_as_float(rb & 0xffff0000u);
            }
            lo[i] = pack_bf16(a0, a1);
            hi[i] = pack_bf16(b0, b1);
          }
        } else if (which == 2) {
#pragma unroll
          for (int i = 0; i < 16; i++) {
            lo[i] = pack_bf16(__uint_as_float(acc[0][2 * i]), __uint_as_float(acc[0][2 * i + 1]));
            hi[i] = pack_bf16(__uint_as_float(acc[1][2 * i]), __uint_as_float(acc[1][2 * i + 1]));
          }
        } else {
          const float* cs = trow;
          const float* sn = trow + 32;
#pragma unroll
          for (int i = 0; i < 16; i++) {
            const float x0a = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[0][2 * i])));
            const float x0b = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[0][2 * i + 1])));
            const float x1a = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[1][2 * i])));
            const float x1b = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[1][2 * i + 1])));
            float y0a, y1a, y0b, y1b;
            rope_pair<1>(x0a, x1a, cs[2 * i], sn[2 * i], y0a, y1a);
            rope_pair<1>(x0b, x1b, cs[2 * i + 1], sn[2 * i + 1], y0b, y1b);
            lo[i] = pack_bf16(y0a, y0b);
            hi[i] = pack_bf16(y1a, y1b);
          }
        }
        if (which == 0 || which == 3) {
          uint4* dst = reinterpret_cast<uint4*>(p.q_out + ((size_t)row * (p.q_cols / 64) + head) * kHeadDim);
#pragma unroll
          for (int c = 0; c < 4; c++) {
            dst[c] = make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
            dst[c + 4] = make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
          }
        } else {
          char* tile = p.storage + tile_off(blk, p.kv_heads, head, which == 2 ? 1 : 0);
#pragma unroll
          for (int c = 0; c < 4; c++) {
            *reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c)) =
                make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
            *reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c + 4)) =
                make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
          }
        }
        }
        __syncwarp();
      }
      }
    }
  } else {
    // ===================== MMA issue =========================================
    // N = 256: the CTA's four heads in one MMA.  The B operand then spans four 128-byte atoms
    // along N, 8 KiB apart (the next head's block): that distance is the descriptor's leading
    // byte offset.  (N = 64 per MMA: 55.8 us per layer, shared-memory operand bandwidth; N = 128: 46.6.)
    constexpr uint32_t kIdesc = idesc_bf16(kGM, kGN, true);
    constexpr uint64_t kLboNextHead = (uint64_t)((kGK * 128) >> 4) << 16;
    // the last CTA row may hold one 128-row half only: its second half is never loaded nor multiplied
    const int n_halves = ((int)blockIdx.y * kGMH + 1 < (p.rows + kGM - 1) / kGM) ? kGMH : 1;
    for (int ks = 0; ks < k_steps; ks++) {
      const int st = ks % kGStages;
      if (!wait_or_abort(bar_full + 8 * st, (uint32_t)((ks / kGStages) & 1), abort_flag)) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t sA = base + st * kStageBytes, sB = sA + kGMH * kABytes;
#pragma unroll 1
        for (int mh = 0; mh < n_halves; mh++)
#pragma unroll
          for (int kk = 0; kk < kGK / 16; kk++)
            umma_ss(tmem + mh * kGN, smem_desc_sw128(sA + mh * kABytes + kk * 32),
                    (smem_desc_sw128(sB + kk * 2048) & ~((uint64_t)0x3FFF << 16)) | kLboNextHead, kIdesc,
                    (ks > 0 || kk > 0) ? 1u : 0u);
        tc_commit(bar_empty + 8 * st);
        if (ks + 1 == k_steps) tc_commit(bar_acc);
      }
      __syncwarp();
    }
  }

  // ---- common exit: release tensor memory -----------------------------------
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.status, kStatusTimeout);
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, kGTmemCols);
  }
}


// Row-major [hidden, cols] weights -> the shared-memory image the GEMM copies:
// block (k-tile of 64 rows, head of 64 columns) = 64 rows of 128 bytes, 16-byte
// chunk c of row r stored at c ^ (r & 7).  One thread per 16-byte chunk.
__global__ void __launch_bounds__(256)
pack_weights_kernel(const __nv_bfloat16* src, char* dst, int hidden, int cols) {
  const size_t total = (size_t)hidden * cols / 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i & 7);
    const size_t rc = i >> 3;                       // (row, head)
    const int head = (int)(rc % (cols / 64));
    const int row = (int)(rc / (cols / 64));
    const int r = row & 63, kt = row >> 6;
    const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)row * cols + head * 64 + c * 8);
    *reinterpret_cast<uint4*>(dst + ((size_t)kt * (cols / 64) + head) * (kGK * 128) + r * 128 + ((c ^ (r & 7)) << 4)) = v;
  }
}

// Row-major activations [rows, hidden] -> per (128-row tile, 64-k tile) a 16 KiB block of 128-byte
// rows, 16-byte chunk c of row r stored at c ^ (r & 7); rows beyond `rows` are zero.
__global__ void __launch_bounds__(256)
pack_x_kernel(const __nv_bfloat16* x, char* dst, int rows, int hidden) {
  const int cpr = hidden / 8;  // chunks per row
  const size_t total = (size_t)((rows + kGM - 1) / kGM) * kGM * cpr;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int cg = (int)(i % cpr);
    const int row = (int)(i / cpr);
    const int r = row % kGM, mt = row / kGM, kt = cg >> 3, c = cg & 7;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows) v = *reinterpret_cast<const uint4*>(x + (size_t)row * hidden + cg * 8);
    *reinterpret_cast<uint4*>(dst + ((size_t)mt * (hidden / kGK) + kt) * kABytes + r * 128 + ((c ^ (r & 7)) << 4)) = v;
  }
}

}  // namespace

cudaError_t launch_pack_x(const void* x, void* dst, int rows, int hidden, cudaStream_t stream) {
  const size_t total = (size_t)((rows + kGM - 1) / kGM) * kGM * (hidden / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  pack_x_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (char*)dst, rows, hidden);
  return cudaGetLastError();
}

cudaError_t launch_pack_weights(const void* src, void* dst, int hidden, int cols, cudaStream_t stream) {
  pack_weights_kernel<<<148 * 4, 256, 0, stream>>>((const __nv_bfloat16*)src, (char*)dst, hidden, cols);
  return cudaGetLastError();
}

cudaError_t launch_qkv_gemm(const QkvGemmParams& p, cudaStream_t stream) {
  if (p.rows <= 0) return cudaSuccess;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(qkv_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const dim3 grid((p.linear ? p.q_cols : p.q_cols + 2 * p.kv_cols) / kGN, (p.rows + kGMH * kGM - 1) / (kGMH * kGM));
  qkv_gemm_kernel<<<grid, kGemmThreads, kGSmem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace pa
