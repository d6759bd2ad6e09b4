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
// One CTA computes 128 tokens x 256 output columns (4 heads of one of Wq, Wk,
// Wv) over K = 2048 in steps of 64:
//   warps 0-3   load: per step the A tile (128 rows x 128 bytes of x) and the B
//               tile (64 weight rows x 512 bytes) go to shared memory with 16-byte
//               cp.async into the 128-byte-swizzle layouts the tensor cores read
//               (A K-major, B MN-major, one 8 KiB block per head), 4 stages;
//               a stage is handed over (wait_group, fence.proxy.async, mbarrier
//               arrive) two steps after it was issued.  After the last step the
//               same warps run the epilogue: thread = token row = TMEM lane.
//   warp 4      issues 16 tcgen05.mma (M128 N64 K16) per step from one elected
//               lane into 4 x 64 TMEM columns and frees the stage with
//               tcgen05.commit.
// Every wait is bounded; on expiry the CTA raises its abort flag, the status
// word gets PA_ERR_TIMEOUT and all warps leave through the common exit, where
// tensor memory is released.
#include "kernels.cuh"
#include "rope.cuh"
#include "tc05.cuh"

namespace pa {

namespace {

constexpr int kGM = 128;        // tokens per CTA
constexpr int kGN = 256;        // output columns per CTA (4 heads)
constexpr int kGK = 64;         // k per stage
constexpr int kGStages = 4;
constexpr int kABytes = kGM * 128;            // 16 KiB
constexpr int kBBytes = (kGN / 64) * kGK * 128;  // 4 head blocks x 8 KiB
constexpr int kGOffBar = kGStages * (kABytes + kBBytes);
constexpr int kGOffMisc = kGOffBar + (2 * kGStages + 1) * 8;
constexpr int kGSmem = kGOffMisc + 16 + 112;
constexpr int kLoadThreads = 128;
constexpr int kGemmThreads = 160;  // 4 load/epilogue warps + the MMA warp
constexpr uint32_t kGTmemCols = 256;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

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
  const int m0 = blockIdx.y * kGM;
  // column tile -> matrix and first column: tiles of Wq, then Wk, then Wv
  const int tq = p.q_cols / kGN, tk = p.kv_cols / kGN;
  const int ct = blockIdx.x;
  const int which = ct < tq ? 0 : (ct < tq + tk ? 1 : 2);
  const int n0 = (ct - (which == 0 ? 0 : (which == 1 ? tq : tq + tk))) * kGN;
  const int n_cols = which == 0 ? p.q_cols : p.kv_cols;
  const __nv_bfloat16* w = which == 0 ? p.wq : (which == 1 ? p.wk : p.wv);
  const int k_steps = p.hidden / kGK;

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kGStages; s++) {
      mbar_init(bar_full + 8 * s, kLoadThreads);
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
    auto hand_over = [&](int ks) {  // stage of step ks has landed: make it visible to the tensor cores
      fence_proxy_async_smem();
      mbar_arrive(bar_full + 8 * (ks % kGStages));
    };
    for (int ks = 0; ks < k_steps && ok; ks++) {
      const int st = ks % kGStages;
      if (!wait_or_abort(bar_empty + 8 * st, (uint32_t)(((ks / kGStages) & 1) ^ 1), abort_flag)) {
        ok = false;
        break;
      }
      const uint32_t sA = base + st * (kABytes + kBBytes), sB = sA + kABytes;
      const int k0 = ks * kGK;
      // A: 128 rows x 8 chunks
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int q = tid + kLoadThreads * j;
        const int r = q >> 3, c = q & 7;
        const bool valid = m0 + r < p.rows;
        const __nv_bfloat16* src = p.x + (size_t)(valid ? m0 + r : 0) * p.hidden + k0 + c * 8;
        cp_async16(sA + r * 128 + ((c ^ (r & 7)) << 4), src, valid);
      }
      // B: 64 weight rows x (4 head blocks x 8 chunks); 32 consecutive threads read 512 contiguous bytes
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const int q = tid + kLoadThreads * j;
        const int r = q >> 5, rem = q & 31;
        const int hb = rem >> 3, c = rem & 7;
        const __nv_bfloat16* src = w + (size_t)(k0 + r) * n_cols + n0 + hb * 64 + c * 8;
        cp_async16(sB + hb * (kGK * 128) + r * 128 + ((c ^ (r & 7)) << 4), src, true);
      }
      cp_async_commit();
      if (ks >= 2) {
        cp_async_wait<2>();
        hand_over(ks - 2);
      }
    }
    if (ok) {
      if (k_steps >= 2) {
        cp_async_wait<1>();
        hand_over(k_steps - 2);
      }
      cp_async_wait<0>();
      hand_over(k_steps - 1);
    } else {
      cp_async_wait<0>();
    }

    // ===================== epilogue ============================================
    if (ok && wait_or_abort(bar_acc, 0, abort_flag)) {
      tc_fence_after();
      const int row = m0 + warp * 32 + lane;  // token row = TMEM lane
      const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
      // which sequence and position this row is
      int seq = -1, lpos = 0, pos = 0;
      for (int s = 0; s < p.n_seqs; s++) {
        const BatchEntry e = p.batch[s];
        if (row >= e.kv_row_off && row < e.kv_row_off + e.n_new) {
          seq = e.seq;
          lpos = e.kv_len - e.n_new + (row - e.kv_row_off);  // position inside the local cache
          pos = e.kv_pos_off + lpos;                          // RoPE position
        }
      }
      int blk = 0;
      if (seq >= 0 && which != 0) {
        blk = p.tables[(size_t)seq * p.max_blocks_per_seq + lpos / kBlockTok];
        if (blk < 0 || blk >= p.num_blocks) {
          atomicExch(p.status, kStatusBadBlock);
          seq = -1;
        }
      }
      const int slot = lpos % kBlockTok;
#pragma unroll 1
      for (int hb = 0; hb < kGN / 64; hb++) {
        uint32_t acc[2][32];
        tmem_ld32(tmem + lane_base + hb * 64, acc[0]);
        tmem_ld32(tmem + lane_base + hb * 64 + 32, acc[1]);
        tmem_wait_ld();
        if (seq < 0) continue;
        const int head = n0 / 64 + hb;
        // the GEMM's bf16 output, then RoPE on it: element i pairs with i + 32
        uint32_t lo[16], hi[16];  // bf16 pairs of elements 0..31 and 32..63
        if (which == 2) {
#pragma unroll
          for (int i = 0; i < 16; i++) {
            lo[i] = pack_bf16(__uint_as_float(acc[0][2 * i]), __uint_as_float(acc[0][2 * i + 1]));
            hi[i] = pack_bf16(__uint_as_float(acc[1][2 * i]), __uint_as_float(acc[1][2 * i + 1]));
          }
        } else {
          const float* cs = p.cos_table + (size_t)pos * 32;
          const float* sn = p.sin_table + (size_t)pos * 32;
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
        if (which == 0) {
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
    }
  } else {
    // ===================== MMA issue =========================================
    constexpr uint32_t kIdesc = idesc_bf16(kGM, 64, true);
    for (int ks = 0; ks < k_steps; ks++) {
      const int st = ks % kGStages;
      if (!wait_or_abort(bar_full + 8 * st, (uint32_t)((ks / kGStages) & 1), abort_flag)) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t sA = base + st * (kABytes + kBBytes), sB = sA + kABytes;
#pragma unroll
        for (int hb = 0; hb < kGN / 64; hb++)
#pragma unroll
          for (int kk = 0; kk < kGK / 16; kk++)
            umma_ss(tmem + hb * 64, smem_desc_sw128(sA + kk * 32),
                    smem_desc_sw128(sB + hb * (kGK * 128) + kk * 2048), kIdesc, (ks > 0 || kk > 0) ? 1u : 0u);
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

}  // namespace

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
  const dim3 grid((p.q_cols + 2 * p.kv_cols) / kGN, (p.rows + kGM - 1) / kGM);
  qkv_gemm_kernel<<<grid, kGemmThreads, kGSmem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace pa
