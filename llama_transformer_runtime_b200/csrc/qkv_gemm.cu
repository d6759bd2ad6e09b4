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
// A PAIR of CTAs (a cluster of two, on the two SMs of one TPC) computes 256 tokens x 384 output
// columns (6 heads of the concatenation Wq | Wk | Wv) over K = 2048 in steps of 64 with
// tcgen05.mma.cta_group::2: M = 256 rows, 128 from each CTA's activation tile, accumulating in
// each CTA's own tensor memory; of every B operand each CTA loads only half of the N columns.  Per
// k-step a CTA moves 16 KiB of activations and 24 KiB of weights for 128 x 384 x 64 multiply-adds
// (one CTA per 256 x 256 tile moved 64 KiB for 256 x 256 x 64 and used 96 SMs).  2048 tokens x 3072
// columns are 8 x 8 pair tiles = 128 CTAs.
//   warp 8      load, 4 stages of 40 KiB.  Lane 0: the A tile (128 token rows x 64 k) with one
//               tiled TMA copy through a tensor map of the row-major activations (128-byte
//               swizzle: the copy lands as the canonical K-major operand; rows past the end read
//               as zeros).  Lanes 1..3: one 8 KiB bulk copy per head block of B (64 weight rows x
//               64 columns) from a tile image of the shared-memory layout the tensor cores want
//               (rows of 128 bytes, 16-byte chunks XOR-swizzled, MN-major), the same idea as the
//               KV cache's tile layout; the weights are packed once, at load time
//               (pack_weights_kernel).  With 16-byte cp.async from row-major weights the kernel
//               ran at 96 us per layer: lg_throttle and long_scoreboard stalls on the load path.
//   warps 0-7   while the MMA loop runs: which token each row is, its cache block, its RoPE
//               factors (into shared memory).  After the last step: thread = token row = TMEM
//               lane; the two warps of a 32-lane quarter take every other head of the tile; a
//               head's 32 rows x 128 bytes go through a staging tile so that the stores are whole
//               128-byte lines.
//   warp 9      first CTA of the pair: waits for its own stage and for the peer's (the peer's warp
//               9 forwards its "stage full" barrier with a remote arrive), then one elected lane
//               issues per 16-wide k-slice one MMA M256 N256 K16 (heads 0..3 of the tile; a CTA
//               holds two of them, 8 KiB apart: the descriptor's leading byte offset) and one
//               M256 N128 K16 (heads 4, 5), and frees the stage in BOTH CTAs with a multicast
//               tcgen05.commit.
// Measured on B200, 2048 tokens, per layer over 16 layers (the Q/K/V launch): 41.9 us with one CTA per 256 x 256
// tile and a packing kernel for the activations; 37.1 us as pairs with the tensor map and the
// coalesced epilogue; 34.8 us with the row lookups moved in front of the accumulator wait; 31.6 us
// with programmatic dependent launch between consecutive calls; 23.2 us (1110 TFLOP/s) once the
// peer's remote arrive was a CTA-scope release instead of a cluster-scope one, which had cost the
// forwarding thread 0.6 us per stage and set the pace of the whole loop (3, 4 and 5 stages, with
// or without the MMAs, with half the bytes: always 1100-1190 cycles per step).
// Every wait is bounded; on expiry the CTA raises its abort flag, the status word gets
// PA_ERR_TIMEOUT and all warps leave through the common exit, where the pair meets once more and
// tensor memory is released.
#include <cuda.h>  // CUtensorMap and the encode function's type; the function itself comes from the runtime's driver entry point

#include "kernels.cuh"
#include "rope.cuh"
#include "tc05.cuh"

namespace pa {

namespace {

constexpr int kGM = 128;        // tokens per CTA = per packed activation tile; the pair's MMA has M = 256
constexpr int kTileHeads = 6;   // most heads (64 output columns) per pair tile: 4 in the first MMA, 2 in the second
constexpr int kGK = 64;         // k per stage
constexpr int kGStages = 4;  // 3 and 5 stages run the MMA loop at the same pace
constexpr int kABytes = kGM * 128;            // 16 KiB
constexpr int kBBlock = kGK * 128;            // 8 KiB: 64 weight rows x one head
constexpr int kBSlots = 3;                    // head blocks a CTA holds per stage: 2 of the first MMA, 1 of the second
constexpr int kStageBytes = kABytes + kBSlots * kBBlock;  // 40 KiB
constexpr int kGOffRope = kGStages * kStageBytes;  // RoPE factors of the CTA's 128 rows: 65 floats per row
constexpr int kRopeBytes = kGM * 65 * 4;
constexpr int kGOffBar = kGOffRope + kRopeBytes;
constexpr int kGOffMisc = kGOffBar + (3 * kGStages + 1) * 8;
constexpr int kGSmem = kGOffMisc + 16 + 112;
constexpr int kEpiWarps = 8;      // two per 32-lane quarter of tensor memory, each takes every other head
constexpr int kLoadWarp = kEpiWarps, kMmaWarp = kEpiWarps + 1;
constexpr int kGemmThreads = (kEpiWarps + 2) * 32;
constexpr uint32_t kGTmemCols = 512;  // 6 heads x 64 fp32 columns, rounded up to a power of two

// Head g of the concatenated output (Q heads, then K heads, then V heads; or the one matrix of a
// plain linear layer): which matrix it comes from and where.
struct HeadSrc {
  const __nv_bfloat16* w;  // packed weights of its matrix
  int heads;               // heads (64-column blocks) of that matrix
  int head;                // head index inside the matrix
  int which;               // 0 Q, 1 K, 2 V (projection with RoPE + append); 3: plain linear layer with residual;
                           // 4: gate (even g) or up (odd g) head of the fused feed-forward GEMM
};
__device__ __forceinline__ HeadSrc head_src(const QkvGemmParams& p, int g) {
  const int hq = p.q_cols / 64, hk = p.kv_cols / 64;
  // gate and up heads alternate, so that a tile holds both accumulators of its output columns
  if (p.linear == 2) return HeadSrc{(g & 1) ? p.wk : p.wq, p.q_cols / 128, g >> 1, 4};
  if (p.linear) return HeadSrc{p.wq, hq, g, 3};
  if (g < hq) return HeadSrc{p.wq, hq, g, 0};
  if (g < hq + hk) return HeadSrc{p.wk, hk, g - hq, 1};
  return HeadSrc{p.wv, hk, g - hq - hk, 2};
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
qkv_gemm_kernel(const __grid_constant__ CUtensorMap x_map, QkvGemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {  // swizzle atoms need 1024-byte alignment (the same in both CTAs of the pair)
    if (threadIdx.x == 0) atomicExch(p.status, kStatusBadBlock);
    return;
  }
  unsigned char* sm = smem_raw;
  const uint32_t bar_full = base + kGOffBar, bar_empty = bar_full + 8 * kGStages;
  const uint32_t bar_peer = bar_empty + 8 * kGStages;  // first CTA only: the peer's stage is full
  const uint32_t bar_acc = bar_peer + 8 * kGStages;
  uint32_t* s_tmem_base = reinterpret_cast<uint32_t*>(sm + kGOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kGOffMisc + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs; 1: the peer
  const int tile_m = (int)blockIdx.y * 2 + (int)rank;  // this CTA's 128-row activation tile
  const int m0 = tile_m * kGM;
  const bool have_rows = m0 < p.rows;  // the last pair may have one row half only: the peer then loads no A
  const int total_heads = p.linear ? p.q_cols / 64 : (p.q_cols + 2 * p.kv_cols) / 64;
  const int g0 = (int)(blockIdx.x >> 1) * p.tile_heads;
  const int n_heads = min(p.tile_heads, total_heads - g0);  // 2, 4 or 6
  const int n1 = min(n_heads, 4);                          // heads of the first MMA
  const int k_steps = p.hidden / kGK;
  // head blocks this CTA loads: slots 0 .. n1/2-1 = its half of the first MMA's heads,
  // slot 2 = its head of the second MMA
  const int my_first = g0 + (int)rank * (n1 / 2);
  const int my_second = n_heads > 4 ? g0 + 4 + (int)rank : -1;

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kGStages; s++) {
      mbar_init(bar_full + 8 * s, 1);   // one arrival (with the byte count of all bulk copies of the stage)
      mbar_init(bar_empty + 8 * s, 1);  // the first CTA's commit, multicast to both
      mbar_init(bar_peer + 8 * s, 1);   // the peer's remote arrive
    }
    mbar_init(bar_acc, 1);
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc_pair(base + kGOffMisc, kGTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before a remote arrive or a multicast commit reaches them
  tc_fence_after();
  const uint32_t tmem = *s_tmem_base;
  // Launched with programmatic stream serialization: the set-up above may overlap the tail of the
  // kernel in front (its CTAs leave their SMs one by one); nothing in global memory is touched
  // before that kernel has completed.  The kernel behind this one may start its own set-up at once.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == kLoadWarp) {
    // ===================== loads ==============================================
    // lane 0: the A tile, through the tensor map of the row-major activations (box 64 k x 128
    // rows, 128-byte swizzle: the copy lands as the canonical K-major operand, rows past the end
    // read as zeros); lane 1 + s: the head block of slot s, from the packed weights
    const int slot = lane - 1;
    int g = -1;
    if (slot >= 0 && slot < n1 / 2) g = my_first + slot;
    if (slot == 2) g = my_second;
    const char* b_img = nullptr;
    size_t b_step = 0;
    if (g >= 0) {
      const HeadSrc h = head_src(p, g);
      b_img = reinterpret_cast<const char*>(h.w) + (size_t)h.head * kBBlock;
      b_step = (size_t)h.heads * kBBlock;
    }
    const uint32_t tx = (have_rows ? kABytes : 0) + (uint32_t)(n1 / 2 + (my_second >= 0 ? 1 : 0)) * kBBlock;
    for (int ks = 0; ks < k_steps; ks++) {
      const int st = ks % kGStages;
      if (!wait_or_abort(bar_empty + 8 * st, (uint32_t)(((ks / kGStages) & 1) ^ 1), abort_flag)) break;
      const uint32_t sA = base + st * kStageBytes, sB = sA + kABytes;
      if (lane == 0) mbar_expect_tx(bar_full + 8 * st, tx);
      __syncwarp();
      if (lane == 0 && have_rows) tensor_g2s_2d(sA, &x_map, ks * kGK, m0, bar_full + 8 * st);
      if (g >= 0) bulk_g2s(sB + slot * kBBlock, b_img + (size_t)ks * b_step, kBBlock, bar_full + 8 * st);
      __syncwarp();
    }
  } else if (warp < kEpiWarps) {
    // ===================== epilogue ============================================
    // Warp w reads the tensor-memory lanes of quarter w % 4 (the only ones it may) and takes the
    // tile's heads w / 4, w / 4 + 2, w / 4 + 4: thread = token row = TMEM lane.
    // Everything that does not need the accumulators happens while the MMA loop runs: which token a
    // row is, its cache block, its RoPE factors.
    {
      const int quarter = warp & 3, hb0 = warp >> 2;
      const int row = m0 + quarter * 32 + lane;  // token row; TMEM lane = quarter * 32 + lane
      const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
      const bool any_rope = !p.linear && g0 < (p.q_cols + p.kv_cols) / 64;
      const bool any_cache = !p.linear && g0 + n_heads > p.q_cols / 64;
      // which sequence and position this row is
      int seq = (p.linear && row < p.rows) ? 0 : -1, lpos = 0, pos = 0;
      for (int s = 0; !p.linear && s < p.n_seqs; s++) {
        const BatchEntry e = p.batch[s];
        if (row >= e.kv_row_off && row < e.kv_row_off + e.n_new) {
          seq = e.seq;
          lpos = e.kv_len - e.n_new + (row - e.kv_row_off);  // position inside the local cache
          pos = e.kv_pos_off + lpos;                          // RoPE position
        }
      }
      int blk = 0;
      if (seq >= 0 && any_cache) {
        blk = p.tables[(size_t)seq * p.max_blocks_per_seq + lpos / kBlockTok];
        if (blk < 0 || blk >= p.num_blocks) {
          atomicExch(p.status, kStatusBadBlock);
          seq = -1;
        }
      }
      const int slot = lpos % kBlockTok;
      // This row's RoPE factors, once per row: 16 vector loads into the row's slot of a shared-memory
      // table, 65 floats apart so that the 32 lanes of a warp hit 32 banks (the two warps of a quarter
      // write the same values).  Read per
      // element from global memory instead (scalar, one 128-byte line per lane and load, every head
      // over) they made the epilogue longer than the whole MMA loop.
      float* trow = reinterpret_cast<float*>(sm + kGOffRope) + (quarter * 32 + lane) * 65;
      if (any_rope && seq >= 0) {
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
      // per row: block id and slot for the cooperative stores below (negative: no token in the row)
      const int row_info = seq >= 0 ? ((blk << 4) | slot) : -1;
      unsigned char* stage = sm + warp * 4096;  // 32 rows x 128 bytes per warp, in the (then idle) stage ring
      const bool acc_ok = wait_or_abort(bar_acc, 0, abort_flag);
      tc_fence_after();
      // gate/up mode: a warp takes every other PAIR of heads (gate at hb, up at hb + 1)
      const bool gate_up = p.linear == 2;
#pragma unroll 1
      for (int hb = gate_up ? 2 * hb0 : hb0; acc_ok && hb < n_heads; hb += gate_up ? kEpiWarps / 2 : kEpiWarps / 4) {
        uint32_t acc[2][32];
        uint32_t lo[16], hi[16];  // bf16 pairs of elements 0..31 and 32..63
        if (gate_up) {
          // h = bf16(SiLU(bf16 gate) * bf16 up), the reference's GEMM outputs and its SiLU kernel's arithmetic
          // (src/kernels/silu/silu_8192.cu:55-100), as ffn_gate_up_kernel computes them for decode rows
#pragma unroll
          for (int half = 0; half < 2; half++) {
            tmem_ld32(tmem + lane_base + hb * 64 + half * 32, acc[0]);
            tmem_ld32(tmem + lane_base + (hb + 1) * 64 + half * 32, acc[1]);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; i++) {
              const float g0f = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[0][2 * i])));
              const float g1f = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[0][2 * i + 1])));
              const float u0f = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[1][2 * i])));
              const float u1f = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[1][2 * i + 1])));
              const float s0 = __fmul_rn(g0f, 1.0f / (1.0f + __expf(-g0f)));
              const float s1 = __fmul_rn(g1f, 1.0f / (1.0f + __expf(-g1f)));
              const uint32_t v = pack_bf16(__fmul_rn(s0, u0f), __fmul_rn(s1, u1f));
              if (half == 0) lo[i] = v; else hi[i] = v;
            }
          }
        } else {
          tmem_ld32(tmem + lane_base + hb * 64, acc[0]);
          tmem_ld32(tmem + lane_base + hb * 64 + 32, acc[1]);
          tmem_wait_ld();
        }
        // rows without a token skip the stores; the warp meets again before the next
        // (warp-wide, aligned) tensor-memory load
        __syncwarp();
        if (seq >= 0) {
        const HeadSrc hs = head_src(p, g0 + hb);
        const int which = hs.which, head = hs.head;
        // the GEMM's bf16 output, then RoPE on it: element i pairs with i + 32
        if (which == 4) {
          // lo and hi are made above
        } else if (which == 3) {
          // plain output: bf16 of the accumulator, then (optionally) the residual added in fp32 and
          // rounded once more, as the reference's GEMM and residual_add kernels do in turn
          const size_t at = (size_t)row * p.q_cols + head * 64;
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
        // this row's 128 bytes -> the warp's staging tile (chunks XOR-swizzled by row: conflict-free)
#pragma unroll
        for (int c = 0; c < 4; c++) {
          *reinterpret_cast<uint4*>(stage + tile_chunk_off(lane, c)) =
              make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
          *reinterpret_cast<uint4*>(stage + tile_chunk_off(lane, c + 4)) =
              make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
        }
        }
        __syncwarp();
        // The warp writes the 32 rows out four at a time, 8 lanes per row: whole 128-byte lines per
        // store instead of one 16-byte piece of 32 different lines.
        {
          const HeadSrc hs = head_src(p, g0 + hb);
          const int rr0 = lane >> 3, c = lane & 7;
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const int rr = it * 4 + rr0;
            const int info = __shfl_sync(0xffffffffu, row_info, rr);
            if (info < 0) continue;  // no token in that row
            const uint4 v = *reinterpret_cast<const uint4*>(stage + tile_chunk_off(rr, c));
            if (hs.which == 0 || hs.which == 3) {
              const size_t r = (size_t)(m0 + quarter * 32 + rr);
              reinterpret_cast<uint4*>(p.q_out + (r * (p.q_cols / 64) + hs.head) * kHeadDim)[c] = v;
            } else if (hs.which == 4) {  // rows of q_cols / 2 columns: one output head per gate/up pair
              const size_t r = (size_t)(m0 + quarter * 32 + rr);
              reinterpret_cast<uint4*>(p.q_out + (r * (p.q_cols / 128) + hs.head) * kHeadDim)[c] = v;
            } else {
              char* tile = p.storage + tile_off(info >> 4, p.kv_heads, hs.head, hs.which == 2 ? 1 : 0);
              *reinterpret_cast<uint4*>(tile + tile_chunk_off(info & 15, c)) = v;
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (rank == 0) {
    // ===================== MMA issue (first CTA of the pair) ====================
    // First MMA: N = 64 * n1 (the tile's heads 0..3), of which each CTA holds half, two 128-byte
    // atoms along N, 8 KiB apart (the next head's block): that distance is the descriptor's
    // leading byte offset.  Second MMA: N = 128 (heads 4, 5), one head per CTA, in slot 2.
    // (One CTA, N = 64 per MMA: 55.8 us per layer, shared-memory operand bandwidth; N = 128: 46.6.)
    const uint32_t idesc1 = idesc_bf16(2 * kGM, 64 * n1, true);
    constexpr uint32_t kIdesc2 = idesc_bf16(2 * kGM, 128, true);
    constexpr uint64_t kLboNextHead = (uint64_t)(kBBlock >> 4) << 16;
    for (int ks = 0; ks < k_steps; ks++) {
      const int st = ks % kGStages;
      const uint32_t par = (uint32_t)((ks / kGStages) & 1);
      if (!wait_or_abort(bar_full + 8 * st, par, abort_flag)) break;
      if (!wait_or_abort_cluster(bar_peer + 8 * st, par, abort_flag)) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t sA = base + st * kStageBytes, sB = sA + kABytes;
#pragma unroll
        for (int kk = 0; kk < kGK / 16; kk++) {
          const uint64_t a_desc = smem_desc_sw128(sA + kk * 32);
          umma_ss_pair(tmem, a_desc,
                       (smem_desc_sw128(sB + kk * 2048) & ~((uint64_t)0x3FFF << 16)) | kLboNextHead, idesc1,
                       (ks > 0 || kk > 0) ? 1u : 0u);
          if (n_heads > 4)
            umma_ss_pair(tmem + 256, a_desc, smem_desc_sw128(sB + 2 * kBBlock + kk * 2048), kIdesc2,
                         (ks > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit_pair(bar_empty + 8 * st, 3);
        if (ks + 1 == k_steps) tc_commit_pair(bar_acc, 3);
      }
      __syncwarp();
    }
  } else {
    // ===================== peer: forward "my stage is full" to the first CTA =====
    for (int ks = 0; ks < k_steps; ks++) {
      const int st = ks % kGStages;
      if (!wait_or_abort(bar_full + 8 * st, (uint32_t)((ks / kGStages) & 1), abort_flag)) break;
      if (lane == 0) mbar_arrive_remote(bar_peer + 8 * st, 0);
      __syncwarp();
    }
  }

  // ---- common exit: the pair meets, then tensor memory is released --------------
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.status, kStatusTimeout);
  cluster_sync_all();  // the peer's shared and tensor memory are no longer in use by this CTA's MMAs
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, kGTmemCols);
  }
}


// ---- the plain and the gate/up GEMM over many tiles: persistent pairs -------------------------
// When a launch has more pair tiles than the GPU has SM pairs (the gate/up GEMM of a prompt: 2048 x
// 16384 x 2048), CTAs that follow one another on an SM overlap nothing: a tile's set-up and epilogue
// (about a third of its time) run with the tensor cores idle.  Here a pair stays and takes tiles
// pair, pair + pairs, ...: tiles of 4 heads (256 columns), so that tensor memory holds TWO accumulator
// sets (2 x 256 columns); the loader and the MMA warp run on into the next tile while warps 0-7 read
// the previous tile's accumulators, and hand the set back with an arrival on the first CTA's
// "accumulators free" barrier (8 warps of each CTA; the peer's arrive remotely, release at cluster
// scope: the MMAs that follow overwrite the peer's tensor memory).  Same operand layouts, MMA shapes
// and epilogue arithmetic as qkv_gemm_kernel's linear modes; no RoPE, no cache.
constexpr int kPHeads = 4;                                  // heads per pair tile
constexpr int kPStageBytes = kABytes + (kPHeads / 2) * kBBlock;  // 32 KiB
constexpr int kPOffStaging = kGStages * kPStageBytes;       // 8 warps x 4 KiB, no longer inside the ring
constexpr int kPOffBar = kPOffStaging + kEpiWarps * 4096;
constexpr int kPOffMisc = kPOffBar + (3 * kGStages + 4) * 8;
constexpr int kPSmem = kPOffMisc + 16 + 112;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
linear_gemm_persistent_kernel(const __grid_constant__ CUtensorMap x_map, QkvGemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicExch(p.status, kStatusBadBlock);
    return;
  }
  unsigned char* sm = smem_raw;
  const uint32_t bar_full = base + kPOffBar, bar_empty = bar_full + 8 * kGStages;
  const uint32_t bar_peer = bar_empty + 8 * kGStages;     // first CTA only: the peer's stage is full
  const uint32_t bar_acc_full = bar_peer + 8 * kGStages;  // [2]: an accumulator set is complete (both CTAs)
  const uint32_t bar_acc_free = bar_acc_full + 16;        // [2], first CTA only: both CTAs have read the set
  uint32_t* s_tmem_base = reinterpret_cast<uint32_t*>(sm + kPOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kPOffMisc + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int total_heads = p.q_cols / 64;
  const int col_tiles = (total_heads + kPHeads - 1) / kPHeads;
  const int row_pairs = (p.rows + 2 * kGM - 1) / (2 * kGM);
  const int n_tiles = col_tiles * row_pairs;
  const int pair = (int)(blockIdx.x >> 1), n_pairs = (int)(gridDim.x >> 1);
  const int k_steps = p.hidden / kGK;

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kGStages; s++) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_peer + 8 * s, 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_free + 8 * b, 2 * kEpiWarps);
    }
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc_pair(base + kPOffMisc, kGTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = *s_tmem_base;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == kLoadWarp) {
    // ===================== loads: lane 0 the A tile, lanes 1, 2 this CTA's head blocks ==========
    uint32_t it = 0;
    bool ok = true;
    for (int t = pair; ok && t < n_tiles; t += n_pairs) {
      const int g0 = (t % col_tiles) * kPHeads, m0 = ((t / col_tiles) * 2 + (int)rank) * kGM;
      const int n_heads = min(kPHeads, total_heads - g0);  // 2 or 4
      const bool have_rows = m0 < p.rows;
      const int slot = lane - 1;
      const char* b_img = nullptr;
      size_t b_step = 0;
      if (slot >= 0 && slot < n_heads / 2) {
        const HeadSrc h = head_src(p, g0 + (int)rank * (n_heads / 2) + slot);
        b_img = reinterpret_cast<const char*>(h.w) + (size_t)h.head * kBBlock;
        b_step = (size_t)h.heads * kBBlock;
      }
      const uint32_t tx = (have_rows ? kABytes : 0) + (uint32_t)(n_heads / 2) * kBBlock;
      for (int ks = 0; ks < k_steps; ks++, it++) {
        const int st = it % kGStages;
        if (!wait_or_abort(bar_empty + 8 * st, ((it / kGStages) & 1) ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        const uint32_t sA = base + st * kPStageBytes, sB = sA + kABytes;
        if (lane == 0) mbar_expect_tx(bar_full + 8 * st, tx);
        __syncwarp();
        if (lane == 0 && have_rows) tensor_g2s_2d(sA, &x_map, ks * kGK, m0, bar_full + 8 * st);
        if (b_img) bulk_g2s(sB + slot * kBBlock, b_img + (size_t)ks * b_step, kBBlock, bar_full + 8 * st);
        __syncwarp();
      }
    }
  } else if (warp < kEpiWarps) {
    // ===================== epilogue: warp w reads lane quarter w % 4, heads (pairs) w / 4, ... ====
    const int quarter = warp & 3, hb0 = warp >> 2;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const bool gate_up = p.linear == 2;
    unsigned char* stage = sm + kPOffStaging + warp * 4096;
    uint32_t tile_iter = 0;
    for (int t = pair; t < n_tiles; t += n_pairs, tile_iter++) {
      const int g0 = (t % col_tiles) * kPHeads, m0 = ((t / col_tiles) * 2 + (int)rank) * kGM;
      const int n_heads = min(kPHeads, total_heads - g0);
      const uint32_t set = tile_iter & 1, acc = tmem + set * 256 + lane_base;
      const int row = m0 + quarter * 32 + lane;
      const bool valid = row < p.rows;
      if (!wait_or_abort(bar_acc_full + 8 * set, (tile_iter >> 1) & 1, abort_flag)) break;
      tc_fence_after();
#pragma unroll 1
      for (int hb = gate_up ? 2 * hb0 : hb0; hb < n_heads; hb += 2) {
        uint32_t a[2][32];
        uint32_t lo[16], hi[16];
        int out_head, out_heads;
        if (gate_up) {
          out_head = (g0 + hb) >> 1;
          out_heads = p.q_cols / 128;
#pragma unroll
          for (int half = 0; half < 2; half++) {
            tmem_ld32(acc + hb * 64 + half * 32, a[0]);
            tmem_ld32(acc + (hb + 1) * 64 + half * 32, a[1]);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; i++) {
              const float g0f = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[0][2 * i])));
              const float g1f = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[0][2 * i + 1])));
              const float u0f = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[1][2 * i])));
              const float u1f = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[1][2 * i + 1])));
              const float s0 = __fmul_rn(g0f, 1.0f / (1.0f + __expf(-g0f)));
              const float s1 = __fmul_rn(g1f, 1.0f / (1.0f + __expf(-g1f)));
              const uint32_t v = pack_bf16(__fmul_rn(s0, u0f), __fmul_rn(s1, u1f));
              if (half == 0) lo[i] = v; else hi[i] = v;
            }
          }
        } else {
          out_head = g0 + hb;
          out_heads = p.q_cols / 64;
          tmem_ld32(acc + hb * 64, a[0]);
          tmem_ld32(acc + hb * 64 + 32, a[1]);
          tmem_wait_ld();
          const size_t at = (size_t)row * p.q_cols + (size_t)out_head * 64;
          uint4 rl[4], rh[4];
          const bool res = p.residual && valid;
          if (res) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
              rl[c] = reinterpret_cast<const uint4*>(p.residual + at)[c];
              rh[c] = reinterpret_cast<const uint4*>(p.residual + at)[c + 4];
            }
          }
#pragma unroll
          for (int i = 0; i < 16; i++) {
            float a0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[0][2 * i])));
            float a1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[0][2 * i + 1])));
            float b0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[1][2 * i])));
            float b1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[1][2 * i + 1])));
            if (res) {
              const uint32_t ra = reinterpret_cast<const uint32_t*>(rl)[i], rb = reinterpret_cast<const uint32_t*>(rh)[i];
              a0 += __uint_as_float(ra << 16);
              a1 += __uint_as_float(ra & 0xffff0000u);
              b0 += __uint_as_float(rb << 16);
              b1 += __uint_as_float(rb & 0xffff0000u);
            }
            lo[i] = pack_bf16(a0, a1);
            hi[i] = pack_bf16(b0, b1);
          }
        }
        __syncwarp();  // the staging tile's previous rows have been written out
#pragma unroll
        for (int c = 0; c < 4; c++) {
          *reinterpret_cast<uint4*>(stage + tile_chunk_off(lane, c)) =
              make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
          *reinterpret_cast<uint4*>(stage + tile_chunk_off(lane, c + 4)) =
              make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
        }
        __syncwarp();
        // 32 rows out four at a time, 8 lanes per row: whole 128-byte lines per store
        const int rr0 = lane >> 3, c = lane & 7;
        const unsigned valid_rows = __ballot_sync(0xffffffffu, valid);
#pragma unroll
        for (int it8 = 0; it8 < 8; it8++) {
          const int rr = it8 * 4 + rr0;
          if (!((valid_rows >> rr) & 1u)) continue;
          const uint4 v = *reinterpret_cast<const uint4*>(stage + tile_chunk_off(rr, c));
          const size_t r = (size_t)(m0 + quarter * 32 + rr);
          reinterpret_cast<uint4*>(p.q_out + (r * out_heads + out_head) * kHeadDim)[c] = v;
        }
      }
      // this warp has read its share of the set: hand it back to the MMA warp of the first CTA
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0)
          mbar_arrive(bar_acc_free + 8 * set);
        else
          asm volatile(
              "{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, %1;\n\t"
              "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(bar_acc_free + 8 * set),
              "r"(0)
              : "memory");
      }
      __syncwarp();
    }
  } else if (rank == 0) {
    // ===================== MMA issue (first CTA of the pair) ====================
    constexpr uint64_t kLboNextHead = (uint64_t)(kBBlock >> 4) << 16;
    uint32_t it = 0, tile_iter = 0;
    bool ok = true;
    for (int t = pair; ok && t < n_tiles; t += n_pairs, tile_iter++) {
      const int g0 = (t % col_tiles) * kPHeads;
      const int n_heads = min(kPHeads, total_heads - g0);
      const uint32_t set = tile_iter & 1, d_tmem = tmem + set * 256;
      const uint32_t idesc = idesc_bf16(2 * kGM, 64 * n_heads, true);
      // the set's previous tile (two tiles ago) has been read by all 16 epilogue warps of the pair
      if (!wait_or_abort_cluster(bar_acc_free + 8 * set, ((tile_iter >> 1) & 1) ^ 1, abort_flag)) break;
      tc_fence_after();
      for (int ks = 0; ks < k_steps; ks++, it++) {
        const int st = it % kGStages;
        const uint32_t par = (it / kGStages) & 1;
        if (!wait_or_abort(bar_full + 8 * st, par, abort_flag) ||
            !wait_or_abort_cluster(bar_peer + 8 * st, par, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (elect_one()) {
          const uint32_t sA = base + st * kPStageBytes, sB = sA + kABytes;
#pragma unroll
          for (int kk = 0; kk < kGK / 16; kk++)
            umma_ss_pair(d_tmem, smem_desc_sw128(sA + kk * 32),
                         (smem_desc_sw128(sB + kk * 2048) & ~((uint64_t)0x3FFF << 16)) | kLboNextHead, idesc,
                         (ks > 0 || kk > 0) ? 1u : 0u);
          tc_commit_pair(bar_empty + 8 * st, 3);
          if (ks + 1 == k_steps) tc_commit_pair(bar_acc_full + 8 * set, 3);
        }
        __syncwarp();
      }
    }
  } else {
    // ===================== peer: forward "my stage is full" to the first CTA =====
    uint32_t it = 0;
    bool ok = true;
    for (int t = pair; ok && t < n_tiles; t += n_pairs)
      for (int ks = 0; ks < k_steps; ks++, it++) {
        const int st = it % kGStages;
        if (!wait_or_abort(bar_full + 8 * st, (it / kGStages) & 1, abort_flag)) {
          ok = false;
          break;
        }
        if (lane == 0) mbar_arrive_remote(bar_peer + 8 * st, 0);
        __syncwarp();
      }
  }

  // ---- common exit: the pair meets, then tensor memory is released --------------
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.status, kStatusTimeout);
  cluster_sync_all();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, kGTmemCols);
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

}  // namespace

cudaError_t launch_pack_weights(const void* src, void* dst, int hidden, int cols, cudaStream_t stream) {
  pack_weights_kernel<<<148 * 4, 256, 0, stream>>>((const __nv_bfloat16*)src, (char*)dst, hidden, cols);
  return cudaGetLastError();
}

namespace {

// cuTensorMapEncodeTiled, fetched through the runtime so that the library does not link the driver.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
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
  const int total_heads = (p.linear ? p.q_cols : p.q_cols + 2 * p.kv_cols) / 64;
  if (total_heads % 2 != 0) return cudaErrorInvalidValue;  // a pair splits every MMA's heads in two
  // The activations as a 2-D tensor [rows, hidden] of bf16, read in boxes of 128 rows x 64 k with the
  // 128-byte swizzle.  Base 16-byte aligned, row pitch a multiple of 16 bytes.
  if ((reinterpret_cast<uintptr_t>(p.x) & 15u) != 0 || p.hidden % 64 != 0) return cudaErrorInvalidValue;
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return cudaErrorNotSupported;
  CUtensorMap x_map;
  const cuuint64_t dims[2] = {(cuuint64_t)p.hidden, (cuuint64_t)p.rows};
  const cuuint64_t pitch[1] = {(cuuint64_t)p.hidden * sizeof(__nv_bfloat16)};
  const cuuint32_t box[2] = {(cuuint32_t)kGK, (cuuint32_t)kGM};
  const cuuint32_t elem_stride[2] = {1, 1};
  if (encode(&x_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(p.x), dims, pitch, box, elem_stride,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  // more pair tiles than SM pairs, no RoPE or cache: the persistent form
  {
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int p_tiles = ((total_heads + kPHeads - 1) / kPHeads) * ((p.rows + 2 * kGM - 1) / (2 * kGM));
    if (p.linear && p_tiles > sms / 2) {
      static bool p_configured[64] = {};
      if (dev >= 0 && dev < 64 && !p_configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(linear_gemm_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPSmem);
        if (e != cudaSuccess) return e;
        p_configured[dev] = true;
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * (sms / 2));
      cfg.blockDim = dim3(kGemmThreads);
      cfg.dynamicSmemBytes = kPSmem;
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      return cudaLaunchKernelEx(&cfg, linear_gemm_persistent_kernel, x_map, p);
    }
  }
  // x: the two CTAs of a pair (the kernel's compile-time cluster) next to each other
  // Tile width: 6 heads per pair, or 4 where that fills the SMs better (2048 columns are 5 1/3 tiles of
  // 6 heads = 96 CTAs for 2048 rows, but 8 tiles of 4 = 128 CTAs of two thirds the work).  Cost of a
  // choice = waves x (heads per tile + 2, the activation tile's share of a step).
  QkvGemmParams q = p;
  const int row_pairs = (p.rows + 2 * kGM - 1) / (2 * kGM);
  if (q.tile_heads != 4 && q.tile_heads != kTileHeads) {
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    auto cost = [&](int th) {
      const long long ctas = 2LL * ((total_heads + th - 1) / th) * row_pairs;
      return ((ctas + sms - 1) / sms) * (th + 2);
    };
    q.tile_heads = cost(4) < cost(kTileHeads) ? 4 : kTileHeads;
  }
  // (Launch order: pairs of one activation tile next to each other.  Pairs of one weight tile next to
  // each other made no difference on 2048 x 16384 x 2048: 308 against 310 us per layer of a prompt.)
  const dim3 grid(2 * ((total_heads + q.tile_heads - 1) / q.tile_heads), row_pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kGSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, qkv_gemm_kernel, x_map, q);
}

}  // namespace pa
