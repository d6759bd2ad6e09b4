// K3: causal GQA prefill attention over the paged cache on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Replaces the reference's flash_attention_fat_kernel for q_seq_len > 1
// (src/kernels/flashattention/flashattention.cu:98-376: mma.sync m16n8k16,
// 64x64 tiles, K/V in a contiguous cache) and its output transpose
// (src/runtime/layout.cu:11-42).  Same numerics contract: bf16 operands, fp32
// scores scaled after the dot product, base-2 online softmax, row sum of the
// un-rounded probabilities, probabilities rounded to bf16 for P*V, O / sum
// rounded to bf16; a query at position p sees keys 0..p.
//
// One work item = 128 query rows of one query head (UMMA M = 128), walking
// 128-key tiles of the cache up to the diagonal; persistent CTAs (two per SM)
// draw items from a counter, heaviest query tiles first.
//   warp 8      loader: per tile 8 K tiles + 8 V tiles (2 KiB each, one cache
//               block each) fetched through the block table with cp.async.bulk
//               into a 3-stage ring.  The cache stores every tile already in
//               the 128-byte swizzle, so the copies land as canonical UMMA
//               operands: K as K-major, V as MN-major.
//   warp 9      issues the MMAs: S = Q K^T (M128 N128 K64 -> TMEM columns
//               0..127) and O += P V (M128 N64 K128 -> TMEM columns 128..191, P
//               read from TMEM columns 192..255); one elected lane issues them;
//               completion is signalled to the other warps with tcgen05.commit.
//   warps 0-7   softmax: S is read with tcgen05.ld in the 16x256b layout (the
//               mma accumulator layout: a row is spread over the 4 threads of
//               a quad, 16 TMEM lanes per warp), so row maxima and sums are
//               quad shuffles and each thread carries only 64 scores; P (bf16)
//               goes back to tensor memory (tcgen05.st 16x128b, two scores per
//               column) as the A operand of the second MMA, so it never
//               touches shared memory; O is rescaled in TMEM only when a row
//               maximum moved by more than 2^8; finally O / sum is written as
//               bf16 straight into the [tokens, heads*64] layout.
// Every wait is bounded; a wait that runs out raises the CTA's abort flag,
// records PA_ERR_TIMEOUT in the status word, and all warps fall through to the
// common exit, where tensor memory is released.
#include "kernels.cuh"
#include "tc05.cuh"

namespace pa {

namespace {

constexpr int kBM = 128;            // query rows per CTA
constexpr int kBN = 128;            // keys per tile
constexpr int kStagesKV = 3;
constexpr int kQBytes = kBM * 128;          // 16 KiB
constexpr int kKBytes = kBN * 128;          // 16 KiB
constexpr int kVBytes = kBN * 128;          // 16 KiB
constexpr int kOffQ = 0;
constexpr int kOffKV = kOffQ + kQBytes;
constexpr int kOffBar = kOffKV + kStagesKV * (kKBytes + kVBytes);
constexpr int kNumBars = 9 + 4 * kStagesKV;  // K and V halves of a stage fill and free separately
constexpr int kOffMisc = kOffBar + kNumBars * 8;  // tensor-memory base address, abort flag, 2 work items
constexpr int kPrefillUsed = kOffMisc + 16;
// Two CTAs per SM: 2 * (request + 1 KiB system reserve) must stay below 228 KiB,
// so there is no room for alignment slack.  The kernel declares no static
// shared memory, which puts the dynamic region at a 1024-byte aligned offset;
// it checks that at run time and refuses to run otherwise.
constexpr int kPrefillSmem = kPrefillUsed + 112;
static_assert(2 * (kPrefillSmem + 1024) <= 228 * 1024, "two CTAs per SM");
constexpr int kSoftmaxThreads = 256;  // warps 0..7
constexpr int kLoadWarp = 8, kMmaWarp = 9;
constexpr int kPrefillThreads = 320;
// S: 128 fp32 columns, O: 64 fp32 columns, P: 128 bf16 = 64 columns; power of two
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128, kColP = 192;
constexpr float kRescaleThreshold = 8.0f;  // log2: rescale O only if a row max moved by > 2^8


// ---- sm_100 scalar helpers: 3-input max and packed fp32x2 arithmetic -----------
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// exp2 of two values without the special-function unit (the busiest pipe of
// this kernel): n = round(x) through the 1.5*2^23 trick, 2^(x-n) by a degree-3
// polynomial on [-0.5, 0.5] (relative error 7.5e-5, far below the bf16 rounding
// of P), the exponent added into the bits.  Inputs are clamped to -126, so a
// masked score (-inf) gives 2^-126 instead of an exact zero.
// Measured on B200, 2048-token causal layer: 37.9 us with 1 group in 4 on this
// path, 39.3 us with 1 in 2, 40.7 us with none.
constexpr int kPolyEvery = 4;  // n > 0: 1 in n column groups (n = 1, 2 or 4) takes this path
__device__ __forceinline__ void exp2_poly_x2(float x0, float x1, float& p0, float& p1) {
  const uint64_t x = pack_f32x2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t magic = pack_f32x2(12582912.f, 12582912.f);
  const uint64_t t = add_f32x2(x, magic);
  const uint64_t n = add_f32x2(t, pack_f32x2(-12582912.f, -12582912.f));
  const uint64_t f = fma_f32x2(n, pack_f32x2(-1.f, -1.f), x);
  uint64_t q = fma_f32x2(f, pack_f32x2(0.055171460f, 0.055171460f), pack_f32x2(0.24261086f, 0.24261086f));
  q = fma_f32x2(q, f, pack_f32x2(0.69326097f, 0.69326097f));
  q = fma_f32x2(q, f, pack_f32x2(0.99992812f, 0.99992812f));
  float t0, t1, q0, q1;
  unpack_f32x2(t, t0, t1);
  unpack_f32x2(q, q0, q1);
  p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
  p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

// 16 lanes x (8 groups of 8 columns): thread t gets, for group i, registers
// 4i..4i+1 = (lane t/4, columns 8i + 2(t%4), +1) and 4i+2..4i+3 = the same
// columns of lane t/4 + 8 (measured on B200; the mma accumulator layout).
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x8.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 16 lanes x 64 columns: thread t gives, for column group j of 4, register 2j =
// (lane t/4, column 4j + t%4) and 2j+1 = the same column of lane t/4 + 8.  With
// two bf16 per column this is the accumulator layout of 128 scores packed in pairs.
__device__ __forceinline__ void tmem_st_16x128b_x16(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// One unit of work: 128 query rows of one head of one sequence.  Items are
// numbered so that drawing them in order takes the heaviest query tiles first.
struct PrefillItem {
  BatchEntry e;
  int z, h, row0, rows, pos0, n_tiles, n_blocks;
  bool valid;
};
__device__ __forceinline__ PrefillItem prefill_item(const PrefillParams& p, int w) {
  PrefillItem it;
  const int heads = p.kv_heads * kGroup;
  it.h = w % heads;
  const int y = (w / heads) % p.grid_y;
  it.z = w / (heads * p.grid_y);
  it.e = p.batch[it.z];
  const int n_q_tiles = (it.e.n_q + kBM - 1) / kBM;
  const int q_tile = n_q_tiles - 1 - y;
  it.valid = q_tile >= 0;  // the item space is sized for the sequence with the most query rows
  it.row0 = q_tile * kBM;
  it.rows = min(kBM, it.e.n_q - it.row0);
  it.pos0 = it.e.q_pos0 + it.row0;  // position of row 0
  // causal: a query at position p sees keys 0..p; otherwise every cached key
  const int last_pos = p.causal ? min(it.pos0 + it.rows - 1, it.e.kv_len - 1) : it.e.kv_len - 1;
  it.n_tiles = last_pos / kBN + 1;
  it.n_blocks = (it.e.kv_len + kBlockTok - 1) / kBlockTok;
  return it;
}

// Persistent CTAs (two per SM) draw items from a counter until none is left,
// so the SMs stay evenly loaded whatever the mix of 1..16-tile items, and a
// CTA's set-up (tensor-memory allocation, barriers) happens once.  The loader
// warp draws an item, publishes it to the other warps through a two-slot
// mailbox and starts on its K/V tiles at once — while the softmax warps are
// still in the previous item's epilogue.  Barrier phases and ring positions run
// on across items.
__global__ void __launch_bounds__(kPrefillThreads, 2)
prefill_kernel(PrefillParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {  // swizzle atoms need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(p.status, kStatusBadBlock);
    return;
  }
  unsigned char* sm = smem_raw;
  const uint32_t sQ = base + kOffQ, sKV = base + kOffKV;
  const uint32_t bar0 = base + kOffBar;
  const uint32_t bar_q = bar0, bar_s = bar0 + 8, bar_p = bar0 + 16, bar_pv = bar0 + 24;
  const uint32_t bar_sfree = bar0 + 32;
  const uint32_t bar_kfull = bar0 + 40, bar_kempty = bar_kfull + 8 * kStagesKV;
  const uint32_t bar_vfull = bar_kempty + 8 * kStagesKV, bar_vempty = bar_vfull + 8 * kStagesKV;
  const uint32_t bar_item_full = bar_vempty + 8 * kStagesKV;  // [2]: the loader has published an item
  const uint32_t bar_item_empty = bar_item_full + 16;         // [2]: every other warp has read it
  uint32_t* s_tmem_base = reinterpret_cast<uint32_t*>(sm + kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kOffMisc + 4);
  volatile int* s_item = reinterpret_cast<volatile int*>(sm + kOffMisc + 8);  // [2]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    *abort_flag = 0;
    if (blockIdx.x == 0) *p.work_clear = 0;  // the counter of a launch far from this one
    for (int s = 0; s < 2; s++) {
      mbar_init(bar_item_full + 8 * s, 1);
      mbar_init(bar_item_empty + 8 * s, 1 + kSoftmaxThreads / 32);
    }
    // the softmax warps arrive once per warp (lane 0 after a warp barrier): 256
    // arrivals on one shared-memory word serialise and cost more than the tile's math
    mbar_init(bar_q, kSoftmaxThreads / 32);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, kSoftmaxThreads / 32);
    mbar_init(bar_pv, 1);
    mbar_init(bar_sfree, kSoftmaxThreads / 32);
    for (int s = 0; s < kStagesKV; s++) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, 1);
    }
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(base + kOffMisc, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem_base;

  if (warp == kLoadWarp) {
    // ===================== loader ============================================
    uint32_t k_cnt = 0, v_cnt = 0;  // tiles put into the K and V rings so far
    bool ok = true;
    for (int it = 0; ok; it++) {
    const int slot = it & 1;
    if (!wait_or_abort(bar_item_empty + 8 * slot, (uint32_t)(((it >> 1) & 1) ^ 1), abort_flag)) break;
    int w = 0;
    if (lane == 0) {
      w = atomicAdd(p.work, 1);
      if (w >= p.n_items) w = -1;
      s_item[slot] = w;
      mbar_arrive(bar_item_full + 8 * slot);
    }
    w = __shfl_sync(0xffffffffu, w, 0);
    if (w < 0) break;
    const PrefillItem item = prefill_item(p, w);
    if (!item.valid) continue;
    const BatchEntry e = item.e;
    const int h = item.h, n_tiles = item.n_tiles, n_blocks = item.n_blocks;
    const int32_t* table = p.tables + (size_t)e.seq * p.max_blocks_per_seq;
    const int hk = h / kGroup;
    // K halves are released right after Q K^T, V halves after P V, so the two
    // streams advance independently: one polling loop serves whichever half
    // is free.  Lanes 0..7 copy the 8 blocks of a tile; the block ids of the
    // next tile are fetched before the wait, off the critical path.
    auto block_of = [&](int kt) {
      // blocks past the end of the sequence re-read its last block: finite
      // data whose keys are masked, never uninitialised shared memory
      int blk = lane < 8 ? table[min(kt * (kBN / kBlockTok) + lane, n_blocks - 1)] : 0;
      if (blk < 0 || blk >= p.num_blocks) {
        atomicExch(p.status, kStatusBadBlock);
        blk = 0;
      }
      return blk;
    };
    int k_next = 0, v_next = 0;
    int blk_k = block_of(0), blk_v = blk_k;
    SpinDeadline dl;
    while (ok && (k_next < n_tiles || v_next < n_tiles)) {
      bool progressed = false;
      if (k_next < n_tiles) {
        const uint32_t ring = k_cnt + (uint32_t)k_next;
        const int st = (int)(ring % kStagesKV);
        if (__all_sync(0xffffffffu, mbar_test(bar_kempty + 8 * st, ((ring / kStagesKV) & 1u) ^ 1u))) {
          if (lane == 0) mbar_expect_tx(bar_kfull + 8 * st, kKBytes);
          __syncwarp();
          if (lane < 8)
            bulk_g2s(sKV + st * (kKBytes + kVBytes) + lane * kTileBytes,
                     p.storage + tile_off(blk_k, p.kv_heads, hk, 0), kTileBytes, bar_kfull + 8 * st);
          k_next++;
          if (k_next < n_tiles) blk_k = block_of(k_next);
          progressed = true;
        }
      }
      if (v_next < n_tiles) {
        const uint32_t ring = v_cnt + (uint32_t)v_next;
        const int st = (int)(ring % kStagesKV);
        if (__all_sync(0xffffffffu, mbar_test(bar_vempty + 8 * st, ((ring / kStagesKV) & 1u) ^ 1u))) {
          if (lane == 0) mbar_expect_tx(bar_vfull + 8 * st, kVBytes);
          __syncwarp();
          if (lane < 8)
            bulk_g2s(sKV + st * (kKBytes + kVBytes) + kKBytes + lane * kTileBytes,
                     p.storage + tile_off(blk_v, p.kv_heads, hk, 1), kTileBytes, bar_vfull + 8 * st);
          v_next++;
          if (v_next < n_tiles) blk_v = block_of(v_next);
          progressed = true;
        }
      }
      if (progressed) {
        dl.restart();
      } else {
        const bool out_of_time = dl.expired();  // nothing freed for a second
        if ((dl.spins & 31u) == 0) {
          bool stop = *abort_flag != 0;
          if (!stop && out_of_time) {
            *abort_flag = 1;
            stop = true;
          }
          if (__any_sync(0xffffffffu, stop)) ok = false;
        }
      }
    }
    k_cnt += (uint32_t)n_tiles;
    v_cnt += (uint32_t)n_tiles;
    }
  } else if (warp == kMmaWarp) {
    // ===================== MMA issue =========================================
    constexpr uint32_t kIdescQK = idesc_bf16(kBM, kBN, false);
    constexpr uint32_t kIdescPV = idesc_bf16(kBM, kHeadDim, true);
    uint32_t t_run = 0;  // tiles of all items so far: ring positions and barrier phases run on
    bool ok = true;
    int n_items_done = 0;
    for (int it = 0; ok; it++) {
    const int slot = it & 1;
    if (!wait_or_abort(bar_item_full + 8 * slot, (uint32_t)((it >> 1) & 1), abort_flag)) break;
    const int w = s_item[slot];
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_item_empty + 8 * slot);
    if (w < 0) break;
    const PrefillItem item = prefill_item(p, w);
    if (!item.valid) continue;
    const int n_tiles = item.n_tiles;
    // the softmax warps have read the previous item's last scores: S may be overwritten
    if (n_items_done > 0 && !wait_or_abort(bar_sfree, (t_run - 1u) & 1u, abort_flag)) break;
    ok = wait_or_abort(bar_q, (uint32_t)(n_items_done & 1), abort_flag);
    n_items_done++;
    auto issue_qk = [&](int kt) {
      const uint32_t ring = t_run + (uint32_t)kt;
      const int st = (int)(ring % kStagesKV);
      if (!wait_or_abort(bar_kfull + 8 * st, (ring / kStagesKV) & 1u, abort_flag)) return false;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t sK = sKV + st * (kKBytes + kVBytes);
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ks++)
          umma_ss(tmem + kColS, smem_desc_sw128(sQ + ks * 32), smem_desc_sw128(sK + ks * 32),
                  kIdescQK, ks > 0 ? 1u : 0u);
        tc_commit(bar_s);
        tc_commit(bar_kempty + 8 * st);  // this stage's K half may be refilled
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int kt = 0; ok && kt < n_tiles; kt++) {
      const uint32_t ring = t_run + (uint32_t)kt;
      const int st = (int)(ring % kStagesKV);
      // S(kt) is in the softmax threads' registers: the next Q K^T may overwrite it
      if (kt + 1 < n_tiles) {
        if (!wait_or_abort(bar_sfree, ring & 1u, abort_flag)) { ok = false; break; }
        if (!issue_qk(kt + 1)) { ok = false; break; }
      }
      if (!wait_or_abort(bar_p, ring & 1u, abort_flag)) { ok = false; break; }
      if (!wait_or_abort(bar_vfull + 8 * st, (ring / kStagesKV) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      if (elect_one()) {
        const uint32_t sV = sKV + st * (kKBytes + kVBytes) + kKBytes;
#pragma unroll
        for (int kk = 0; kk < kBN / 16; kk++)
          umma_ts(tmem + kColO, tmem + kColP + kk * 8, smem_desc_sw128(sV + kk * kTileBytes), kIdescPV,
                  (kt > 0 || kk > 0) ? 1u : 0u);
        tc_commit(bar_pv);
        tc_commit(bar_vempty + 8 * st);
      }
      __syncwarp();
    }
    t_run += (uint32_t)n_tiles;
    }
  } else {
    // ===================== softmax / epilogue ==================================
    // Warp w works on TMEM lanes [32*(w&3) + 16*(w>>2), +16) in the 16x256b
    // register layout (the mma accumulator layout): thread t holds rows
    // rA = first + t/4 and rB = rA + 8, and of every group of 8 columns the two
    // at 2*(t%4).  A row is spread over the 4 threads of a quad, so row maxima
    // and sums are quad shuffles, and P goes back to tensor memory (tcgen05.st) in the same layout.
    const int first_row = (warp & 3) * 32 + (warp >> 2) * 16;
    const uint32_t lane_base = (uint32_t)first_row << 16;
    const int rA = first_row + (lane >> 2), rB = rA + 8;
    const int cq = (lane & 3) * 2;
    uint32_t t_run = 0;
    int n_items_done = 0;
    bool ok = true;
    for (int it = 0; ok; it++) {
    const int slot = it & 1;
    if (!wait_or_abort(bar_item_full + 8 * slot, (uint32_t)((it >> 1) & 1), abort_flag)) break;
    const int w = s_item[slot];
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_item_empty + 8 * slot);
    if (w < 0) break;
    const PrefillItem item = prefill_item(p, w);
    if (!item.valid) continue;
    const BatchEntry e = item.e;
    const int z = item.z, h = item.h, row0 = item.row0, rows = item.rows, pos0 = item.pos0, n_tiles = item.n_tiles;
    n_items_done++;
    // Q tile -> shared memory (K-major, swizzled): thread = (row, half row).  Every
    // Q K^T of the previous item is complete: this thread has seen its last scores.
    {
      const int r = tid >> 1, c0 = (tid & 1) * 4;
      uint4 v[4];
      if (r < rows) {
        const uint4* src = reinterpret_cast<const uint4*>(
            p.q + (size_t)z * p.q_seq_stride + (size_t)(e.q_row_off + row0 + r) * p.q_row_stride +
            (size_t)h * p.q_head_stride);
#pragma unroll
        for (int c = 0; c < 4; c++) v[c] = src[c0 + c];
      } else {
#pragma unroll
        for (int c = 0; c < 4; c++) v[c] = make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int c = 0; c < 4; c++)
        *reinterpret_cast<uint4*>(sm + kOffQ + r * 128 + (((c0 + c) ^ (r & 7)) << 4)) = v[c];
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_q);
    }

    const int qposA = pos0 + rA, qposB = pos0 + rB;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
    for (int kt = 0; kt < n_tiles; kt++) {
      if (!wait_or_abort(bar_s, (t_run + (uint32_t)kt) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int key0 = kt * kBN;
      const bool need_mask = (p.causal && key0 + kBN - 1 > pos0) || (key0 + kBN > e.kv_len);

      // S -> registers (both column halves in flight, one wait); the tensor
      // memory copy is then free for the next tile's Q K^T
      uint32_t s[2][32];
      tmem_ld_16x256b_x8(tmem + lane_base + kColS, s[0]);
      tmem_ld_16x256b_x8(tmem + lane_base + kColS + 64, s[1]);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sfree);

      if (need_mask) {
        const int limA = (p.causal ? min(qposA, e.kv_len - 1) : e.kv_len - 1) - key0;  // keys <= lim are visible
        const int limB = (p.causal ? min(qposB, e.kv_len - 1) : e.kv_len - 1) - key0;
#pragma unroll
        for (int hf = 0; hf < 2; hf++)
#pragma unroll
          for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int col = hf * 64 + i * 8 + cq + (j & 1);
              if (col > ((j & 2) ? limB : limA)) s[hf][4 * i + j] = 0xff800000u;  // -inf
            }
      }
      // row maxima of the raw scores (the scale is positive): two chains per row
      float mxA, mxB;
      {
        float a0 = -INFINITY, a1 = -INFINITY, b0 = -INFINITY, b1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          a0 = max3(a0, __uint_as_float(s[0][4 * i]), __uint_as_float(s[0][4 * i + 1]));
          a1 = max3(a1, __uint_as_float(s[1][4 * i]), __uint_as_float(s[1][4 * i + 1]));
          b0 = max3(b0, __uint_as_float(s[0][4 * i + 2]), __uint_as_float(s[0][4 * i + 3]));
          b1 = max3(b1, __uint_as_float(s[1][4 * i + 2]), __uint_as_float(s[1][4 * i + 3]));
        }
        mxA = fmaxf(a0, a1);
        mxB = fmaxf(b0, b1);
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2)) * p.scale_log2;
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2)) * p.scale_log2;
      }
      // lazy rescale: keep the old reference maximum unless it is off by > 2^8
      float corrA = 1.f, corrB = 1.f;
      if (mxA > mA + kRescaleThreshold) {
        corrA = ex2(mA - mxA);  // 0 on the first tile
        mA = mxA;
      }
      if (mxB > mB + kRescaleThreshold) {
        corrB = ex2(mB - mxB);
        mB = mxB;
      }
      const bool any_corr = __any_sync(0xffffffffu, corrA != 1.f || corrB != 1.f);

      // probabilities -> bf16 in registers: the exponentials (the bulk of the
      // work) run while the previous tile's P V is still in the tensor pipe
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
      const uint64_t negA2 = pack_f32x2(-mA, -mA), negB2 = pack_f32x2(-mB, -mB);
      uint64_t laccA = 0ull, laccB = 0ull;
      uint32_t pk[32];  // register 2j: row A, 2j+1: row B of packed column 4j + lane%4
#pragma unroll
      for (int hf = 0; hf < 2; hf++)
#pragma unroll
        for (int i = 0; i < 8; i++) {
          float x0, x1, y0, y1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[hf][4 * i]), __uint_as_float(s[hf][4 * i + 1])),
                                 scale2, negA2), x0, x1);
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[hf][4 * i + 2]), __uint_as_float(s[hf][4 * i + 3])),
                                 scale2, negB2), y0, y1);
          float p0, p1, p2, p3;
          if ((i & 3) == kPolyEvery - 1 && kPolyEvery > 0) {
            // every kPolyEvery-th column group: exp2 on the FMA pipes instead of the MUFU
            exp2_poly_x2(x0, x1, p0, p1);
            exp2_poly_x2(y0, y1, p2, p3);
          } else {
            p0 = ex2(x0);
            p1 = ex2(x1);
            p2 = ex2(y0);
            p3 = ex2(y1);
          }
          laccA = add_f32x2(laccA, pack_f32x2(p0, p1));
          laccB = add_f32x2(laccB, pack_f32x2(p2, p3));
          pk[2 * (hf * 8 + i)] = pack_bf16(p0, p1);
          pk[2 * (hf * 8 + i) + 1] = pack_bf16(p2, p3);
        }

      // P of the previous tile must have been consumed, O must be quiescent
      if (kt > 0) {
        if (!wait_or_abort(bar_pv, (t_run + (uint32_t)kt - 1u) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (any_corr) {
          uint32_t o[32];
          tmem_ld_16x256b_x8(tmem + lane_base + kColO, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; i++) {
            o[4 * i] = __float_as_uint(__uint_as_float(o[4 * i]) * corrA);
            o[4 * i + 1] = __float_as_uint(__uint_as_float(o[4 * i + 1]) * corrA);
            o[4 * i + 2] = __float_as_uint(__uint_as_float(o[4 * i + 2]) * corrB);
            o[4 * i + 3] = __float_as_uint(__uint_as_float(o[4 * i + 3]) * corrB);
          }
          tmem_st_16x256b_x8(tmem + lane_base + kColO, o);
          tmem_wait_st();
        }
      }
      {
        float a0, a1, b0, b1;
        unpack_f32x2(laccA, a0, a1);
        unpack_f32x2(laccB, b0, b1);
        lA = lA * corrA + (a0 + a1);
        lB = lB * corrB + (b0 + b1);
      }

      // P -> tensor memory, the A operand of the second MMA
      tmem_st_16x128b_x16(tmem + lane_base + kColP, pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
    }

    // epilogue: O / sum -> bf16, [tokens, heads*64] layout (or the caller's strides)
    if (ok) ok = wait_or_abort(bar_pv, (t_run + (uint32_t)n_tiles - 1u) & 1u, abort_flag);
    if (ok) {
      tc_fence_after();
      lA += __shfl_xor_sync(0xffffffffu, lA, 1);
      lB += __shfl_xor_sync(0xffffffffu, lB, 1);
      lA += __shfl_xor_sync(0xffffffffu, lA, 2);
      lB += __shfl_xor_sync(0xffffffffu, lB, 2);
      const float invA = lA > 0.f ? 1.f / lA : 0.f, invB = lB > 0.f ? 1.f / lB : 0.f;
      uint32_t o[32];
      tmem_ld_16x256b_x8(tmem + lane_base + kColO, o);
      tmem_wait_ld();
      __nv_bfloat16* obase = p.out + (size_t)z * p.o_seq_stride + (size_t)h * p.o_head_stride + cq;
      if (rA < rows) {
        __nv_bfloat16* orow = obase + (size_t)(e.q_row_off + row0 + rA) * p.o_row_stride;
#pragma unroll
        for (int i = 0; i < 8; i++)
          *reinterpret_cast<uint32_t*>(orow + 8 * i) =
              pack_bf16(__uint_as_float(o[4 * i]) * invA, __uint_as_float(o[4 * i + 1]) * invA);
      }
      if (rB < rows) {
        __nv_bfloat16* orow = obase + (size_t)(e.q_row_off + row0 + rB) * p.o_row_stride;
#pragma unroll
        for (int i = 0; i < 8; i++)
          *reinterpret_cast<uint32_t*>(orow + 8 * i) =
              pack_bf16(__uint_as_float(o[4 * i + 2]) * invB, __uint_as_float(o[4 * i + 3]) * invB);
      }
      if (p.lse && (lane & 3) == 0) {
        float* lrow = p.lse + (size_t)z * p.lse_seq_stride + (size_t)h * e.n_q + row0;
        if (rA < rows) lrow[rA] = lA > 0.f ? kLn2 * (mA + log2f(lA)) : -INFINITY;
        if (rB < rows) lrow[rB] = lB > 0.f ? kLn2 * (mB + log2f(lB)) : -INFINITY;
      }
    }
    t_run += (uint32_t)n_tiles;
    }
  }

  // ---- common exit: release tensor memory -----------------------------------
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.status, kStatusTimeout);
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

cudaError_t launch_prefill(const PrefillParams& p, int n_seqs, int n_q, cudaStream_t stream) {
  if (n_q <= 0 || n_seqs <= 0) return cudaSuccess;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kPrefillSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  static int sm_count[64] = {};
  if (dev >= 0 && dev < 64 && sm_count[dev] == 0)
    cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  const int sms = (dev >= 0 && dev < 64 && sm_count[dev] > 0) ? sm_count[dev] : 148;
  PrefillParams q = p;
  q.grid_y = (n_q + kBM - 1) / kBM;
  q.n_items = p.kv_heads * kGroup * q.grid_y * n_seqs;
  const int ctas = q.n_items < 2 * sms ? q.n_items : 2 * sms;  // two CTAs per SM stay resident
  prefill_kernel<<<ctas, kPrefillThreads, kPrefillSmem, stream>>>(q);
  return cudaGetLastError();
}

}  // namespace pa
