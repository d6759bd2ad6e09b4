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
// One CTA = 128 query rows of one query head (UMMA M = 128), walking 128-key
// tiles of the cache up to the diagonal.
//   warp 4      loader: per tile 8 K tiles + 8 V tiles (2 KiB each, one cache
//               block each) fetched through the block table with cp.async.bulk
//               into a 2-stage ring.  The cache stores every tile already in
//               the 128-byte swizzle, so the copies land as canonical UMMA
//               operands: K as K-major, V as MN-major.
//   warp 5      issues the MMAs: S = Q K^T (M128 N128 K64 -> TMEM columns
//               0..127) and O += P V (M128 N64 K128 -> TMEM columns 128..191);
//               completion is signalled to the other warps with tcgen05.commit.
//   warps 0-3   softmax: thread r owns query row r = TMEM lane r; reads S with
//               tcgen05.ld, writes P (bf16) into shared memory in K-major
//               swizzled layout for the second MMA, rescales O in TMEM only
//               when a row maximum moved by more than 2^8, and finally writes
//               O / sum as bf16 straight into the [tokens, heads*64] layout.
// Every wait is bounded; a wait that runs out raises the CTA's abort flag,
// records PA_ERR_TIMEOUT in the status word, and all warps fall through to the
// common exit, where tensor memory is released.
#include "kernels.cuh"

namespace pa {

namespace {

constexpr int kBM = 128;            // query rows per CTA
constexpr int kBN = 128;            // keys per tile
constexpr int kStagesKV = 2;
constexpr int kQBytes = kBM * 128;          // 16 KiB
constexpr int kKBytes = kBN * 128;          // 16 KiB
constexpr int kVBytes = kBN * 128;          // 16 KiB
constexpr int kPBytes = kBM * kBN * 2;      // 32 KiB (two 64-key halves)
constexpr int kOffQ = 0;
constexpr int kOffKV = kOffQ + kQBytes;
constexpr int kOffP = kOffKV + kStagesKV * (kKBytes + kVBytes);
constexpr int kOffBar = kOffP + kPBytes;
constexpr int kNumBars = 5 + 2 * kStagesKV;
constexpr int kOffMisc = kOffBar + kNumBars * 8;  // tensor-memory base address, abort flag
constexpr int kPrefillUsed = kOffMisc + 16;
// Two CTAs per SM: 2 * (request + 1 KiB system reserve) must stay below 228 KiB,
// so there is no room for alignment slack.  The kernel declares no static
// shared memory, which puts the dynamic region at a 1024-byte aligned offset;
// it checks that at run time and refuses to run otherwise.
constexpr int kPrefillSmem = kPrefillUsed + 112;
static_assert(2 * (kPrefillSmem + 1024) <= 228 * 1024, "two CTAs per SM");
constexpr int kPrefillThreads = 192;
constexpr uint32_t kTmemCols = 256;  // S: 128 columns, O: 64 columns, power of two
constexpr uint32_t kColS = 0, kColO = 128;
constexpr float kRescaleThreshold = 8.0f;  // log2: rescale O only if a row max moved by > 2^8

// ---- tcgen05 wrappers ---------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

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

// Shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes
// apart (version 1 = Blackwell, layout type 2 = SWIZZLE_128B).  The same
// encoding serves K-major operands (rows = M or N index, 128 bytes of K per
// row) and MN-major ones (rows = K index, 128 bytes of N per row).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);   // start address
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused with this swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                       // descriptor version
  d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
  return d;
}
// Instruction descriptor, kind::f16: D fp32, A/B bf16, A K-major.
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// mbarrier wait that also gives up when another warp raised the abort flag.
__device__ __forceinline__ bool wait_one(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  uint32_t spins = 0;
  while (!mbar_test(bar, parity)) {
    if ((++spins & 31u) == 0) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// Whole-warp form: every lane gets the same answer, so the warp stays converged
// for the .sync.aligned tcgen05 instructions that follow.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, wait_one(bar, parity, abort_flag));
}

__global__ void __launch_bounds__(kPrefillThreads, 2)
prefill_kernel(PrefillParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {  // swizzle atoms need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(p.status, kStatusBadBlock);
    return;
  }
  unsigned char* sm = smem_raw;
  const uint32_t sQ = base + kOffQ, sKV = base + kOffKV, sP = base + kOffP;
  const uint32_t bar0 = base + kOffBar;
  const uint32_t bar_q = bar0, bar_s = bar0 + 8, bar_p = bar0 + 16, bar_pv = bar0 + 24;
  const uint32_t bar_sfree = bar0 + 32;
  const uint32_t bar_full = bar0 + 40, bar_empty = bar_full + 8 * kStagesKV;
  uint32_t* s_tmem_base = reinterpret_cast<uint32_t*>(sm + kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kOffMisc + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int z = blockIdx.z;
  const BatchEntry e = p.batch[z];
  const int n_q_tiles = (e.n_q + kBM - 1) / kBM;
  // CTAs are dispatched in linear order (x fastest): all heads of the heaviest
  // query tile first, the lightest tiles last, so the tail of the grid is short
  const int q_tile = n_q_tiles - 1 - (int)blockIdx.y;
  const int h = blockIdx.x;
  if (q_tile < 0) return;  // the grid is sized for the sequence with the most query rows
  const int row0 = q_tile * kBM;
  const int rows = min(kBM, e.n_q - row0);
  const int pos0 = e.q_pos0 + row0;                            // position of row 0
  // causal: a query at position p sees keys 0..p; otherwise every cached key
  const int last_pos = p.causal ? min(pos0 + rows - 1, e.kv_len - 1) : e.kv_len - 1;
  const int n_tiles = last_pos / kBN + 1;
  const int n_blocks = (e.kv_len + kBlockTok - 1) / kBlockTok;
  const int q_heads = p.kv_heads * kGroup;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar_q, 128);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_pv, 1);
    mbar_init(bar_sfree, 128);
    for (int s = 0; s < kStagesKV; s++) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(base + kOffMisc, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem_base;

  if (warp == 4) {
    // ===================== loader ============================================
    const int32_t* table = p.tables + (size_t)e.seq * p.max_blocks_per_seq;
    const int hk = h / kGroup;
    for (int kt = 0; kt < n_tiles; kt++) {
      const int st = kt % kStagesKV;
      if (!wait_or_abort(bar_empty + 8 * st, (uint32_t)(((kt / kStagesKV) & 1) ^ 1), abort_flag)) break;
      if (lane == 0) mbar_expect_tx(bar_full + 8 * st, kKBytes + kVBytes);
      __syncwarp();
      if (lane < 16) {
        const int b = lane & 7, kv = lane >> 3;
        // blocks past the end of the sequence re-read its last block: finite
        // data whose keys are masked, never uninitialised shared memory
        int bi = min(kt * (kBN / kBlockTok) + b, n_blocks - 1);
        int blk = table[bi];
        if (blk < 0 || blk >= p.num_blocks) {
          atomicExch(p.status, kStatusBadBlock);
          blk = 0;
        }
        const char* src = p.storage + tile_off(blk, p.kv_heads, hk, kv);
        const uint32_t dst = sKV + st * (kKBytes + kVBytes) + kv * kKBytes + b * kTileBytes;
        bulk_g2s(dst, src, kTileBytes, bar_full + 8 * st);
      }
      __syncwarp();
    }
  } else if (warp == 5) {
    // ===================== MMA issue =========================================
    constexpr uint32_t kIdescQK = idesc_bf16(kBM, kBN, false);
    constexpr uint32_t kIdescPV = idesc_bf16(kBM, kHeadDim, true);
    bool ok = wait_or_abort(bar_q, 0, abort_flag);
    auto issue_qk = [&](int kt) {
      const int st = kt % kStagesKV;
      if (!wait_or_abort(bar_full + 8 * st, (uint32_t)((kt / kStagesKV) & 1), abort_flag)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t sK = sKV + st * (kKBytes + kVBytes);
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ks++)
          umma_ss(tmem + kColS, smem_desc_sw128(sQ + ks * 32), smem_desc_sw128(sK + ks * 32),
                  kIdescQK, ks > 0 ? 1u : 0u);
        tc_commit(bar_s);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int kt = 0; ok && kt < n_tiles; kt++) {
      const int st = kt % kStagesKV;
      // S(kt) is in the softmax threads' registers: the next Q K^T may overwrite it
      if (kt + 1 < n_tiles) {
        if (!wait_or_abort(bar_sfree, (uint32_t)(kt & 1), abort_flag)) break;
        if (!issue_qk(kt + 1)) break;
      }
      if (!wait_or_abort(bar_p, (uint32_t)(kt & 1), abort_flag)) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t sV = sKV + st * (kKBytes + kVBytes) + kKBytes;
#pragma unroll
        for (int kk = 0; kk < kBN / 16; kk++)
          umma_ss(tmem + kColO, smem_desc_sw128(sP + (kk >> 2) * (kBM * 128) + (kk & 3) * 32),
                  smem_desc_sw128(sV + kk * kTileBytes), kIdescPV, (kt > 0 || kk > 0) ? 1u : 0u);
        tc_commit(bar_pv);
        tc_commit(bar_empty + 8 * st);
      }
      __syncwarp();
    }
  } else {
    // ===================== softmax / epilogue (thread = query row) ===========
    const int r = tid;  // 0..127 = TMEM lane
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    // Q tile -> shared memory (K-major, swizzled); rows past the end are zero
    {
      uint4 v[8];
      if (r < rows) {
        const uint4* src = reinterpret_cast<const uint4*>(
            p.q + (size_t)z * p.q_seq_stride + (size_t)(e.q_row_off + row0 + r) * p.q_row_stride +
            (size_t)h * p.q_head_stride);
#pragma unroll
        for (int c = 0; c < 8; c++) v[c] = src[c];
      } else {
#pragma unroll
        for (int c = 0; c < 8; c++) v[c] = make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int c = 0; c < 8; c++)
        *reinterpret_cast<uint4*>(sm + kOffQ + r * 128 + ((c ^ (r & 7)) << 4)) = v[c];
      fence_proxy_async_smem();
      mbar_arrive(bar_q);
    }

    const int qpos = pos0 + r;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int kt = 0; kt < n_tiles; kt++) {
      if (!wait_or_abort(bar_s, (uint32_t)(kt & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int key0 = kt * kBN;
      const bool need_mask = (p.causal && key0 + kBN - 1 > pos0) || (key0 + kBN > e.kv_len);
      const int limit = (p.causal ? min(qpos, e.kv_len - 1) : e.kv_len - 1) - key0;  // keys <= limit are visible

      // S -> registers in one go (four loads in flight, one wait); the tensor
      // memory copy is then free for the next tile's Q K^T
      uint32_t sreg[4][32];
#pragma unroll
      for (int c = 0; c < 4; c++) tmem_ld32(tmem + lane_base + kColS + c * 32, sreg[c]);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar_sfree);

      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (c * 32 + j > limit) sreg[c][j] = 0xff800000u;  // -inf
      }
      // row maximum (raw scores; the scale is positive)
      // four independent chains of 3-input max
      float mxc[4];
#pragma unroll
      for (int c = 0; c < 4; c++) {
        mxc[c] = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          mxc[c] = max3(mxc[c], __uint_as_float(sreg[c][j]), __uint_as_float(sreg[c][j + 1]));
      }
      float mx = fmaxf(fmaxf(mxc[0], mxc[1]), fmaxf(mxc[2], mxc[3])) * p.scale_log2;
      // lazy rescale: keep the old reference maximum unless it is off by > 2^8
      float corr = 1.f;
      if (mx > m_used + kRescaleThreshold) {
        corr = ex2(m_used - mx);  // 0 on the first tile
        m_used = mx;
      }
      const bool any_corr = __any_sync(0xffffffffu, corr != 1.f);

      // probabilities -> bf16, kept in registers: the exponentials (the bulk of
      // the work) run while the previous tile's P V is still in the tensor pipe
      const float neg_m = -m_used;
      // packed fp32x2 arithmetic (two values per instruction) around the exp2
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
      const uint64_t negm2 = pack_f32x2(neg_m, neg_m);
      uint64_t lacc[4];
      uint32_t pk[4][16];
#pragma unroll
      for (int c = 0; c < 4; c++) {
        lacc[c] = 0ull;
#pragma unroll
        for (int u = 0; u < 16; u++) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sreg[c][2 * u]),
                                            __uint_as_float(sreg[c][2 * u + 1])), scale2, negm2), x0, x1);
          const float p0 = ex2(x0), p1 = ex2(x1);
          lacc[c] = add_f32x2(lacc[c], pack_f32x2(p0, p1));
          pk[c][u] = pack_bf16(p0, p1);
        }
      }
      float l_tile;
      {
        float a0, a1;
        unpack_f32x2(add_f32x2(add_f32x2(lacc[0], lacc[1]), add_f32x2(lacc[2], lacc[3])), a0, a1);
        l_tile = a0 + a1;
      }

      // P of the previous tile must have been consumed, O must be quiescent
      if (kt > 0) {
        if (!wait_or_abort(bar_pv, (uint32_t)((kt - 1) & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (any_corr) {
#pragma unroll 1
          for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
            uint32_t oreg[32];
            tmem_ld32(tmem + lane_base + kColO + c0, oreg);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j++) oreg[j] = __float_as_uint(__uint_as_float(oreg[j]) * corr);
            tmem_st32(tmem + lane_base + kColO + c0, oreg);
          }
          tmem_wait_st();
        }
      }
      l_sum = l_sum * corr + l_tile;

      // P -> shared memory (K-major, swizzled)
#pragma unroll
      for (int c = 0; c < 4; c++) {
        unsigned char* prow = sm + kOffP + (c >> 1) * (kBM * 128) + r * 128;
#pragma unroll
        for (int g = 0; g < 4; g++) {
          const int chunk = (c & 1) * 4 + g;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(pk[c][4 * g], pk[c][4 * g + 1], pk[c][4 * g + 2], pk[c][4 * g + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar_p);
    }

    // epilogue: O / sum -> bf16, [tokens, heads*64] layout
    if (ok && wait_or_abort(bar_pv, (uint32_t)((n_tiles - 1) & 1), abort_flag)) {
      tc_fence_after();
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = p.out + (size_t)z * p.o_seq_stride +
                            (size_t)(e.q_row_off + row0 + r) * p.o_row_stride + (size_t)h * p.o_head_stride;
#pragma unroll 1
      for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
        uint32_t oreg[32];
        tmem_ld32(tmem + lane_base + kColO + c0, oreg);
        tmem_wait_ld();
        if (r < rows) {
#pragma unroll
          for (int c = 0; c < 4; c++) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(oreg[8 * c + 0]) * inv, __uint_as_float(oreg[8 * c + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(oreg[8 * c + 2]) * inv, __uint_as_float(oreg[8 * c + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(oreg[8 * c + 4]) * inv, __uint_as_float(oreg[8 * c + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(oreg[8 * c + 6]) * inv, __uint_as_float(oreg[8 * c + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + 8 * c) = v;
          }
        }
      }
      if (p.lse && r < rows)
        p.lse[(size_t)z * p.lse_seq_stride + (size_t)h * e.n_q + row0 + r] = l_sum > 0.f ? kLn2 * (m_used + log2f(l_sum)) : -INFINITY;
    }
  }

  // ---- common exit: release tensor memory -----------------------------------
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.status, kStatusTimeout);
  if (warp == 5) {
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
  dim3 grid(p.kv_heads * kGroup, (n_q + kBM - 1) / kBM, n_seqs);
  prefill_kernel<<<grid, kPrefillThreads, kPrefillSmem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace pa
