// K2: paged split-KV GQA decode attention with an in-kernel log-sum-exp combine.
//
// Replaces the reference's use of its prefill kernel at q_seq_len == 1
// (src/kernels/flashattention/flashattention.cu:98-376 as launched from
// src/runtime/attention.cu:303-334: one CTA per query head walking the whole
// sequence, K/V read once per query head) and the separate output transpose
// (src/runtime/layout.cu:11-42).
//
// Decode is an HBM stream: 4 KiB (K tile + V tile of one block and KV head)
// per 16 tokens, read exactly once for the 4 query heads that share it.
//   * a CTA owns a contiguous run of blocks (a chunk) of one sequence's table
//     for one KV head; its WARPS consumer warps take the blocks round-robin;
//   * every consumer warp has its own ring of STAGES 4 KiB buffers.  A producer
//     warp fills them: its lane w waits for a stage of warp w to be handed back
//     (empty barrier) and issues the next bulk (TMA) copy, which completes on
//     the stage's full barrier.  Arming a barrier and issuing a bulk copy costs
//     a thread about 300 cycles — a quarter of a tile's time when the consumers
//     did it themselves.  WARPS*STAGES*4 KiB are in flight per CTA and no
//     CTA-wide barrier sits in the loop;
//   * tiles land in shared memory exactly as stored (rows of 128 bytes, chunks
//     XOR-swizzled), which ldmatrix reads without bank conflicts;
//   * the 4 query heads are rows 0..3 of an m16n8k16 A fragment (rows 4..15
//     zero); scores and P*V use mma.sync, softmax is done on the accumulator
//     fragments with quad shuffles, base 2, fp32 (numerics of the reference
//     kernel: scale after the dot product, sum of un-rounded probabilities,
//     probabilities rounded to bf16 for P*V, flashattention.cu:249-336);
//   * warps merge through shared memory; chunks merge through a workspace.  In
//     the kernel of one layer (decode_kernel) the last CTA to take a ticket for
//     a (sequence, KV head) combines and writes the [tokens, 2048]-layout row;
//   * a multi-layer decode step is ONE cooperative launch (decode_step_kernel):
//     the streaming CTAs go from layer to layer as one flat stream of tiles,
//     1, 2 or 4 extra CTAs per (sequence, KV head) combine (and, across GPUs,
//     exchange and merge) the layers behind them.
#include "kernels.cuh"
#include "rope.cuh"

namespace pa {

namespace {

template <int WARPS, int STAGES>
struct DecodeSmem {
  static constexpr int kTiles = WARPS * STAGES * kPairBytes;
  static constexpr int kBars = WARPS * STAGES * 8;
  static constexpr int kMergeFloats = WARPS * (kGroup * kHeadDim + 2 * kGroup);
  static constexpr int kBytes = 128 + kTiles + kBars + kMergeFloats * 4 + 16;
  // the step kernel appends: "stage free" barriers + the publisher's word, the CTA's slice of
  // the block table (entries beyond kStepTblCap are read from global memory), and every layer's
  // rotated query rows [layers][4][64] bf16
  static constexpr int kStepTblCap = 1024;
  static constexpr int kStepEmpty = (kTiles + kBars + kMergeFloats * 4 + 16 + 127) & ~127;
  static constexpr int kStepTbl = kStepEmpty + ((kBars + 8 + 127) & ~127);
  static constexpr int kStepQ = kStepTbl + kStepTblCap * 4;
  static constexpr int step_bytes(int layers) { return 128 + kStepQ + layers * kGroup * kHeadDim * 2; }
  // the kernel of one layer in its cluster form: behind the one layer's query rows, the partials
  // (O [4][64], m [4], l [4]) of up to 16 chunks, pushed into the cluster's first CTA by its peers
  static constexpr int kClusterPartFloats = kGroup * kHeadDim + 2 * kGroup;
  static constexpr int kClusterParts = ((kStepQ + kGroup * kHeadDim * 2 + 15) & ~15) + 16;  // 16 bytes in front: the chunk count
  static constexpr int one_layer_bytes() { return 128 + kClusterParts + 16 * kClusterPartFloats * 4; }
  static constexpr int kStepThreads = (WARPS + 2) * 32;  // consumers + producer warp + publisher warp
};

// Barrier among the first `threads` threads of the CTA (the consumer warps); the producer and
// publisher warps of a streaming CTA never take part, so __syncthreads is not used past set-up.
__device__ __forceinline__ void consumer_sync(int threads) {
  asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

// Store into the shared memory of CTA `rank` of the cluster, at the address `local` has in this CTA.
__device__ __forceinline__ void st_cluster_f32(const float* local, uint32_t rank, float v) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}

// One 8-byte word {value, step number}: value in the low half, step number in the high half,
// moved by ONE scalar 64-bit access, which the ISA makes single-copy atomic (a vector access is a
// set of scalar accesses that may formally be seen in parts).
__device__ __forceinline__ void st_word_sys(unsigned long long* p, float v, unsigned int seq) {
  const unsigned long long w = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ld_word_sys(const unsigned long long* p, float& v, unsigned int& seq) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  v = __uint_as_float((unsigned int)(w & 0xffffffffull));
  seq = (unsigned int)(w >> 32);
}

__device__ __forceinline__ void write_row_outputs(const DecodeParams& p, int z, int h, int r, int d,
                                                  float o, float m, float l) {
  const int q_heads = p.kv_heads * kGroup;
  const int head = h * kGroup + r;
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const float v = o * inv;
  if (p.out) p.out[(size_t)z * p.out_stride + head * kHeadDim + d] = __float2bfloat16_rn(v);
  if (p.out_f32) p.out_f32[((size_t)z * q_heads + head) * kHeadDim + d] = v;
  if (p.lse && d == 0)
    p.lse[(size_t)z * q_heads + head] = l > 0.f ? kLn2 * (m + log2f(l)) : -INFINITY;
  if (p.hs_world > 0) {
    // KV-head sharding: the all-gather of head outputs is these peer stores
    const __nv_bfloat16 b = __float2bfloat16_rn(v);
    const size_t at = (size_t)z * p.hs_stride + p.hs_col0 + head * kHeadDim + d;
    for (int g = 0; g < p.hs_world; g++) p.hs_rows[g][at] = b;
  }
  if (p.xchg_world > 0) {
    // sequence-range sharding: push this rank's normalised partial and its LSE
    // into every rank's receive buffer (plain peer stores over NVLink; each
    // rank later reads only its own memory)
    const int row = z * q_heads + head;
    const size_t at = ((size_t)(p.xchg_slot * p.xchg_world + p.xchg_rank) * p.xchg_rows + row) * kXchgRowFloats;
    const float lse = l > 0.f ? kLn2 * (m + log2f(l)) : -INFINITY;
    if (p.xchg_out) {
      // merged in this kernel: {value, step number} words, valid on arrival; the word region has
      // kXchgWordSlots slots (step number modulo that)
      const size_t atw = ((size_t)((p.xchg_seq & (kXchgWordSlots - 1u)) * p.xchg_world + p.xchg_rank) * p.xchg_rows + row) * kXchgRowFloats;
      for (int g = 0; g < p.xchg_world; g++) {
        st_word_sys(p.xchg_ll[g] + atw + d, v, p.xchg_seq);
        if (d == 0) st_word_sys(p.xchg_ll[g] + atw + kHeadDim, lse, p.xchg_seq);
      }
    } else {
      for (int g = 0; g < p.xchg_world; g++) {
        p.xchg_peer[g][at + d] = v;
        if (d == 0) p.xchg_peer[g][at + kHeadDim] = lse;
      }
    }
  }
}

// After a (sequence, KV head) group's rows have been pushed: make them visible
// system-wide, then publish the step number in every rank's flag for this
// source rank and head.  Called by all `nthreads` consumer threads of the CTA.
__device__ __forceinline__ void publish_exchange(const DecodeParams& p, int z, int h, int nthreads) {
  if (p.hs_world > 0) {
    // rows of this (sequence, KV head) are stored everywhere: count one arrival
    // per rank, released at system scope after the CTA's stores
    consumer_sync(nthreads);
    if ((int)threadIdx.x < p.hs_world) {
      __threadfence_system();
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.hs_counter[threadIdx.x]) : "memory");
    }
  }
  if (p.xchg_world <= 0 || p.xchg_out) return;  // words carry their own step number
  // the CTA barrier orders every thread's peer stores before the publishing
  // threads' system-scope fence, which is cumulative: one fence per flag
  // instead of one per thread
  consumer_sync(nthreads);
  if ((int)threadIdx.x < p.xchg_world) {
    __threadfence_system();
    unsigned int* flag = p.xchg_flag[threadIdx.x] + ((size_t)p.xchg_rank * p.xchg_groups + z * p.kv_heads + h);
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(p.xchg_seq) : "memory");
  }
}

// In-kernel merge of a sharded decode: the CTA that has just published this
// rank's partial of (sequence z, KV head h) waits — bounded — until every
// rank's partial of that group has landed in THIS rank's buffer, merges the
// group's 4 rows from local memory and writes them as bf16.
__device__ __forceinline__ void exchange_wait_merge(const DecodeParams& p, int z, int h, int* s_flag, int nthreads) {
  if (p.xchg_world <= 0 || !p.xchg_out) return;
  if (threadIdx.x == 0) *s_flag = 1;
  consumer_sync(nthreads);
  const int q_heads = p.kv_heads * kGroup;
  const unsigned long long* base =
      p.xchg_ll[p.xchg_rank] + (size_t)(p.xchg_seq & (kXchgWordSlots - 1u)) * p.xchg_world * p.xchg_rows * kXchgRowFloats;
  for (int idx = threadIdx.x; idx < kGroup * kHeadDim; idx += nthreads) {
    const int r = idx >> 6, d = idx & 63;
    const int head = h * kGroup + r;
    const int row = z * q_heads + head;
    // every rank's LSE and value d of this row: all still-missing words are loaded in one go (the
    // loads overlap), then checked; a word is valid once it carries this step's number
    float lse[8], val[8];
    bool ok = true;
    unsigned int need_l = (1u << p.xchg_world) - 1u, need_v = need_l;
    SpinDeadline dl;
    while (need_l | need_v) {
      float tl[8], tv[8];
      unsigned int sl[8], sv[8];
#pragma unroll
      for (int g = 0; g < 8; g++) {
        if (g >= p.xchg_world) continue;
        const unsigned long long* rowp = base + ((size_t)g * p.xchg_rows + row) * kXchgRowFloats;
        if ((need_l >> g) & 1u) ld_word_sys(rowp + kHeadDim, tl[g], sl[g]);
        if ((need_v >> g) & 1u) ld_word_sys(rowp + d, tv[g], sv[g]);
      }
#pragma unroll
      for (int g = 0; g < 8; g++) {
        if (g >= p.xchg_world) continue;
        if (((need_l >> g) & 1u) && sl[g] == p.xchg_seq) {
          lse[g] = tl[g];
          need_l &= ~(1u << g);
        }
        if (((need_v >> g) & 1u) && sv[g] == p.xchg_seq) {
          val[g] = tv[g];
          need_v &= ~(1u << g);
        }
      }
      if ((need_l | need_v) && dl.expired()) {
        ok = false;
        break;
      }
    }
    if (!ok) {
      *s_flag = 0;
      continue;
    }
    float M = -INFINITY;
#pragma unroll
    for (int g = 0; g < 8; g++)
      if (g < p.xchg_world) M = fmaxf(M, lse[g]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int g = 0; g < 8; g++) {
        if (g >= p.xchg_world) continue;
        const float w = lse[g] == -INFINITY ? 0.f : __expf(lse[g] - M);
        L += w;
        O += w * val[g];
      }
    }
    p.xchg_out[(size_t)z * p.xchg_out_stride + head * kHeadDim + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
  }
  consumer_sync(nthreads);
  if (!*s_flag && threadIdx.x == 0) atomicExch(p.status, kStatusTimeout);
}

template <int WARPS, int STAGES>
__device__ __forceinline__ void combine_pair(const DecodeParams& p, const int z, const int h, const int n_chunks,
                                             unsigned char* smem, int* s_wait_ok_p);

// Parameters of layer l of a persistent step: every per-layer pointer advanced.
__device__ __forceinline__ DecodeParams step_layer_params(const DecodeStepParams& sp, int l) {
  DecodeParams p = sp.base;
  p.q += (size_t)l * sp.q_layer_stride;
  if (p.k_new) p.k_new += (size_t)l * sp.kv_layer_stride;
  if (p.v_new) p.v_new += (size_t)l * sp.kv_layer_stride;
  if (p.q_rot_out) p.q_rot_out += (size_t)l * sp.q_layer_stride;
  p.storage += (size_t)l * sp.layer_bytes;
  p.storage_w += (size_t)l * sp.layer_bytes;
  if (p.out) p.out += (size_t)l * sp.out_layer_stride;
  if (p.xchg_out) p.xchg_out += (size_t)l * sp.out_layer_stride;
  if (p.lse) p.lse += (size_t)l * sp.lse_layer_stride;
  p.ws_acc += (size_t)l * sp.ws_layer_items * (kGroup * kHeadDim);
  p.ws_ml += (size_t)l * sp.ws_layer_items * (2 * kGroup);
  p.ws_count += (size_t)l * sp.n_seqs * sp.base.kv_heads;
  p.xchg_seq = sp.base.xchg_seq + (unsigned)l;
  p.xchg_slot = (int)(p.xchg_seq & 1u);
  return p;
}

// Combine the n_chunks partials of (sequence z, KV head h) from the workspace,
// write the rows (and run the cross-GPU exchange when one is configured), and
// clear the pair's arrival counter.  Called by the WARPS * 32 consumer threads of a CTA.
template <int WARPS, int STAGES>
__device__ __forceinline__ void combine_pair(const DecodeParams& p, const int z, const int h, const int n_chunks,
                                             unsigned char* smem, int* s_wait_ok_p) {
  using S = DecodeSmem<WARPS, STAGES>;
  unsigned char* tiles = smem;
  float* mrg = reinterpret_cast<float*>(smem + S::kTiles + S::kBars);
  float* mrg_o = mrg;
  float* mrg_m = mrg + WARPS * kGroup * kHeadDim;
  float* mrg_l = mrg_m + WARPS * kGroup;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The tile ring is idle now and serves as scratch: (m, l) of every chunk,
  // then one weight per chunk and row.  All loads of a phase are independent,
  // so their latencies overlap instead of adding up.
  constexpr int T = WARPS * 32;
  if (n_chunks * 48 > S::kTiles) {  // the host sizes chunks so that this cannot happen
    if (threadIdx.x == 0) {
      atomicExch(p.status, kStatusBadBlock);
      p.ws_count[z * p.kv_heads + h] = 0u;
    }
    return;
  }
  const size_t item0 = (size_t)(z * p.kv_heads + h) * p.max_chunks;
  float* cm = reinterpret_cast<float*>(tiles);  // [n_chunks][8]
  float* cw = cm + (size_t)n_chunks * 8;        // [n_chunks][4]
  // thread = (chunk group g, float4 column q): 64 float4 columns cover the 4x64 outputs.  The
  // first four partial loads of every thread do not depend on the weights: they are issued
  // together with the (m, l) loads, so the two latencies overlap.
  constexpr int G = T / 64;
  const int q4 = threadIdx.x & 63, g = threadIdx.x >> 6;
  const int r4 = q4 >> 4;
  const float4* src = reinterpret_cast<const float4*>(p.ws_acc + item0 * (kGroup * kHeadDim)) + q4;
  float4 v0[4];
#pragma unroll
  for (int u = 0; u < 4; u++)
    v0[u] = g + u * G < n_chunks ? __ldcg(src + (size_t)(g + u * G) * 64) : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = threadIdx.x; i < n_chunks * 8; i += T) cm[i] = __ldcg(p.ws_ml + item0 * 8 + i);
  consumer_sync(T);
  for (int r = warp; r < kGroup; r += WARPS) {
    float M = -INFINITY;
    for (int c = lane; c < n_chunks; c += 32) M = fmaxf(M, cm[c * 8 + r]);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, s));
    float L = 0.f;
    for (int c = lane; c < n_chunks; c += 32) {
      const float mc = cm[c * 8 + r];
      const float wgt = mc == -INFINITY ? 0.f : ex2(mc - M);
      cw[c * 4 + r] = wgt;
      L += wgt * cm[c * 8 + kGroup + r];
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) L += __shfl_xor_sync(0xffffffffu, L, s);
    if (lane == 0) {
      mrg_m[r] = M;
      mrg_l[r] = L;
    }
  }
  consumer_sync(T);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int u = 0; u < 4; u++) {
    if (g + u * G >= n_chunks) continue;
    const float wgt = cw[(g + u * G) * 4 + r4];
    acc.x += wgt * v0[u].x;
    acc.y += wgt * v0[u].y;
    acc.z += wgt * v0[u].z;
    acc.w += wgt * v0[u].w;
  }
  int c = g + 4 * G;
  for (; c + 3 * G < n_chunks; c += 4 * G) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; u++) v[u] = __ldcg(src + (size_t)(c + u * G) * 64);
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const float wgt = cw[(c + u * G) * 4 + r4];
      acc.x += wgt * v[u].x;
      acc.y += wgt * v[u].y;
      acc.z += wgt * v[u].z;
      acc.w += wgt * v[u].w;
    }
  }
  for (; c < n_chunks; c += G) {
    const float4 v = __ldcg(src + (size_t)c * 64);
    const float wgt = cw[c * 4 + r4];
    acc.x += wgt * v.x;
    acc.y += wgt * v.y;
    acc.z += wgt * v.z;
    acc.w += wgt * v.w;
  }
  reinterpret_cast<float4*>(mrg_o)[g * 64 + q4] = acc;
  consumer_sync(T);
  for (int idx = threadIdx.x; idx < kGroup * kHeadDim; idx += T) {
    float O = 0.f;
#pragma unroll
    for (int gg = 0; gg < G; gg++) O += mrg_o[gg * (kGroup * kHeadDim) + idx];
    write_row_outputs(p, z, h, idx >> 6, idx & 63, O, mrg_m[idx >> 6], mrg_l[idx >> 6]);
  }
  if (threadIdx.x == 0) p.ws_count[z * p.kv_heads + h] = 0u;
  publish_exchange(p, z, h, T);
  exchange_wait_merge(p, z, h, s_wait_ok_p, T);
}

// What a streaming CTA needs beyond the layer-0 launch descriptor: how many layers it walks and
// how far apart the layers' tensors are.  The kernel of one layer uses layers = 1.
struct StreamArgs {
  int layers, n_seqs, ws_layer_items;
  long long q_layer_stride, kv_layer_stride;
  unsigned long long layer_bytes;
};

// A streaming CTA: chunk x of (sequence z, KV head h), over a.layers layers.
// WARPS consumer warps, one producer warp, one publisher warp.
//  * Everything that does not depend on the tiles is done ONCE, before the first layer: the batch
//    entry, the CTA's slice of the block table (shared memory; it is the same for every layer,
//    only the cache base moves), every layer's 4 query rows (rotated here when the append is
//    fused in; kept in shared memory as bf16, ready to be picked up as A fragments), the
//    rotated-query output rows and the appended K/V rows of all layers.
//  * The producer warp's lane w feeds consumer warp w's ring: it waits for a freed stage (empty
//    barrier) and issues the next bulk copy, across layer borders, so the tiles of layer l+1 are
//    in flight while the consumers merge layer l.
//  * STEP (the one-launch step): a layer end costs the consumers two barriers among themselves and
//    one partial; the arrival count is released by the publisher warp, off their path (a
//    gpu-scope release takes about 0.6 us), and the pair's combining CTA does the rest.
//  * !STEP (the kernel of one layer): a single chunk writes its rows directly; otherwise partials
//    meet through arrival tickets and the last CTA of a (sequence, head) combines them.
template <int WARPS, int STAGES, bool STEP>
__device__ __forceinline__ void stream_cta(const DecodeParams& b, const StreamArgs& a, const int x, const int h,
                                           const int z, unsigned char* smem) {
  using S = DecodeSmem<WARPS, STAGES>;
  constexpr int T = WARPS * 32;  // consumer threads
  unsigned char* tiles = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kTiles);
  float* mrg = reinterpret_cast<float*>(smem + S::kTiles + S::kBars);
  float* mrg_o = mrg;                                // [WARPS][4][64]
  float* mrg_m = mrg + WARPS * kGroup * kHeadDim;     // [WARPS][4]
  float* mrg_l = mrg_m + WARPS * kGroup;              // [WARPS][4]
  uint64_t* empty_bars = reinterpret_cast<uint64_t*>(smem + S::kStepEmpty);
  int32_t* tbl_s = reinterpret_cast<int32_t*>(smem + S::kStepTbl);
  __nv_bfloat16* qsm = reinterpret_cast<__nv_bfloat16*>(smem + S::kStepQ);  // [layers][4][64], rotated
  __shared__ unsigned int s_ticket;
  __shared__ int s_wait_ok;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int layers = a.layers;
  const BatchEntry e = b.batch[z];
  const int n_blocks = (e.kv_len + kBlockTok - 1) / kBlockTok;
  const int n_chunks = max(1, (n_blocks + b.chunk_blocks - 1) / b.chunk_blocks);
  if (!STEP && b.cluster > 0 && x == 0 && threadIdx.x == 0)
    *reinterpret_cast<int*>(smem + S::kClusterParts - 16) = n_chunks;  // for cluster_finish, behind the cluster meeting
  if (x >= n_chunks) return;  // CTA-uniform
  const int blk_lo = x * b.chunk_blocks;
  const int cnt = max(0, min(n_blocks, blk_lo + b.chunk_blocks) - blk_lo);
  const int32_t* table = b.tables + (size_t)e.seq * b.max_blocks_per_seq + blk_lo;
  const int q_heads = b.kv_heads * kGroup;
  // layers whose partial this CTA has stored: written by consumer thread 0, polled by the publisher
  const uint32_t pub_word = smem_u32(empty_bars) + WARPS * STAGES * 8;
  // this CTA writes the new token's K/V rows into the sequence's last block before streaming it
  const bool appends = b.fuse && e.n_new > 0 && x == n_chunks - 1 && cnt > 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < WARPS * STAGES; s++) {
      mbar_init(smem_u32(bars) + s * 8, 1);
      mbar_init(smem_u32(empty_bars) + s * 8, 1);
    }
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(pub_word), "r"(0u) : "memory");
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncthreads();

  if (warp == WARPS) {
    // ================================ producer warp ==============================================
    const int held = min(cnt, S::kStepTblCap);
    for (int j = lane; j < held; j += 32) tbl_s[j] = table[j];
    if (appends && STEP) {
      // (The kernel of one layer appends from its consumer side, see the tile loop: the owner of the
      // last tile patches the new rows into the tile it has just received, so this CTA streams at
      // once like every other and pays no store -> fence -> copy round trip behind the wait.)
      // Appended rows of ALL layers: same arithmetic and placement as append_kernel; the
      // generic-proxy stores are ordered before this warp's own bulk (async-proxy) reads of that
      // block by the proxy fence below.  pdl == 2: k_new and v_new are the output of the kernel
      // in front, so this CTA's producer waits for it first; all other CTAs stream at once.
      if (b.pdl == 2) asm volatile("griddepcontrol.wait;" ::: "memory");
      if (lane < 8) {
        const int lpos = e.kv_len - 1;
        const int pos = e.kv_pos_off + lpos;
        const int blk = b.tables[(size_t)e.seq * b.max_blocks_per_seq + lpos / kBlockTok];
        const int slot = lpos % kBlockTok;
        const int c = lane & 3, is_v = lane >> 2;
        if (blk < 0 || blk >= b.num_blocks) {
          atomicExch(b.status, kStatusBadBlock);
        } else {
          float4 c8[2], s8[2];
          if (!is_v) {
            const float4* cs = reinterpret_cast<const float4*>(b.cos_table + (size_t)pos * 32 + c * 8);
            const float4* sn = reinterpret_cast<const float4*>(b.sin_table + (size_t)pos * 32 + c * 8);
            c8[0] = cs[0], c8[1] = cs[1], s8[0] = sn[0], s8[1] = sn[1];
          }
          for (int l = 0; l < layers; l++) {
            const __nv_bfloat16* row = (is_v ? b.v_new : b.k_new) + (size_t)l * a.kv_layer_stride +
                                       ((size_t)e.kv_row_off * b.kv_heads + h) * kHeadDim;
            const uint4* src = reinterpret_cast<const uint4*>(row);
            char* tile = b.storage_w + (size_t)l * a.layer_bytes + tile_off(blk, b.kv_heads, h, is_v);
            uint4 lo = src[c], hi = src[c + 4];
            if (!is_v) {
              uint4 ylo, yhi;
              rope_chunks<1>(lo, hi, reinterpret_cast<const float*>(c8), reinterpret_cast<const float*>(s8), ylo, yhi);
              lo = ylo;
              hi = yhi;
            }
            *reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c)) = lo;
            *reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c + 4)) = hi;
          }
        }
      }
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncwarp();
    if (lane < WARPS) {
      const int w = lane;
      const int my_n = cnt > w ? (cnt - w + WARPS - 1) / WARPS : 0;
      const uint32_t tile0 = smem_u32(tiles) + w * STAGES * kPairBytes;
      const uint32_t full0 = smem_u32(bars) + w * STAGES * 8;
      const uint32_t empty0 = smem_u32(empty_bars) + w * STAGES * 8;
      const size_t block_stride = (size_t)b.kv_heads * kPairBytes;
      const uint32_t total = (uint32_t)layers * (uint32_t)my_n;
      int i = 0;
      const char* layer_base = b.storage + (size_t)h * kPairBytes;
      for (uint32_t t = 0; t < total; t++) {
        const int st = (int)(t % STAGES);
        if (t >= (uint32_t)STAGES && !mbar_wait(empty0 + st * 8, ((t / STAGES) - 1u) & 1u)) {
          atomicExch(b.status, kStatusTimeout);
          break;
        }
        const int j = w + i * WARPS;
        int blk = j < S::kStepTblCap ? tbl_s[j] : table[j];
        if (blk < 0 || blk >= b.num_blocks) {
          atomicExch(b.status, kStatusBadBlock);
          blk = 0;
        }
        mbar_expect_tx(full0 + st * 8, kPairBytes);
        bulk_g2s(tile0 + st * kPairBytes, layer_base + (size_t)blk * block_stride, kPairBytes, full0 + st * 8);
        if (++i == my_n) {
          i = 0;
          layer_base += a.layer_bytes;
        }
      }
    }
    return;
  }
  if (warp == WARPS + 1) {
    // ================================ publisher warp =============================================
    // Consumer thread 0 stores the number of finished layers (release, CTA scope) after the barrier
    // that follows the CTA's partial stores; acquiring that word and then releasing at gpu scope
    // makes the stores visible (the release is cumulative) to the pair's combining CTA, which
    // acquires the count.  A word, not a barrier phase: the consumers may finish several short
    // layers while one release is still under way.  The kernel of one layer has no use for it.
    if (STEP && lane == 0) {
      const int pair = z * b.kv_heads + h;
      unsigned int done = 0;
      for (int l = 0; l < layers; l++) {
        SpinDeadline dl;
        while (done <= (unsigned)l) {
          asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(done) : "r"(pub_word) : "memory");
          if (done <= (unsigned)l && dl.expired()) break;
        }
        if (done <= (unsigned)l) {
          atomicExch(b.status, kStatusTimeout);
          break;
        }
        unsigned int* cntp = b.ws_count + (size_t)l * a.n_seqs * b.kv_heads + pair;
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(cntp) : "memory");
      }
    }
    return;
  }

  // ================================== consumer warps =============================================
  const int my_n = cnt > warp ? (cnt - warp + WARPS - 1) / WARPS : 0;
  const uint32_t tile0 = smem_u32(tiles) + warp * STAGES * kPairBytes;
  const uint32_t bar0 = smem_u32(bars) + warp * STAGES * 8;
  const uint32_t empty0 = smem_u32(empty_bars) + warp * STAGES * 8;

  // The kernel of one layer appends here: lanes 0..7 of the warp that owns the sequence's last tile
  // hold the new token's K (lanes 0..3, chunk pairs c and c + 4) and V (lanes 4..7) rows.  What does
  // not depend on the kernel in front (block id, RoPE factors) is fetched before the wait.
  const bool patcher = !STEP && appends && warp == (cnt - 1) % WARPS && lane < 8;
  int new_blk = 0;
  float4 nc8[2] = {}, ns8[2] = {};
  if (patcher) {
    new_blk = table[cnt - 1];
    if ((lane >> 2) == 0) {
      const int pos = e.kv_pos_off + e.kv_len - 1;
      const float4* cs = reinterpret_cast<const float4*>(b.cos_table + (size_t)pos * 32 + (lane & 3) * 8);
      const float4* sn = reinterpret_cast<const float4*>(b.sin_table + (size_t)pos * 32 + (lane & 3) * 8);
      nc8[0] = cs[0], nc8[1] = cs[1], ns8[0] = sn[0], ns8[1] = sn[1];
    }
  }
  // pdl == 2: the query rows (and the new K/V rows) are the output of the kernel in front
  if (b.pdl == 2) asm volatile("griddepcontrol.wait;" ::: "memory");
  uint4 new_lo = make_uint4(0, 0, 0, 0), new_hi = new_lo;
  if (patcher) {
    const int c = lane & 3, is_v = lane >> 2;
    const uint4* src = reinterpret_cast<const uint4*>((is_v ? b.v_new : b.k_new) +
                                                      ((size_t)e.kv_row_off * b.kv_heads + h) * kHeadDim);
    new_lo = src[c];
    new_hi = src[c + 4];
  }
  // ---- every layer's query rows into shared memory: rotated here (fp32, the rounding of
  // append_kernel) when the append is fused in, copied as they are otherwise
  {
    const size_t qrow0 = ((size_t)z * q_heads + h * kGroup) * kHeadDim;
    if (b.fuse) {
      const float* cs = b.cos_table + (size_t)e.q_pos0 * 32;
      const float* sn = b.sin_table + (size_t)e.q_pos0 * 32;
      for (int idx = threadIdx.x; idx < layers * kGroup * 32; idx += T) {
        const int c = idx & 31, r = (idx >> 5) & 3, l = idx >> 7;
        const __nv_bfloat16* qp = b.q + (size_t)l * a.q_layer_stride + qrow0 + r * kHeadDim;
        float y0, y1;
        rope_pair<1>(__bfloat162float(qp[c]), __bfloat162float(qp[c + 32]), cs[c], sn[c], y0, y1);
        const __nv_bfloat16 b0 = __float2bfloat16_rn(y0), b1 = __float2bfloat16_rn(y1);
        qsm[(l * kGroup + r) * kHeadDim + c] = b0;
        qsm[(l * kGroup + r) * kHeadDim + c + 32] = b1;
        if (b.q_rot_out && x == 0) {
          __nv_bfloat16* qo = b.q_rot_out + (size_t)l * a.q_layer_stride + qrow0 + r * kHeadDim;
          qo[c] = b0;
          qo[c + 32] = b1;
        }
      }
    } else {
      for (int idx = threadIdx.x; idx < layers * kGroup * 32; idx += T) {
        const int c = idx & 31, r = (idx >> 5) & 3, l = idx >> 7;
        const uint32_t* qp = reinterpret_cast<const uint32_t*>(b.q + (size_t)l * a.q_layer_stride + qrow0 + r * kHeadDim);
        reinterpret_cast<uint32_t*>(qsm + (l * kGroup + r) * kHeadDim)[c] = qp[c];
      }
    }
  }
  consumer_sync(T);

  const int qrow = lane >> 2, qcol = (lane & 3) * 2;
  const int mj = lane >> 3, rr = lane & 7;
  const uint32_t k_row_off = (uint32_t)(((mj >> 1) * 8 + rr) * 128);
  const uint32_t v_row_off = (uint32_t)(kTileBytes + ((mj & 1) * 8 + rr) * 128);
  const int pair = z * b.kv_heads + h;
  const int item = pair * b.max_chunks + x;
  bool failed = false;
  uint32_t t = 0;

  for (int l = 0; l < layers; l++) {
    // Query fragments of this layer: rows 0..3 are the group's heads, the rest zero.
    uint32_t qa[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ks++) {
      qa[ks][0] = qa[ks][1] = qa[ks][2] = qa[ks][3] = 0u;
      if (qrow < kGroup) {
        const __nv_bfloat16* qp = qsm + (l * kGroup + qrow) * kHeadDim + ks * 16 + qcol;
        qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp);
        qa[ks][2] = *reinterpret_cast<const uint32_t*>(qp + 8);
      }
    }
    float o[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; nt++) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    for (int i = 0; i < my_n; i++, t++) {
      const int st = (int)(t % STAGES);
      if (!failed) {
        const bool ok = mbar_wait(bar0 + st * 8, (t / STAGES) & 1u);
        if (!__all_sync(0xffffffffu, ok)) {
          failed = true;
          if (lane == 0) atomicExch(b.status, kStatusTimeout);
        }
      }
      if (failed) continue;  // keeps joining the layer barriers; its producer lane runs into its own limit
      const uint32_t tile = tile0 + st * kPairBytes;
      if (!STEP && appends && i == my_n - 1 && warp == (cnt - 1) % WARPS) {
        // the sequence's last block has arrived with its old contents: put the new token's rows into
        // the shared-memory tile and into the cache (same arithmetic and placement as append_kernel)
        if (patcher) {
          const int c = lane & 3, is_v = lane >> 2;
          const int slot = (e.kv_len - 1) % kBlockTok;
          if (new_blk < 0 || new_blk >= b.num_blocks) {
            atomicExch(b.status, kStatusBadBlock);
          } else {
            uint4 lo = new_lo, hi = new_hi;
            if (!is_v) {
              uint4 ylo, yhi;
              rope_chunks<1>(lo, hi, reinterpret_cast<const float*>(nc8), reinterpret_cast<const float*>(ns8), ylo, yhi);
              lo = ylo;
              hi = yhi;
            }
            const uint32_t base = tile + (is_v ? kTileBytes : 0);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + tile_chunk_off(slot, c)), "r"(lo.x),
                         "r"(lo.y), "r"(lo.z), "r"(lo.w)
                         : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + tile_chunk_off(slot, c + 4)), "r"(hi.x),
                         "r"(hi.y), "r"(hi.z), "r"(hi.w)
                         : "memory");
            char* gt = b.storage_w + tile_off(new_blk, b.kv_heads, h, is_v);
            *reinterpret_cast<uint4*>(gt + tile_chunk_off(slot, c)) = lo;
            *reinterpret_cast<uint4*>(gt + tile_chunk_off(slot, c + 4)) = hi;
          }
        }
        __syncwarp();
      }

      float s[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, tile + k_row_off + ((((ks * 2 + (mj & 1)) ^ rr)) << 4));
        mma_bf16(s[0], qa[ks], b0, b1);
        mma_bf16(s[1], qa[ks], b2, b3);
      }

      // scaled scores (base 2), tail mask, online softmax on rows lane/4
      const int key0 = (blk_lo + warp + i * WARPS) * kBlockTok + qcol;
      float tt[4];
      tt[0] = s[0][0] * b.scale_log2;
      tt[1] = s[0][1] * b.scale_log2;
      tt[2] = s[1][0] * b.scale_log2;
      tt[3] = s[1][1] * b.scale_log2;
      if (key0 + 9 >= e.kv_len) {
        if (key0 >= e.kv_len) tt[0] = -INFINITY;
        if (key0 + 1 >= e.kv_len) tt[1] = -INFINITY;
        if (key0 + 8 >= e.kv_len) tt[2] = -INFINITY;
        if (key0 + 9 >= e.kv_len) tt[3] = -INFINITY;
      }
      float mx = fmaxf(fmaxf(tt[0], tt[1]), fmaxf(tt[2], tt[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float corr = ex2(m_run - m_new);
      m_run = m_new;
      const float p0 = ex2(tt[0] - m_new), p1 = ex2(tt[1] - m_new);
      const float p2 = ex2(tt[2] - m_new), p3 = ex2(tt[3] - m_new);
      l_run = l_run * corr + ((p0 + p1) + (p2 + p3));
      uint32_t pa[4];
      pa[0] = pack_bf16(p0, p1);
      pa[1] = 0u;
      pa[2] = pack_bf16(p2, p3);
      pa[3] = 0u;
#pragma unroll
      for (int nt = 0; nt < 8; nt++) {
        o[nt][0] *= corr;
        o[nt][1] *= corr;
      }
#pragma unroll
      for (int np = 0; np < 4; np++) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(b0, b1, b2, b3, tile + v_row_off + ((((np * 2 + (mj >> 1)) ^ rr)) << 4));
        mma_bf16(o[2 * np], pa, b0, b1);
        mma_bf16(o[2 * np + 1], pa, b2, b3);
      }

      // all lanes have read the stage (their ldmatrix results are in registers): hand it back
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + st * 8);
    }

    // pdl == 1 (the layers of a step as one kernel each): the streaming above only read the
    // cache; the workspace, tickets and outputs written from here on are shared with the previous
    // layer's kernel, which must have completed
    if (!STEP && b.pdl == 1) asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- end of the layer: merge the warps of this CTA --------------------------------------------
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (qrow < kGroup) {
      float* orow = mrg_o + (warp * kGroup + qrow) * kHeadDim;
#pragma unroll
      for (int nt = 0; nt < 8; nt++)
        *reinterpret_cast<float2*>(orow + nt * 8 + qcol) = make_float2(o[nt][0], o[nt][1]);
      if ((lane & 3) == 0) {
        mrg_m[warp * kGroup + qrow] = m_run;
        mrg_l[warp * kGroup + qrow] = l_run;
      }
    }
    consumer_sync(T);
    float* ws_acc = b.ws_acc + ((size_t)l * a.ws_layer_items + item) * (kGroup * kHeadDim);
    float* ws_ml = b.ws_ml + ((size_t)l * a.ws_layer_items + item) * (2 * kGroup);
    for (int idx = threadIdx.x; idx < kGroup * kHeadDim; idx += T) {
      const int r = idx >> 6, d = idx & 63;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; w++) M = fmaxf(M, mrg_m[w * kGroup + r]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; w++) {
        const float mw = mrg_m[w * kGroup + r];
        const float wgt = mw == -INFINITY ? 0.f : ex2(mw - M);
        L += wgt * mrg_l[w * kGroup + r];
        O += wgt * mrg_o[(w * kGroup + r) * kHeadDim + d];
      }
      if (!STEP && n_chunks == 1) {
        write_row_outputs(b, z, h, r, d, O, M, L);
      } else if (!STEP && b.cluster > 0) {
        // the CTA's partial goes into slot x of the first CTA's shared memory (remote stores: the
        // cluster meeting behind them makes them visible), so that CTA merges from local memory
        const float* slot = reinterpret_cast<const float*>(smem + S::kClusterParts) + x * S::kClusterPartFloats;
        st_cluster_f32(slot + idx, 0u, O);
        if (d == 0) {
          st_cluster_f32(slot + kGroup * kHeadDim + r, 0u, M);
          st_cluster_f32(slot + kGroup * kHeadDim + kGroup + r, 0u, L);
        }
      } else {
        ws_acc[idx] = O;
        if (d == 0) {
          ws_ml[r] = M;
          ws_ml[kGroup + r] = L;
        }
      }
    }
    if (STEP) {
      // orders every consumer's partial stores before thread 0's store of the layer count (which the
      // publisher warp turns into the released arrival) and frees the merge buffers for the next layer
      consumer_sync(T);
      if (threadIdx.x == 0)
        asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(pub_word), "r"((unsigned)(l + 1)) : "memory");
    }
  }
  if (STEP) return;

  // ---- the kernel of one layer: finish the (sequence, head) --------------------------------------
  if (n_chunks == 1) {
    publish_exchange(b, z, h, T);
    exchange_wait_merge(b, z, h, &s_wait_ok, T);
    return;
  }
  if (b.cluster > 0) return;  // combined by the cluster's first CTA (cluster_finish)
  // combine across chunks: the last CTA to arrive does it
  __threadfence();
  consumer_sync(T);
  if (threadIdx.x == 0) s_ticket = atomicAdd(&b.ws_count[pair], 1u);
  consumer_sync(T);
  if (s_ticket != (unsigned)(n_chunks - 1)) return;
  __threadfence();
  combine_pair<WARPS, STAGES>(b, z, h, n_chunks, smem, &s_wait_ok);
}

// Cluster form of the one-layer kernel: the consumer threads of the cluster's first CTA merge the
// chunks' partials (O [4][64], m [4], l [4]), which the peers have pushed into its shared memory,
// and finish the (sequence, head) as the last-arriving CTA does in the workspace form.
template <int WARPS, int STAGES>
__device__ __forceinline__ void cluster_finish(const DecodeParams& p, const int h, const int z, unsigned char* smem) {
  using S = DecodeSmem<WARPS, STAGES>;
  constexpr int T = WARPS * 32;
  __shared__ int s_wait_ok;
  // the chunk count of this (sequence, head): left in shared memory by the streaming part (a load of
  // the batch entry here would put a round trip to L2 on the critical path)
  const int n_chunks = *reinterpret_cast<const int*>(smem + S::kClusterParts - 16);
  if (n_chunks <= 1) return;  // a single chunk has written its rows itself
  const float* parts = reinterpret_cast<const float*>(smem + S::kClusterParts);
  for (int idx = threadIdx.x; idx < kGroup * kHeadDim; idx += T) {
    const int r = idx >> 6, d = idx & 63;
    float M = -INFINITY;
    for (int c = 0; c < n_chunks; c++) M = fmaxf(M, parts[c * S::kClusterPartFloats + kGroup * kHeadDim + r]);
    float L = 0.f, O = 0.f;
    for (int c = 0; c < n_chunks; c++) {
      const float* pc = parts + c * S::kClusterPartFloats;
      const float mc = pc[kGroup * kHeadDim + r];
      const float wgt = mc == -INFINITY ? 0.f : ex2(mc - M);
      L += wgt * pc[kGroup * kHeadDim + kGroup + r];
      O += wgt * pc[idx];
    }
    write_row_outputs(p, z, h, r, d, O, M, L);
  }
  publish_exchange(p, z, h, T);
  exchange_wait_merge(p, z, h, &s_wait_ok, T);
}

template <int WARPS, int STAGES>
__global__ void __launch_bounds__(DecodeSmem<WARPS, STAGES>::kStepThreads)
decode_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  // let the kernel behind take SMs (and start the part of its work that does not depend on this
  // one) as soon as this one's CTAs leave them
  if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const StreamArgs a{1, (int)gridDim.z, 0, 0, 0, 0ull};
  stream_cta<WARPS, STAGES, false>(p, a, blockIdx.x, blockIdx.y, blockIdx.z, smem);
  if (p.cluster > 0) {
    // Every thread of every CTA of the cluster comes through here, whatever it did above (CTAs
    // beyond a sequence's chunks, the producer warp, a thread whose wait ran out), so the meeting
    // never waits for a thread that left — and the first CTA, whose shared memory the peers store
    // into, is still there when they do.
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
    // every partial is in the first CTA's shared memory; nobody touches a peer's memory from here on
    if (blockIdx.x == 0 && (int)threadIdx.x < WARPS * 32) cluster_finish<WARPS, STAGES>(p, blockIdx.y, blockIdx.z, smem);
  }
}

template <int WARPS, int STAGES>
__device__ __forceinline__ void decode_step_body(const DecodeStepParams& sp, const int b, unsigned char* smem) {
  __shared__ int s_ok;
  __shared__ int s_wait_ok;
  const int n_stream = sp.n_stream;
  if (b < n_stream) {
    int z = 0;
    while (z + 1 < sp.n_seqs && b >= (int)sp.seq_first[z + 1]) z++;
    const int local = b - (int)sp.seq_first[z];
    const int chunks_z = ((int)sp.seq_first[z + 1] - (int)sp.seq_first[z]) / sp.base.kv_heads;
    const int x = local % chunks_z, h = local / chunks_z;
    const StreamArgs a{sp.layers, sp.n_seqs, sp.ws_layer_items, sp.q_layer_stride, sp.kv_layer_stride, sp.layer_bytes};
    stream_cta<WARPS, STAGES, true>(sp.base, a, x, h, z, smem);
    return;
  }
  if ((int)threadIdx.x >= WARPS * 32) return;  // the producer and publisher warps have no part in combining
  // Combining CTAs: sp.combiners per (sequence, head), taking the layers in turn.  One CTA needs
  // about 5 us per layer (2.2 us of combine, the rest waiting on its own loads and polls), more
  // than a streaming CTA needs at short contexts (3.5 us), so with one the combiners set the pace.
  const int n_pairs = sp.n_seqs * sp.base.kv_heads;
  const int pair = (b - n_stream) % n_pairs, turn = (b - n_stream) / n_pairs;
  if (turn >= sp.combiners) return;
  const int z = pair / sp.base.kv_heads, h = pair % sp.base.kv_heads;
  const BatchEntry e = sp.base.batch[z];
  const int n_blocks = (e.kv_len + kBlockTok - 1) / kBlockTok;
  const int n_chunks = max(1, (n_blocks + sp.base.chunk_blocks - 1) / sp.base.chunk_blocks);
  for (int l = turn; l < sp.layers; l += sp.combiners) {
    const DecodeParams p = step_layer_params(sp, l);
    if (threadIdx.x == 0) {
      const unsigned int* cnt = p.ws_count + pair;
      SpinDeadline dl;
      int ok = 1;
      for (;;) {
        unsigned int v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
        if (v >= (unsigned)n_chunks) break;
        if (dl.expired()) {
          ok = 0;
          break;
        }
      }
      s_ok = ok;
    }
    consumer_sync(WARPS * 32);
    if (!s_ok) {  // a streaming CTA never arrived: record it and leave
      if (threadIdx.x == 0) atomicExch(p.status, kStatusTimeout);
      return;
    }
    combine_pair<WARPS, STAGES>(p, z, h, n_chunks, smem, &s_wait_ok);
    consumer_sync(WARPS * 32);
  }
}

template <int WARPS, int STAGES>
__global__ void __launch_bounds__(DecodeSmem<WARPS, STAGES>::kStepThreads, 1)
decode_step_kernel(const __grid_constant__ DecodeStepParams sp) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  decode_step_body<WARPS, STAGES>(sp, blockIdx.x, smem);
}

// Several ranks of a range-sharded batch whose pools live on the SAME GPU, as one cooperative
// launch: CTAs [r * ctas_per_rank, (r + 1) * ctas_per_rank) are rank r's step.  The ranks wait on
// each other's exchange words, so they must be co-resident, which separate launches on one GPU
// would not guarantee.
template <int WARPS, int STAGES>
__global__ void __launch_bounds__(DecodeSmem<WARPS, STAGES>::kStepThreads, 1)
decode_step_ranks_kernel(const __grid_constant__ ColocatedStepParams cp) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  const int r = blockIdx.x / cp.ctas_per_rank;
  if (r >= cp.world) return;
  decode_step_body<WARPS, STAGES>(cp.rank[r], blockIdx.x - r * cp.ctas_per_rank, smem);
}

template <int WARPS, int STAGES>
cudaError_t launch_decode_cfg(const DecodeParams& p, int n_seqs, cudaStream_t stream) {
  using S = DecodeSmem<WARPS, STAGES>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(decode_kernel<WARPS, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::one_layer_bytes());
    if (e != cudaSuccess) return e;
    // clusters of up to 16 CTAs (8 is the portable limit)
    e = cudaFuncSetAttribute(decode_kernel<WARPS, STAGES>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  dim3 grid(p.max_chunks, p.kv_heads, n_seqs);
  if (!p.pdl && p.cluster <= 0) {
    decode_kernel<WARPS, STAGES><<<grid, S::kStepThreads, S::one_layer_bytes(), stream>>>(p);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(S::kStepThreads);
  cfg.dynamicSmemBytes = S::one_layer_bytes();
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (p.pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    n_attr++;
  }
  if (p.cluster > 0) {
    if (p.cluster != p.max_chunks) return cudaErrorInvalidValue;  // a cluster is all chunks of a (sequence, head)
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = (unsigned)p.cluster;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    n_attr++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return cudaLaunchKernelEx(&cfg, decode_kernel<WARPS, STAGES>, p);
}

}  // namespace

size_t decode_ws_acc_floats_per_item() { return kGroup * kHeadDim; }

namespace {
template <int WARPS, int STAGES>
int cluster_limit_cfg() {
  using S = DecodeSmem<WARPS, STAGES>;
  cudaFuncSetAttribute(decode_kernel<WARPS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::one_layer_bytes());
  cudaFuncSetAttribute(decode_kernel<WARPS, STAGES>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  for (int size = 16; size >= 2; size /= 2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(size, 1, 1);
    cfg.blockDim = dim3(S::kStepThreads);
    cfg.dynamicSmemBytes = S::one_layer_bytes();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, decode_kernel<WARPS, STAGES>, &cfg) == cudaSuccess && n >= 1) return size;
    cudaGetLastError();  // an unsupported size is an answer, not an error to keep
  }
  return 0;
}
}  // namespace

// Largest cluster size (16, 8, 4, 2; 0 = none) the one-layer kernel of this shape can be launched
// with on the current device, asked of the occupancy calculator once per device and shape.
int decode_cluster_limit(int warps, int stages) {
  static int cache[64][2] = {};  // [device][shape]: 0 = not asked yet, else limit + 1
  int dev = 0;
  cudaGetDevice(&dev);
  const int shape = (warps == 8 && stages == 4) ? 0 : ((warps == 4 && stages == 4) ? 1 : -1);
  if (shape < 0 || dev < 0 || dev >= 64) return 0;  // the planner's two shapes only
  if (cache[dev][shape] == 0) cache[dev][shape] = 1 + (shape == 0 ? cluster_limit_cfg<8, 4>() : cluster_limit_cfg<4, 4>());
  return cache[dev][shape] - 1;
}

bool decode_shape_supported(int warps, int stages) {
  return (warps == 4 && (stages == 3 || stages == 4 || stages == 6)) ||
         (warps == 8 && (stages == 2 || stages == 3 || stages == 4 || stages == 6)) ||
         (warps == 2 && (stages == 4 || stages == 8));
}

cudaError_t launch_decode(const DecodeParams& p, int n_seqs, int warps, int stages,
                          cudaStream_t stream) {
  if (n_seqs <= 0) return cudaSuccess;
  switch (warps * 16 + stages) {
    case 4 * 16 + 3: return launch_decode_cfg<4, 3>(p, n_seqs, stream);
    case 4 * 16 + 6: return launch_decode_cfg<4, 6>(p, n_seqs, stream);
    case 8 * 16 + 2: return launch_decode_cfg<8, 2>(p, n_seqs, stream);
    case 8 * 16 + 3: return launch_decode_cfg<8, 3>(p, n_seqs, stream);
    case 8 * 16 + 4: return launch_decode_cfg<8, 4>(p, n_seqs, stream);
    case 8 * 16 + 6: return launch_decode_cfg<8, 6>(p, n_seqs, stream);
    case 2 * 16 + 4: return launch_decode_cfg<2, 4>(p, n_seqs, stream);
    case 2 * 16 + 8: return launch_decode_cfg<2, 8>(p, n_seqs, stream);
    default: return launch_decode_cfg<4, 4>(p, n_seqs, stream);
  }
}

template <int WARPS, int STAGES>
cudaError_t launch_decode_step_cfg(const DecodeStepParams& sp, cudaStream_t stream) {
  using S = DecodeSmem<WARPS, STAGES>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_kernel<WARPS, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::step_bytes(kMaxStepLayers));
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  DecodeStepParams args = sp;
  void* kargs[] = {&args};
  // cooperative: the combining CTAs wait for the streaming CTAs of the same grid
  return cudaLaunchCooperativeKernel((const void*)decode_step_kernel<WARPS, STAGES>, dim3(decode_step_ctas(sp)),
                                     dim3(S::kStepThreads), kargs, S::step_bytes(sp.layers), stream);
}

cudaError_t launch_decode_step_colocated(const ColocatedStepParams& cp, cudaStream_t stream) {
  using S = DecodeSmem<8, 4>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_ranks_kernel<8, 4>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::step_bytes(kMaxStepLayers));
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  ColocatedStepParams args = cp;
  void* kargs[] = {&args};
  return cudaLaunchCooperativeKernel((const void*)decode_step_ranks_kernel<8, 4>, dim3(cp.world * cp.ctas_per_rank),
                                     dim3(S::kStepThreads), kargs, S::step_bytes(cp.rank[0].layers), stream);
}

cudaError_t launch_decode_step(const DecodeStepParams& sp, int warps, int stages, cudaStream_t stream) {
  if (sp.n_seqs <= 0 || sp.layers <= 0) return cudaSuccess;
  if (warps == 8 && stages == 4) return launch_decode_step_cfg<8, 4>(sp, stream);
  if (warps == 8 && stages == 3) return launch_decode_step_cfg<8, 3>(sp, stream);
  if (warps == 4 && stages == 4) return launch_decode_step_cfg<4, 4>(sp, stream);
  return cudaErrorInvalidConfiguration;
}

// ---- merge of split-KV partials from disjoint key ranges ---------------------
// One thread per output element; n_parts is small (one part per GPU).
__global__ void __launch_bounds__(256)
merge_kernel(MergeParams p) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.rows * kHeadDim) return;
  const int r = idx >> 6;
  float M = -INFINITY;
  for (int k = 0; k < p.n_parts; k++) M = fmaxf(M, p.lse_parts[(size_t)k * p.rows + r]);
  float L = 0.f, O = 0.f;
  if (M > -INFINITY) {
    for (int k = 0; k < p.n_parts; k++) {
      const float lk = p.lse_parts[(size_t)k * p.rows + r];
      const float w = lk == -INFINITY ? 0.f : __expf(lk - M);
      L += w;
      O += w * p.o_parts[(size_t)k * p.rows * kHeadDim + idx];
    }
  }
  const float v = L > 0.f ? O / L : 0.f;
  if (p.out) p.out[idx] = __float2bfloat16_rn(v);
  if (p.out_f32) p.out_f32[idx] = v;
  if (p.lse_out && (idx & 63) == 0) p.lse_out[r] = L > 0.f ? M + __logf(L) : -INFINITY;
}

cudaError_t launch_merge(const MergeParams& p, cudaStream_t stream) {
  if (p.rows <= 0 || p.n_parts <= 0) return cudaSuccess;
  const int total = p.rows * kHeadDim;
  merge_kernel<<<(total + 255) / 256, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace pa
