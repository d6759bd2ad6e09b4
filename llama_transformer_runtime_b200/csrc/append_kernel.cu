// K1: fused RoPE + paged append, and the un-paging gather.
//
// Replaces, in one launch, the reference's rope_q_kernel, rope_k_kernel and
// transpose_v_kernel (src/kernels/rope/rope.cu:23-262) and the host loop of
// 2*8*tokens 128-byte cudaMemcpy calls that appends to the cache
// (src/runtime/attention.cu:239-262).  Pure HBM streaming: every thread moves
// 16-byte chunks; RoPE pairs element i with i+32, so one thread owns chunk c
// (elements 8c..8c+7) and its partner chunk c+4.
#include "kernels.cuh"
#include "rope.cuh"

namespace pa {

constexpr int kAppendThreads = 256;
constexpr int kAppendTokPerCta = 4;
// units of one token: (32 query heads + 8 K heads + 8 V heads) x 4 chunk pairs at most
constexpr int kAppendMaxIters = (kAppendTokPerCta * (32 + 8 + 8) * 4 + kAppendThreads - 1) / kAppendThreads;

// What one thread moves: chunk pair (c, c + 4) of one head row of one token.
struct AppendUnit {
  const uint4* src;   // the 64-element row in q_in / k_in / v_in
  uint4* dst_lo;      // where chunk c goes (rotated-Q row or cache tile)
  uint4* dst_hi;      // where chunk c + 4 goes
  const float* cs;    // 8 cos values of pairs 8c..8c+7 (nullptr: V, no rotation)
  const float* sn;
};

__global__ void __launch_bounds__(kAppendThreads)
append_kernel(AppendParams p) {
  constexpr int VARIANT = 1;  // the rounding of the reference's compiled kernel (rope.cuh)
  const BatchEntry e = p.batch[blockIdx.y];
  const int tok0 = blockIdx.x * kAppendTokPerCta;
  const int n_q = p.q_out ? e.n_q : 0;
  const int span = max(n_q, e.n_new);
  if (tok0 >= span) return;
  const int ntok = min(kAppendTokPerCta, span - tok0);
  const int q_heads = p.kv_heads * kGroup;
  const int q_units = p.q_out ? q_heads * 4 : 0;
  const int k_units = p.kv_heads * 4;
  const int units_per_tok = q_units + 2 * k_units;
  const int32_t* table = p.tables + (size_t)e.seq * p.max_blocks_per_seq;

  // Where a unit reads and writes.  A unit with nothing to do (a token beyond this sequence's
  // query rows or new tokens, a block id outside the pool) comes back with src == nullptr.
  auto unit_of = [&](int u) {
    AppendUnit a{nullptr, nullptr, nullptr, nullptr, nullptr};
    const int t = u / units_per_tok;
    int w = u - t * units_per_tok;
    const int tok = tok0 + t;
    const int c = w & 3;  // chunk pair (c, c+4)
    if (w < q_units) {
      if (tok >= n_q) return a;
      const int h = w >> 2;
      const size_t row = (size_t)e.q_row_off + tok;
      const int pos = e.q_pos0 + tok;
      a.src = reinterpret_cast<const uint4*>(p.q_in + (row * q_heads + h) * kHeadDim) + c;
      a.dst_lo = reinterpret_cast<uint4*>(p.q_out + (row * q_heads + h) * kHeadDim) + c;
      a.dst_hi = a.dst_lo + 4;
      a.cs = p.cos_table + (size_t)pos * 32 + c * 8;
      a.sn = p.sin_table + (size_t)pos * 32 + c * 8;
      return a;
    }
    if (tok >= e.n_new) return a;
    w -= q_units;
    const size_t row = (size_t)e.kv_row_off + tok;
    const int lpos = e.kv_len - e.n_new + tok;  // position inside the local cache
    const int pos = e.kv_pos_off + lpos;        // RoPE position
    const int blk = table[lpos / kBlockTok];
    const int slot = lpos % kBlockTok;
    if (blk < 0 || blk >= p.num_blocks) {
      atomicExch(p.status, kStatusBadBlock);
      return a;
    }
    const int is_v = w >= k_units;
    const int h = (is_v ? w - k_units : w) >> 2;
    a.src = reinterpret_cast<const uint4*>((is_v ? p.v_in : p.k_in) + (row * p.kv_heads + h) * kHeadDim) + c;
    char* tile = p.storage + tile_off(blk, p.kv_heads, h, is_v);
    a.dst_lo = reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c));
    a.dst_hi = reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c + 4));
    if (!is_v) {
      a.cs = p.cos_table + (size_t)pos * 32 + c * 8;
      a.sn = p.sin_table + (size_t)pos * 32 + c * 8;
    }
    return a;
  };

  // All loads of a thread's units are issued before the first store (q_out may alias q_in, so the
  // compiler cannot move them itself): the thread has every load in flight at once instead of one
  // load-rotate-store chain after another.
  const int total = ntok * units_per_tok;
  // kAppendMaxIters covers the model's head counts in one pass; other head counts take more passes
#pragma unroll 1
  for (int base = 0; base < total; base += kAppendMaxIters * kAppendThreads) {
    AppendUnit un[kAppendMaxIters];
    uint4 lo[kAppendMaxIters], hi[kAppendMaxIters];
    float4 c8[kAppendMaxIters][2], s8[kAppendMaxIters][2];
#pragma unroll
    for (int it = 0; it < kAppendMaxIters; it++) {
      const int u = base + threadIdx.x + it * kAppendThreads;
      un[it] = u < total ? unit_of(u) : AppendUnit{nullptr, nullptr, nullptr, nullptr, nullptr};
      if (un[it].src) {
        lo[it] = un[it].src[0];
        hi[it] = un[it].src[4];
        if (un[it].cs) {
          c8[it][0] = reinterpret_cast<const float4*>(un[it].cs)[0];
          c8[it][1] = reinterpret_cast<const float4*>(un[it].cs)[1];
          s8[it][0] = reinterpret_cast<const float4*>(un[it].sn)[0];
          s8[it][1] = reinterpret_cast<const float4*>(un[it].sn)[1];
        }
      }
    }
#pragma unroll
    for (int it = 0; it < kAppendMaxIters; it++) {
      if (!un[it].src) continue;
      uint4 ylo = lo[it], yhi = hi[it];
      if (un[it].cs)
        rope_chunks<VARIANT>(lo[it], hi[it], reinterpret_cast<const float*>(c8[it]),
                             reinterpret_cast<const float*>(s8[it]), ylo, yhi);
      *un[it].dst_lo = ylo;
      *un[it].dst_hi = yhi;
    }
  }
}

cudaError_t launch_append(const AppendParams& p, int n_seqs, int max_new, cudaStream_t stream) {
  if (n_seqs <= 0 || max_new <= 0) return cudaSuccess;
  dim3 grid((max_new + kAppendTokPerCta - 1) / kAppendTokPerCta, n_seqs);
  append_kernel<<<grid, kAppendThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

// ---- gather: cache -> contiguous [kv_heads][stride][64] ----------------------
// What Attention::get_key_cache()/get_value_cache() expose in the reference
// (src/runtime/attention.cu:93-98): one thread per 16-byte chunk.
__global__ void __launch_bounds__(256)
gather_kernel(GatherParams p) {
  const size_t total = (size_t)p.length * p.kv_heads * 2 * 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i & 7);
    const int kv = (int)((i >> 3) & 1);
    const size_t r = i >> 4;
    const int h = (int)(r % p.kv_heads);
    const int pos = (int)(r / p.kv_heads);
    const int blk = p.table[pos / kBlockTok];
    if (blk < 0 || blk >= p.num_blocks) {
      atomicExch(p.status, kStatusBadBlock);
      continue;
    }
    const char* tile = p.storage + tile_off(blk, p.kv_heads, h, kv);
    uint4 v = *reinterpret_cast<const uint4*>(tile + tile_chunk_off(pos % kBlockTok, c));
    __nv_bfloat16* dst = (kv ? p.v_out : p.k_out) + ((size_t)h * p.out_stride + pos) * kHeadDim;
    reinterpret_cast<uint4*>(dst)[c] = v;
  }
}

cudaError_t launch_gather(const GatherParams& p, cudaStream_t stream) {
  if (p.length <= 0) return cudaSuccess;
  size_t total = (size_t)p.length * p.kv_heads * 16;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  gather_kernel<<<blocks, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace pa
