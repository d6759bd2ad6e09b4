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

  for (int u = threadIdx.x; u < ntok * units_per_tok; u += kAppendThreads) {
    const int t = u / units_per_tok;
    int w = u - t * units_per_tok;
    const int tok = tok0 + t;
    const int c = w & 3;  // chunk pair (c, c+4)

    if (w < q_units) {
      if (tok >= n_q) continue;
      const int h = w >> 2;
      const size_t row = (size_t)e.q_row_off + tok;
      const int pos = e.q_pos0 + tok;
      const uint4* src = reinterpret_cast<const uint4*>(p.q_in + (row * q_heads + h) * kHeadDim);
      uint4* dst = reinterpret_cast<uint4*>(p.q_out + (row * q_heads + h) * kHeadDim);
      const float4* cs = reinterpret_cast<const float4*>(p.cos_table + (size_t)pos * 32 + c * 8);
      const float4* sn = reinterpret_cast<const float4*>(p.sin_table + (size_t)pos * 32 + c * 8);
      float4 c8[2] = {cs[0], cs[1]}, s8[2] = {sn[0], sn[1]};
      uint4 lo = src[c], hi = src[c + 4], ylo, yhi;
      rope_chunks<VARIANT>(lo, hi, reinterpret_cast<const float*>(c8),
                           reinterpret_cast<const float*>(s8), ylo, yhi);
      dst[c] = ylo;
      dst[c + 4] = yhi;
      continue;
    }
    if (tok >= e.n_new) continue;
    w -= q_units;
    const size_t row = (size_t)e.kv_row_off + tok;
    const int lpos = e.kv_len - e.n_new + tok;  // position inside the local cache
    const int pos = e.kv_pos_off + lpos;        // RoPE position
    const int blk = table[lpos / kBlockTok];
    const int slot = lpos % kBlockTok;
    if (blk < 0 || blk >= p.num_blocks) {
      atomicExch(p.status, kStatusBadBlock);
      continue;
    }
    if (w < k_units) {
      const int h = w >> 2;
      const uint4* src = reinterpret_cast<const uint4*>(p.k_in + (row * p.kv_heads + h) * kHeadDim);
      char* tile = p.storage + tile_off(blk, p.kv_heads, h, 0);
      const float4* cs = reinterpret_cast<const float4*>(p.cos_table + (size_t)pos * 32 + c * 8);
      const float4* sn = reinterpret_cast<const float4*>(p.sin_table + (size_t)pos * 32 + c * 8);
      float4 c8[2] = {cs[0], cs[1]}, s8[2] = {sn[0], sn[1]};
      uint4 lo = src[c], hi = src[c + 4], ylo, yhi;
      rope_chunks<VARIANT>(lo, hi, reinterpret_cast<const float*>(c8),
                           reinterpret_cast<const float*>(s8), ylo, yhi);
      *reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c)) = ylo;
      *reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c + 4)) = yhi;
    } else {
      w -= k_units;
      const int h = w >> 2;
      const uint4* src = reinterpret_cast<const uint4*>(p.v_in + (row * p.kv_heads + h) * kHeadDim);
      char* tile = p.storage + tile_off(blk, p.kv_heads, h, 1);
      *reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c)) = src[c];
      *reinterpret_cast<uint4*>(tile + tile_chunk_off(slot, c + 4)) = src[c + 4];
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
