// Device-side building blocks shared by the sm_100a kernels: mbarrier waits
// with a time limit, bulk (TMA) copies, ldmatrix / mma.sync wrappers and the
// address arithmetic of the cache layout.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pa {

constexpr int kHeadDim = 64;
constexpr int kGroup = 4;          // query heads per KV head
constexpr int kBlockTok = 16;      // tokens per cache block
constexpr int kTileBytes = 2048;   // one (block, head) K or V tile: 16 rows of 128 bytes
constexpr int kPairBytes = 4096;   // K tile followed by V tile of one (block, head)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Status values a kernel may record in the pool's device status word.
constexpr int kStatusTimeout = 5;
constexpr int kStatusBadBlock = 1;

// Descriptor of one batch entry, uploaded by pa_batch_set.
struct BatchEntry {
  int32_t seq;         // sequence id (row of the device table mirror)
  int32_t kv_len;      // tokens in the local cache including this step's new ones
  int32_t n_new;       // tokens appended to the local cache this step
  int32_t kv_row_off;  // first row of this sequence in k_in/v_in
  int32_t n_q;         // query rows of this sequence this step
  int32_t q_row_off;   // first row of this sequence in q_in/q_out
  int32_t q_pos0;      // RoPE position of its first query row
  int32_t kv_pos_off;  // RoPE position of local token 0 (0 unless the sequence is range-sharded)
};

// Byte offset of chunk `c` (16 bytes, 0..7) of token slot `r` (0..15) inside a
// tile: rows of 128 bytes, chunks XOR-swizzled with the row index.
__host__ __device__ __forceinline__ int tile_chunk_off(int r, int c) {
  return r * 128 + ((c ^ (r & 7)) << 4);
}

// Byte offset of tile (block, head, kv) inside one layer's storage.
__host__ __device__ __forceinline__ size_t tile_off(int block, int kv_heads, int head, int kv) {
  return (((size_t)block * kv_heads + head) * 2 + kv) * (size_t)kTileBytes;
}

// ---- shared-memory addresses and barriers -----------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Deadline of a polling loop.  %globaltimer is a slow register, so it is not
// read when a wait begins: the first read happens after 256 polls and starts
// the clock, later reads (every 256 polls) compare against the limit.
constexpr uint64_t kWaitLimitNs = 1000000000ull;
struct SpinDeadline {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  // call once per failed poll; true = the limit (~1 s) ran out
  __device__ __forceinline__ bool expired() {
    if ((++spins & 255u) != 0) return false;
    const uint64_t now = global_ns();
    if (t0 == 0) {
      t0 = now;
      return false;
    }
    return now - t0 > kWaitLimitNs;
  }
  __device__ __forceinline__ void restart() {
    spins = 0;
    t0 = 0;
  }
};
// Wait for the phase with the given parity, at most ~1 s.  Returns false when
// the limit ran out (the caller records it and leaves).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  SpinDeadline dl;
  while (!mbar_test(bar, parity)) {
    if (dl.expired()) return false;
  }
  return true;
}

// Bulk copy global -> shared, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---- warp-level matrix helpers (legacy tensor path, used by decode only) -----
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                        uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                          uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace pa
