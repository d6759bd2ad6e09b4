/* TEST INFRASTRUCTURE — CPU restatement of the reference's KV-cache attention
 * path (see oracle.h for the contract and what pins it).  Plain C, OpenMP for
 * the timed CPU-baseline leg.  Built with -ffp-contract=off so that every
 * fused multiply-add below is an explicit fmaf(). */
#define _GNU_SOURCE
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define D ORC_HEAD_DIM
#define R ORC_ROTARY_DIM
#define BT ORC_BLOCK_TOKENS

void orc_gemm_bf16(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int m = 0; m < M; m++)
    for (int n = 0; n < N; n++) {
      double acc = 0.0;
      for (int k = 0; k < K; k++)
        acc += (double)orc_bf16_to_f32(A[(size_t)m * K + k]) * (double)orc_bf16_to_f32(B[(size_t)k * N + n]);
      C[(size_t)m * N + n] = orc_f32_to_bf16((float)acc);
    }
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---- bf16 <-> fp32 (round to nearest even, as __float2bfloat16) ---------- */
uint16_t orc_f32_to_bf16(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

float orc_bf16_to_f32(uint16_t x) {
  uint32_t u = (uint32_t)x << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* ---- RoPE tables: src/runtime/llama_runtime.cu:320-451 -------------------
 * All arithmetic in float, powf/cosf/sinf as std::pow/std::cos/std::sin on
 * float arguments resolve to. */
void orc_build_rope_tables(float* cos_table, float* sin_table, int seq_len) {
  const float theta = 500000.0f, factor = 32.0f, low_ff = 1.0f, high_ff = 4.0f,
              orig_ctx = 8192.0f;
  for (int pair = 0; pair < R; pair++) {
    float exponent = (float)(2 * pair) / (float)D;
    float inv_freq = 1.0f / powf(theta, exponent);
    float wavelen = 2.0f * (float)M_PI / inv_freq;
    float low_wl = orig_ctx / low_ff;
    float high_wl = orig_ctx / high_ff;
    float inv;
    if (wavelen < high_wl) {
      inv = inv_freq;
    } else if (wavelen <= low_wl) {
      float smooth = (orig_ctx / wavelen - low_ff) / (high_ff - low_ff);
      inv = (1.0f - smooth) * (inv_freq / factor) + smooth * inv_freq;
    } else {
      inv = inv_freq / factor;
    }
    for (int pos = 0; pos < seq_len; pos++) {
      float angle = (float)pos * inv;
      cos_table[(size_t)pos * R + pair] = cosf(angle);
      sin_table[(size_t)pos * R + pair] = sinf(angle);
    }
  }
}

/* ---- RoPE: src/kernels/rope/rope.cu:23-210 ------------------------------- */
void orc_rope(const uint16_t* in, uint16_t* out, const float* cos_table,
              const float* sin_table, int tokens, int heads,
              int position_offset, int y0_variant, int out_token_major) {
  for (int t = 0; t < tokens; t++) {
    const float* c_row = cos_table + (size_t)(t + position_offset) * R;
    const float* s_row = sin_table + (size_t)(t + position_offset) * R;
    for (int h = 0; h < heads; h++) {
      const uint16_t* x = in + ((size_t)t * heads + h) * D;
      uint16_t* y = out_token_major ? out + ((size_t)t * heads + h) * D
                                    : out + ((size_t)h * tokens + t) * D;
      for (int i = 0; i < R; i++) {
        float c = c_row[i], s = s_row[i];
        float x0 = orc_bf16_to_f32(x[i]);
        float x1 = orc_bf16_to_f32(x[i + R]);
        float y0;
        if (y0_variant == 0) {
          float a = x0 * c, b = x1 * s;
          y0 = a - b;
        } else if (y0_variant == 1) {
          float b = x1 * s;
          y0 = fmaf(x0, c, -b);
        } else {
          float a = x0 * c;
          y0 = fmaf(-x1, s, a);
        }
        float b1 = x1 * c;
        float y1 = fmaf(x0, s, b1);
        y[i] = orc_f32_to_bf16(y0);
        y[i + R] = orc_f32_to_bf16(y1);
      }
    }
  }
}

/* ---- V transpose: src/kernels/rope/rope.cu:211-262 ----------------------- */
void orc_transpose_v(const uint16_t* v_in, uint16_t* v_out, int tokens,
                     int kv_heads) {
  for (int t = 0; t < tokens; t++)
    for (int h = 0; h < kv_heads; h++)
      memcpy(v_out + ((size_t)h * tokens + t) * D,
             v_in + ((size_t)t * kv_heads + h) * D, D * sizeof(uint16_t));
}

/* ---- contiguous append: src/runtime/attention.cu:239-262 ----------------- */
void orc_append_contig(uint16_t* cache, const uint16_t* flash, int kv_heads,
                       int max_seq_len, int position, int tokens) {
  for (int h = 0; h < kv_heads; h++)
    for (int t = 0; t < tokens; t++)
      memcpy(cache + (size_t)h * max_seq_len * D + (size_t)(position + t) * D,
             flash + (size_t)h * tokens * D + (size_t)t * D,
             D * sizeof(uint16_t));
}

/* ---- paged placement model ----------------------------------------------- */
static size_t pool_off(int kv_heads, int block, int head, int kv, int slot) {
  return ((((size_t)block * kv_heads + head) * 2 + kv) * BT + slot) * D;
}

void orc_paged_append(uint16_t* pool, int kv_heads, const int32_t* table,
                      const uint16_t* k_flash, const uint16_t* v_flash,
                      int position, int tokens) {
  for (int h = 0; h < kv_heads; h++)
    for (int t = 0; t < tokens; t++) {
      int p = position + t;
      int blk = table[p / BT], slot = p % BT;
      memcpy(pool + pool_off(kv_heads, blk, h, 0, slot),
             k_flash + ((size_t)h * tokens + t) * D, D * sizeof(uint16_t));
      memcpy(pool + pool_off(kv_heads, blk, h, 1, slot),
             v_flash + ((size_t)h * tokens + t) * D, D * sizeof(uint16_t));
    }
}

void orc_paged_gather(const uint16_t* pool, int kv_heads, const int32_t* table,
                      int length, uint16_t* k_out, uint16_t* v_out,
                      int out_stride_tokens) {
  for (int h = 0; h < kv_heads; h++)
    for (int p = 0; p < length; p++) {
      int blk = table[p / BT], slot = p % BT;
      memcpy(k_out + ((size_t)h * out_stride_tokens + p) * D,
             pool + pool_off(kv_heads, blk, h, 0, slot), D * sizeof(uint16_t));
      memcpy(v_out + ((size_t)h * out_stride_tokens + p) * D,
             pool + pool_off(kv_heads, blk, h, 1, slot), D * sizeof(uint16_t));
    }
}

/* ---- attention core ------------------------------------------------------
 * One query row against keys [j0, j1) of one KV head; rows are fetched
 * through row_ptr() so the contiguous and the paged caller share it.
 * Produces the un-normalised accumulator, the running max (of scaled scores)
 * and the sum of exp(score - max). */
typedef struct {
  const uint16_t* K;
  const uint16_t* V;       /* contiguous: per-head base pointers            */
  const uint16_t* pool;    /* paged: logical pool + table                   */
  const int32_t* table;
  int kv_heads, head;
} kv_src;

static inline const uint16_t* k_row(const kv_src* s, int j) {
  if (s->pool)
    return s->pool + pool_off(s->kv_heads, s->table[j / BT], s->head, 0, j % BT);
  return s->K + (size_t)j * D;
}
static inline const uint16_t* v_row(const kv_src* s, int j) {
  if (s->pool)
    return s->pool + pool_off(s->kv_heads, s->table[j / BT], s->head, 1, j % BT);
  return s->V + (size_t)j * D;
}

static void attend_range(const float* qf, const kv_src* src, int j0, int j1,
                         float scale, int round_p, float* scores, float* acc,
                         float* m_out, float* l_out) {
  float m = -INFINITY;
  for (int j = j0; j < j1; j++) {
    const uint16_t* kr = k_row(src, j);
    float part[16] = {0};
    for (int d = 0; d < D; d += 16)
      for (int u = 0; u < 16; u++)
        part[u] += qf[d + u] * orc_bf16_to_f32(kr[d + u]);
    float dot = 0.f;
    for (int u = 0; u < 16; u++) dot += part[u];
    float s = dot * scale;
    scores[j - j0] = s;
    if (s > m) m = s;
  }
  float l = 0.f;
  for (int d = 0; d < D; d++) acc[d] = 0.f;
  for (int j = j0; j < j1; j++) {
    float p = expf(scores[j - j0] - m);
    l += p;
    float pv = round_p ? orc_bf16_to_f32(orc_f32_to_bf16(p)) : p;
    const uint16_t* vr = v_row(src, j);
    for (int d = 0; d < D; d++) acc[d] += pv * orc_bf16_to_f32(vr[d]);
  }
  *m_out = m;
  *l_out = l;
}

#define CHUNK 4096

/* Merge un-normalised partials (acc, m, l) of one row into out / lse. */
static void merge_row(const float* acc, const float* m, const float* l,
                      int n_chunks, float* out, float* lse) {
  float M = -INFINITY;
  for (int c = 0; c < n_chunks; c++)
    if (m[c] > M) M = m[c];
  double L = 0.0;
  double o[D];
  for (int d = 0; d < D; d++) o[d] = 0.0;
  for (int c = 0; c < n_chunks; c++) {
    if (m[c] == -INFINITY) continue;
    double w = exp((double)m[c] - (double)M);
    L += w * l[c];
    for (int d = 0; d < D; d++) o[d] += w * acc[(size_t)c * D + d];
  }
  for (int d = 0; d < D; d++) out[d] = (L > 0.0) ? (float)(o[d] / L) : 0.f;
  if (lse) *lse = (L > 0.0) ? (float)((double)M + log(L)) : -INFINITY;
}

void orc_attention(const uint16_t* Q, const uint16_t* K, const uint16_t* V,
                   float* O, float* LSE, int q_heads, int kv_heads,
                   int q_seq_len, int kv_seq_len, int kv_stride, float scale,
                   int causal, int round_p_bf16) {
  const int group = q_heads / kv_heads;
  const int q_off = kv_seq_len - q_seq_len;
  const int max_chunks = (kv_seq_len + CHUNK - 1) / CHUNK;
  const long rows = (long)q_heads * q_seq_len;
  const long items = rows * max_chunks;
  float* p_acc = (float*)malloc((size_t)items * D * sizeof(float));
  float* p_m = (float*)malloc((size_t)items * sizeof(float));
  float* p_l = (float*)malloc((size_t)items * sizeof(float));
#pragma omp parallel
  {
    float* scores = (float*)malloc(CHUNK * sizeof(float));
    float qf[D];
#pragma omp for schedule(dynamic, 4)
    for (long it = 0; it < items; it++) {
      long row = it / max_chunks;
      int c = (int)(it % max_chunks);
      int h = (int)(row / q_seq_len), i = (int)(row % q_seq_len);
      int visible = causal ? q_off + i + 1 : kv_seq_len;
      if (visible > kv_seq_len) visible = kv_seq_len;
      if (visible < 0) visible = 0;
      int j0 = c * CHUNK, j1 = j0 + CHUNK;
      if (j1 > visible) j1 = visible;
      if (j0 >= j1) {
        p_m[it] = -INFINITY;
        p_l[it] = 0.f;
        continue;
      }
      const uint16_t* q = Q + ((size_t)h * q_seq_len + i) * D;
      for (int d = 0; d < D; d++) qf[d] = orc_bf16_to_f32(q[d]);
      kv_src src = {K + (size_t)(h / group) * kv_stride * D,
                    V + (size_t)(h / group) * kv_stride * D, NULL, NULL,
                    kv_heads, h / group};
      attend_range(qf, &src, j0, j1, scale, round_p_bf16, scores,
                   p_acc + (size_t)it * D, &p_m[it], &p_l[it]);
    }
    free(scores);
#pragma omp for schedule(static)
    for (long row = 0; row < rows; row++)
      merge_row(p_acc + (size_t)row * max_chunks * D, p_m + row * max_chunks,
                p_l + row * max_chunks, max_chunks, O + (size_t)row * D,
                LSE ? LSE + row : NULL);
  }
  free(p_acc);
  free(p_m);
  free(p_l);
}

void orc_decode_paged(const uint16_t* q, const uint16_t* pool, int q_heads,
                      int kv_heads, const int32_t* table, int tok_begin,
                      int tok_end, float scale, float* out, float* lse) {
  const int group = q_heads / kv_heads;
  int len = tok_end - tok_begin;
  if (len < 0) len = 0;
  const int max_chunks = len > 0 ? (len + CHUNK - 1) / CHUNK : 1;
  const long items = (long)q_heads * max_chunks;
  float* p_acc = (float*)malloc((size_t)items * D * sizeof(float));
  float* p_m = (float*)malloc((size_t)items * sizeof(float));
  float* p_l = (float*)malloc((size_t)items * sizeof(float));
#pragma omp parallel
  {
    float* scores = (float*)malloc(CHUNK * sizeof(float));
    float qf[D];
#pragma omp for schedule(dynamic, 1)
    for (long it = 0; it < items; it++) {
      int h = (int)(it / max_chunks), c = (int)(it % max_chunks);
      int j0 = tok_begin + c * CHUNK, j1 = j0 + CHUNK;
      if (j1 > tok_end) j1 = tok_end;
      if (j0 >= j1) {
        p_m[it] = -INFINITY;
        p_l[it] = 0.f;
        continue;
      }
      for (int d = 0; d < D; d++) qf[d] = orc_bf16_to_f32(q[(size_t)h * D + d]);
      kv_src src = {NULL, NULL, pool, table, kv_heads, h / group};
      attend_range(qf, &src, j0, j1, scale, 0, scores, p_acc + (size_t)it * D,
                   &p_m[it], &p_l[it]);
    }
    free(scores);
#pragma omp for schedule(static)
    for (int h = 0; h < q_heads; h++)
      merge_row(p_acc + (size_t)h * max_chunks * D, p_m + (size_t)h * max_chunks,
                p_l + (size_t)h * max_chunks, max_chunks, out + (size_t)h * D,
                lse ? lse + h : NULL);
  }
  free(p_acc);
  free(p_m);
  free(p_l);
}

void orc_lse_merge(const float* O_parts, const float* lse_parts, int n_parts,
                   int rows, float* O, float* lse) {
  for (int r = 0; r < rows; r++) {
    double M = -INFINITY;
    for (int p = 0; p < n_parts; p++) {
      double v = lse_parts[(size_t)p * rows + r];
      if (v > M) M = v;
    }
    double L = 0.0, o[D];
    for (int d = 0; d < D; d++) o[d] = 0.0;
    if (M > -INFINITY) {
      for (int p = 0; p < n_parts; p++) {
        double v = lse_parts[(size_t)p * rows + r];
        if (v == -INFINITY) continue;
        double w = exp(v - M);
        L += w;
        const float* op = O_parts + ((size_t)p * rows + r) * D;
        for (int d = 0; d < D; d++) o[d] += w * op[d];
      }
    }
    for (int d = 0; d < D; d++)
      O[(size_t)r * D + d] = (L > 0.0) ? (float)(o[d] / L) : 0.f;
    if (lse) lse[r] = (L > 0.0) ? (float)(M + log(L)) : -INFINITY;
  }
}

/* ---- output layout: src/runtime/layout.cu:11-42 -------------------------- */
void orc_output_layout_f32(const float* in, float* out, int heads, int tokens) {
  for (int h = 0; h < heads; h++)
    for (int t = 0; t < tokens; t++)
      memcpy(out + ((size_t)t * heads + h) * D, in + ((size_t)h * tokens + t) * D,
             D * sizeof(float));
}
void orc_output_layout_bf16(const uint16_t* in, uint16_t* out, int heads,
                            int tokens) {
  for (int h = 0; h < heads; h++)
    for (int t = 0; t < tokens; t++)
      memcpy(out + ((size_t)t * heads + h) * D, in + ((size_t)h * tokens + t) * D,
             D * sizeof(uint16_t));
}

/* ---- RMSNorm: src/kernels/rmsnorm/rmsnorm.cu:51-110 -------------------------
 * y = bf16((x * r) * w), r = 1/sqrt(mean(x^2) + eps), all in fp32.  The sum of squares follows
 * the kernel's order for its launch with 256 threads: thread t sums the squares of its 8-element
 * chunks (t, t + 256, ...) with fused multiply-adds (the compiler contracts `s += v*v`), the 32
 * lanes of a warp combine by shuffle-down 16, 8, 4, 2, 1 (lane i adds lane i + offset), and the
 * warp totals combine the same way in the first warp (:9-46).  The kernel's rsqrtf is a hardware
 * approximation (2 ulp); 1/sqrtf here can differ from it in the last bits, which moves an output
 * by at most one bf16 ulp. */
static float shuffle_down_sum(const float* lanes_in) {
  float v[64];
  for (int i = 0; i < 32; i++) v[i] = lanes_in[i];
  for (int i = 32; i < 64; i++) v[i] = 0.f;
  for (int off = 16; off > 0; off >>= 1) {
    float nv[32];
    /* a lane beyond the warp (i + off >= 32) reads its own value back */
    for (int i = 0; i < 32; i++) nv[i] = v[i] + (i + off < 32 ? v[i + off] : v[i]);
    for (int i = 0; i < 32; i++) v[i] = nv[i];
  }
  return v[0];
}

void orc_rmsnorm(const uint16_t* x, const uint16_t* w, uint16_t* y, int rows, int hidden, float eps) {
  const int chunks = hidden / 8;
  for (int r = 0; r < rows; r++) {
    const uint16_t* xr = x + (size_t)r * hidden;
    float thread_sum[256];
    for (int t = 0; t < 256; t++) {
      float s = 0.f;
      for (int i = t; i < chunks; i += 256)
        for (int j = 0; j < 8; j++) {
          const float v = orc_bf16_to_f32(xr[i * 8 + j]);
          s = fmaf(v, v, s);
        }
      thread_sum[t] = s;
    }
    float warp_sum[32];
    for (int i = 0; i < 32; i++) warp_sum[i] = 0.f;
    for (int wdx = 0; wdx < 8; wdx++) warp_sum[wdx] = shuffle_down_sum(thread_sum + 32 * wdx);
    const float total = shuffle_down_sum(warp_sum);
    const float recip = 1.0f / sqrtf(total / (float)hidden + eps);
    for (int k = 0; k < hidden; k++) {
      const float xr_k = orc_bf16_to_f32(xr[k]);
      y[(size_t)r * hidden + k] = orc_f32_to_bf16((xr_k * recip) * orc_bf16_to_f32(w[k]));
    }
  }
}

/* h = bf16((g * (1 / (1 + exp(-g)))) * u) on bf16 gate and up values, as silu_mul of the
 * reference's activation kernel does in fp32 (src/kernels/silu/silu_8192.cu:55-100; the device
 * evaluates exp with __expf, here it is expf: results may differ in the last bf16 bit). */
void orc_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, long long n) {
  for (long long i = 0; i < n; i++) {
    const float g = orc_bf16_to_f32(gate[i]), u = orc_bf16_to_f32(up[i]);
    const float s = g * (1.0f / (1.0f + expf(-g)));
    out[i] = orc_f32_to_bf16(s * u);
  }
}
