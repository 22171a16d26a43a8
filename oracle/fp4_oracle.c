/* CPU restatement in plain C of the NVFP4 producers of the FP4 hot path.
 * TEST INFRASTRUCTURE: used as the checker in tests and as the timed CPU baseline of
 * bench.py; never linked or called by the product library.
 *
 * The arithmetic follows the reference CUDA sources (paths relative to the reference root):
 *   scale rules   fp4_runtime/TK_quantisation/nvfp4_v5/core.cuh:36-113
 *   block math    fp4_runtime/TK_quantisation/nvfp4_v5/fused_amax_quantize.cuh:216-381
 *   scale tiles   fp4_runtime/TK_quantisation/nvfp4_v5/persistent_quantize.cuh:33-36
 *   RMSNorm       fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:1025-1111
 * It is validated against the numpy oracle (oracle/fp4_oracle.py), which in turn is pinned
 * to the golden vectors of the reference's CPU emulation.
 * Build: make -C oracle   (gcc -O2 -pthread -ffp-contract=off; no fast-math).  Rows are split
 * over ORACLE_THREADS threads (default: all online cores).
 */
#include <math.h>
#include <stdint.h>
#include <pthread.h>
#include <stdlib.h>
#include <unistd.h>
#include <string.h>

#define FLT_MAX_F 3.4028235e+38f


/* ---- minimal parallel-for over [0, n) with pthreads ---- */
typedef void (*range_fn)(int64_t lo, int64_t hi, void* ctx, int tid);
typedef struct { range_fn fn; void* ctx; int64_t lo, hi; int tid; } job_t;
static void* job_main(void* p) { job_t* j = (job_t*)p; j->fn(j->lo, j->hi, j->ctx, j->tid); return NULL; }
int oracle_num_threads(void) {
  const char* e = getenv("ORACLE_THREADS");
  long n = e ? atol(e) : sysconf(_SC_NPROCESSORS_ONLN);
  if (n < 1) n = 1; if (n > 256) n = 256;
  return (int)n;
}
static void parallel_for(int64_t n, range_fn fn, void* ctx) {
  int T = oracle_num_threads();
  if (T > n) T = (int)(n > 0 ? n : 1);
  pthread_t th[256]; job_t jobs[256];
  for (int t = 0; t < T; ++t) {
    jobs[t].fn = fn; jobs[t].ctx = ctx; jobs[t].tid = t;
    jobs[t].lo = n * t / T; jobs[t].hi = n * (t + 1) / T;
    if (t > 0) pthread_create(&th[t], NULL, job_main, &jobs[t]);
  }
  job_main(&jobs[0]);
  for (int t = 1; t < T; ++t) pthread_join(th[t], NULL);
}

static inline float bf16_to_f32(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* fp32 -> E4M3, RN-even, saturating (finite inputs >= 0 only are needed here) */
static uint8_t e4m3_encode(float x) {
  uint8_t sign = signbit(x) ? 0x80 : 0;
  double a = fabs((double)x);
  if (isnan(a)) return 0x7F;
  if (isinf(a)) return sign | 0x7E;
  if (a < 0.015625) { /* 2^-6 */
    int q = (int)nearbyint(a * 512.0);
    return sign | (uint8_t)q;
  }
  int ex; double m = frexp(a, &ex); /* a = m * 2^ex, m in [0.5,1) */
  int e = ex - 1;
  int q = (int)nearbyint((m * 2.0 - 1.0) * 8.0);
  if (q == 8) { q = 0; e += 1; }
  if (e > 8 || (e == 8 && q == 7)) return sign | 0x7E;
  return sign | (uint8_t)(((e + 7) << 3) | q);
}
static float e4m3_decode(uint8_t c) {
  int e = (c >> 3) & 0xF, m = c & 7;
  float v = e == 0 ? (float)m * 0.001953125f : (1.0f + (float)m / 8.0f) * ldexpf(1.0f, e - 7);
  return (c & 0x80) ? -v : v;
}
static inline uint8_t e2m1_encode(float v) {
  float a = fabsf(v); uint8_t i = 0;
  if (a > 0.25f) i = 1; if (a >= 0.75f) i = 2; if (a > 1.25f) i = 3; if (a >= 1.75f) i = 4;
  if (a > 2.5f) i = 5; if (a >= 3.5f) i = 6; if (a > 5.0f) i = 7;
  return i | (signbit(v) ? 8 : 0);
}
static float global_encode_scale(float amax) {
  if (amax == 0.0f) return 1.0f;
  float s = 2688.0f / amax;
  if (s > FLT_MAX_F) s = FLT_MAX_F;
  return s == 0.0f ? 1.0f : s;
}
static void block_scale(float b, float s_enc, int encode_centric, uint8_t* stored, float* coeff) {
  if (encode_centric) {
    uint8_t m8;
    if (b <= 1.0e-9f) m8 = 0x7E;
    else { float m = 6.0f / (b * s_enc); if (m > FLT_MAX_F) m = FLT_MAX_F; m8 = e4m3_encode(m); }
    float mf = e4m3_decode(m8);
    *coeff = mf * s_enc;
    *stored = e4m3_encode(1.0f / mf);
  } else {
    float s = b / 6.0f * s_enc; if (s > FLT_MAX_F) s = FLT_MAX_F;
    *stored = e4m3_encode(s);
    float s_dec = 1.0f / s_enc;
    float c = 1.0f / (e4m3_decode(*stored) * s_dec);
    *coeff = c > FLT_MAX_F ? FLT_MAX_F : c;
  }
}
static inline size_t scale_offset(int64_t r, int64_t kb, int64_t ntk) {
  return (size_t)(((r / 128) * ntk + kb / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + (kb % 4));
}

/* Quantise rows of v (bf16 bits, [R, C], leading dimension ld in elements, element (r,c) at
 * v[r*rs + c*cs]) along c in 16-blocks.  out [R, C/2], sc swizzled [R/128, C/64, 512]. */
typedef struct { const uint16_t* v; int64_t R, C, rs, cs; float s_enc; int ec; uint8_t* out; uint8_t* sc; } qa_ctx;
static void quantize_rows(int64_t lo, int64_t hi, void* p, int tid) {
  (void)tid;
  qa_ctx* q = (qa_ctx*)p;
  const int64_t nb = q->C / 16, ntk = q->C / 64;
  for (int64_t r = lo; r < hi; ++r) {
    for (int64_t kb = 0; kb < nb; ++kb) {
      float x[16], b = 0.0f;
      for (int i = 0; i < 16; ++i) { x[i] = bf16_to_f32(q->v[r * q->rs + (kb * 16 + i) * q->cs]); float a = fabsf(x[i]); if (a > b) b = a; }
      uint8_t st; float co; block_scale(b, q->s_enc, q->ec, &st, &co);
      q->sc[scale_offset(r, kb, ntk)] = st;
      for (int i = 0; i < 16; i += 2) {
        uint8_t l = e2m1_encode(x[i] * co), h = e2m1_encode(x[i + 1] * co);
        q->out[r * (q->C / 2) + kb * 8 + i / 2] = (uint8_t)(l | (h << 4));
      }
    }
  }
}
static void quantize_axis(const uint16_t* v, int64_t R, int64_t C, int64_t rs, int64_t cs, float s_enc,
                          int encode_centric, uint8_t* out, uint8_t* sc) {
  qa_ctx q = {v, R, C, rs, cs, s_enc, encode_centric, out, sc};
  parallel_for(R, quantize_rows, &q);
}

/* inv_rms with the summation tree of the reference pass-1 kernel */
static float row_inv_rms(const uint16_t* x, int64_t K, float eps) {
  float acc[256]; memset(acc, 0, sizeof acc);
  for (int64_t base = 0; base < K; base += 512) {
    int64_t n = (K - base < 512 ? K - base : 512) / 2;
    for (int64_t t = 0; t < n; ++t) {
      float a = bf16_to_f32(x[base + 2 * t]), b = bf16_to_f32(x[base + 2 * t + 1]);
      acc[t] = fmaf(a, a, acc[t]); acc[t] = fmaf(b, b, acc[t]);
    }
  }
  float w[8];
  for (int wp = 0; wp < 8; ++wp) {
    float v[32], t[32]; memcpy(v, acc + wp * 32, sizeof v);
    for (int mask = 16; mask > 0; mask >>= 1) { for (int l = 0; l < 32; ++l) t[l] = v[l] + v[l ^ mask]; memcpy(v, t, sizeof v); }
    w[wp] = v[0];
  }
  for (int mask = 4; mask > 0; mask >>= 1) { float t[8]; for (int l = 0; l < 8; ++l) t[l] = w[l] + w[l ^ mask]; memcpy(w, t, sizeof t); }
  float mean = w[0] / (float)K + eps;
  return (float)(1.0 / sqrt((double)mean));
}

/* Fused RMSNorm + NVFP4 row/column quantisation.  inv_rms: in/out [M] (computed when
 * compute_inv != 0).  normed: scratch [M*K] of bf16 bits (caller-allocated).  amax_sg[2] out. */
typedef struct { const uint16_t* x; const uint16_t* gamma; float eps; int64_t K; float* inv_rms; int compute_inv;
                 uint16_t* normed; float amax[256]; } nm_ctx;
static void norm_rows(int64_t lo, int64_t hi, void* p, int tid) {
  nm_ctx* c = (nm_ctx*)p;
  float amax = 0.0f;
  for (int64_t r = lo; r < hi; ++r) {
    if (c->compute_inv) c->inv_rms[r] = row_inv_rms(c->x + r * c->K, c->K, c->eps);
    const float inv = c->inv_rms[r];
    for (int64_t k = 0; k < c->K; ++k) {
      float t = bf16_to_f32(c->x[r * c->K + k]) * inv;
      t = t * bf16_to_f32(c->gamma[k]);
      uint16_t nb = f32_to_bf16(t);
      c->normed[r * c->K + k] = nb;
      float a = fabsf(bf16_to_f32(nb));
      if (a > amax) amax = a;
    }
  }
  c->amax[tid] = amax;
}
typedef struct { const uint16_t* x; float amax[256]; } am_ctx;
static void amax_range(int64_t lo, int64_t hi, void* p, int tid) {
  am_ctx* c = (am_ctx*)p; float amax = 0.0f;
  for (int64_t i = lo; i < hi; ++i) { float a = fabsf(bf16_to_f32(c->x[i])); if (a > amax) amax = a; }
  c->amax[tid] = amax;
}

/* Fused RMSNorm + NVFP4 row/column quantisation.  inv_rms: in/out [M] (computed when
 * compute_inv != 0).  normed: scratch [M*K] of bf16 bits (caller-allocated).  amax_sg[2] out. */
int oracle_fused_norm_quantize(const uint16_t* x, const uint16_t* gamma, float eps, int64_t M, int64_t K,
                               float* inv_rms, int compute_inv, int encode_centric, uint16_t* normed,
                               uint8_t* row_fp4, uint8_t* row_sc, uint8_t* col_fp4, uint8_t* col_sc,
                               float* amax_sg) {
  nm_ctx c; memset(&c, 0, sizeof c);
  c.x = x; c.gamma = gamma; c.eps = eps; c.K = K; c.inv_rms = inv_rms; c.compute_inv = compute_inv; c.normed = normed;
  parallel_for(M, norm_rows, &c);
  float amax = 0.0f;
  for (int t = 0; t < 256; ++t) if (c.amax[t] > amax) amax = c.amax[t];
  amax_sg[0] = amax; amax_sg[1] = amax / 2688.0f;
  const float s_enc = global_encode_scale(amax);
  quantize_axis(normed, M, K, K, 1, s_enc, encode_centric, row_fp4, row_sc);
  if (col_fp4) quantize_axis(normed, K, M, 1, K, s_enc, encode_centric, col_fp4, col_sc);
  return 0;
}

/* Plain row/column quantisation with tensor amax (tk_quantize_for_gemm). */
int oracle_quantize_for_gemm(const uint16_t* x, int64_t M, int64_t K, int encode_centric, uint8_t* row_fp4,
                             uint8_t* row_sc, uint8_t* col_fp4, uint8_t* col_sc, float* amax_sg) {
  am_ctx c; memset(&c, 0, sizeof c); c.x = x;
  parallel_for(M * K, amax_range, &c);
  float amax = 0.0f;
  for (int t = 0; t < 256; ++t) if (c.amax[t] > amax) amax = c.amax[t];
  amax_sg[0] = amax; amax_sg[1] = amax / 2688.0f;
  const float s_enc = global_encode_scale(amax);
  quantize_axis(x, M, K, K, 1, s_enc, encode_centric, row_fp4, row_sc);
  if (col_fp4) quantize_axis(x, K, M, 1, K, s_enc, encode_centric, col_fp4, col_sc);
  return 0;
}
