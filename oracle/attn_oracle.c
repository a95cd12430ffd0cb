/*
 * attn_oracle.c — CPU restatement of pooled's reference attention arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing on the product path (the CUDA library, its
 * Python host mirror) may include, link, load or call this file; it exists to
 * check the CUDA kernels and to be timed as the CPU baseline.
 *
 * pooled's attention path is JavaScript + WGSL, which cannot be compiled as C,
 * so every function here restates the reference's arithmetic and cites the
 * reference file:line it follows (paths relative to the pooled repository).
 * The reference's tests hold no numeric output vectors for this path: they
 * generate inputs from seeded LCGs and compare the GPU against float64 exact
 * attention computed in the test itself.  The pins are therefore (1) the f16
 * conversion rules, checked against an independent IEEE implementation over
 * every half and every rounding midpoint, (2) the reference tests' input
 * generators reproduced bit for bit, and (3) the float64 exact-attention
 * definition of the tests, cross-checked against an independent NumPy twin.
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -shared)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define PO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ f16 -- */

static inline uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* f32 -> f16 bits, round to nearest even, subnormals kept, overflow -> inf,
 * NaN -> quiet.  tests/reference/qsa_ref.mjs:64-79 (f16bits), the same rule as
 * engine/wgsl/f16.js:15-31 (f16_rne). */
PO_API uint16_t po_f16_rne(float x) {
  uint32_t i = f32_bits(x);
  uint32_t s = (i >> 16) & 0x8000u;
  int32_t e = (int32_t)((i >> 23) & 0xff) - 127 + 15;
  uint32_t m = i & 0x7fffffu;
  if (((i >> 23) & 0xff) == 0xff) return (uint16_t)(s | 0x7c00u | (m ? 0x200u : 0u));
  if (e >= 31) return (uint16_t)(s | 0x7c00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)s;
    uint32_t mm = m | 0x800000u, sh = (uint32_t)(14 - e);
    uint32_t h = mm >> sh, rem = mm & ((1u << sh) - 1u), half = 1u << (sh - 1);
    if (rem > half || (rem == half && (h & 1u))) h++;
    return (uint16_t)(s | h);
  }
  uint32_t h = s | ((uint32_t)e << 10) | (m >> 13);
  if ((m & 0x1fffu) > 0x1000u || ((m & 0x1fffu) == 0x1000u && (h & 1u))) h++;
  return (uint16_t)h;
}

/* f32 -> f16 bits with ties rounded up in magnitude: engine/gguf.js:17-37
 * (f32ToF16), the conversion tests/unit/attn_tile_test.js uses for its K/V. */
PO_API uint16_t po_f16_ties_up(float v) {
  uint32_t x = f32_bits(v);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t e = (int32_t)((x >> 23) & 0xff);
  uint32_t m = x & 0x7fffffu;
  if (e == 0xff) return (uint16_t)(sign | 0x7c00u | (m ? 0x200u : 0u));
  e = e - 127 + 15;
  if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign;
    m = (m | 0x800000u) >> (1 - e);
    return (uint16_t)(sign | ((m + 0x1000u) >> 13));
  }
  return (uint16_t)(sign | (((uint32_t)e << 10) + ((m + 0x1000u) >> 13)));
}

/* The local f16() of tests/test_attn_dec.js:24-25: the double is first stored
 * as f32, then rounded to nearest even; results below the f16 normal range are
 * flushed to signed zero and there is no NaN case. */
PO_API uint16_t po_f16_flush(double xd) {
  float x = (float)xd;
  uint32_t i = f32_bits(x);
  uint32_t s = (i >> 16) & 0x8000u;
  int32_t e = (int32_t)((i >> 23) & 0xff) - 127 + 15;
  uint32_t m = i & 0x7fffffu;
  if (e <= 0) return (uint16_t)s;
  if (e >= 31) return (uint16_t)(s | 0x7c00u);
  uint32_t h = s | ((uint32_t)e << 10) | (m >> 13);
  if ((m & 0x1fffu) > 0x1000u || ((m & 0x1fffu) == 0x1000u && (h & 1u))) h++;
  return (uint16_t)h;
}

/* f16 bits -> f32, exact for every input: engine/wgsl/f16.js:34-41 (f16_f32),
 * tests/reference/qsa_ref.mjs:80-84 (h2f). */
PO_API float po_h2f(uint16_t h) {
  uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  float v;
  if (e == 0) v = (float)m * 5.9604644775390625e-8f;
  else if (e == 31) v = bits_f32(0x7f800000u | (m << 13));
  else v = bits_f32(((e + 112u) << 23) | (m << 13));
  return (h & 0x8000u) ? -v : v;
}

PO_API void po_f16_rne_array(const float* x, uint16_t* h, size_t n) { for (size_t i = 0; i < n; i++) h[i] = po_f16_rne(x[i]); }
PO_API void po_h2f_array(const uint16_t* h, float* x, size_t n) { for (size_t i = 0; i < n; i++) x[i] = po_h2f(h[i]); }

/* ------------------------------------------------------------ head norm -- */

/* QK head-norm, the step before RoPE in the reference's attention glue: per head,
 * the sum of squares accumulated serially in double, inv = 1/sqrt(ss/n + eps),
 * out[i] = f32((x[i] * inv) * w[i]).  tests/reference/ref_q38.mjs:50-57 (rmsnorm)
 * as applied to the q and k heads at :163-164; the shader form (f32, thread 0
 * serial) is engine/wgsl/qwen35.js:1112-1122. */
PO_API void po_head_norm_f64(float* vec, uint32_t heads, uint32_t hd, const float* w, double eps) {
  for (uint32_t h = 0; h < heads; h++) {
    float* p = vec + (size_t)h * hd;
    double ss = 0.0;
    for (uint32_t i = 0; i < hd; i++) ss += (double)p[i] * (double)p[i];
    double inv = 1.0 / sqrt(ss / (double)hd + eps);
    for (uint32_t i = 0; i < hd; i++) p[i] = (float)(((double)p[i] * inv) * (double)w[i]);
  }
}

/* ----------------------------------------------------------------- RoPE -- */

/* NeoX rotation of the first n_rot dims of every head, pairs (i, i + n_rot/2),
 * angle pos * theta^(-2i/n_rot) evaluated in double, products in double, result
 * stored as f32.  tests/reference/ref_q38.mjs:67-79 (ropeNeox, partial) and
 * tests/reference/ref_qwen.mjs:32-44 (rope, n_rot == head_dim). */
PO_API void po_rope_neox_f64(float* vec, uint32_t heads, uint32_t hd, uint32_t n_rot, double pos, double theta) {
  uint32_t half = n_rot / 2;
  for (uint32_t h = 0; h < heads; h++) {
    float* p = vec + (size_t)h * hd;
    for (uint32_t i = 0; i < half; i++) {
      double ang = pos * pow(theta, -(2.0 * (double)i) / (double)n_rot);
      double c = cos(ang), s = sin(ang);
      double a = p[i], b = p[i + half];
      p[i] = (float)(a * c - b * s);
      p[i + half] = (float)(b * c + a * s);
    }
  }
}

/* ggml-style rotation: theta_0 = f32(pos), theta_{i+1} = f32(theta_i * ts),
 * ts = f32(base^(-2/n_rot)); cos/sin rounded to f32; every product and sum
 * rounded to f32.  tests/reference/qsa_ref.mjs:97-110 (rope), the recurrence
 * the Flash engine evaluates on the host (engine/qwen4exp.js:549-553). */
PO_API void po_rope_table_f32(float* cs, uint32_t n_rot, double pos, double base) {
  uint32_t half = n_rot / 2;
  float ts = (float)pow(base, -2.0 / (double)n_rot);
  float th = (float)pos;
  for (uint32_t i = 0; i < half; i++) {
    cs[2 * i] = (float)cos((double)th);
    cs[2 * i + 1] = (float)sin((double)th);
    th = th * ts;
  }
}
PO_API void po_rope_ggml_f32(float* vec, uint32_t heads, uint32_t hd, uint32_t n_rot, double pos, double base) {
  uint32_t half = n_rot / 2;
  float cs[512];
  po_rope_table_f32(cs, n_rot, pos, base);
  for (uint32_t h = 0; h < heads; h++) {
    float* p = vec + (size_t)h * hd;
    for (uint32_t i = 0; i < half; i++) {
      float c = cs[2 * i], s = cs[2 * i + 1];
      float a = p[i], b = p[i + half];
      volatile float ac = a * c, bs = b * s, as = a * s, bc = b * c; /* no contraction */
      p[i] = ac - bs;
      p[i + half] = as + bc;
    }
  }
}

/* ------------------------------------------------------------ KV append -- */

/* Row pos of each cache gets the f16 (RNE) image of the f32 k / v row, element
 * order unchanged.  engine/wgsl/qwen35.js:889-906 (kv_store); the bit rule is
 * pinned by tests/test_q38flash_mc.js:231-236. */
PO_API void po_kv_append(const float* k, const float* v, uint32_t kv_dim, uint64_t pos, uint16_t* k_cache, uint16_t* v_cache) {
  for (uint32_t i = 0; i < kv_dim; i++) {
    k_cache[pos * kv_dim + i] = po_f16_rne(k[i]);
    v_cache[pos * kv_dim + i] = po_f16_rne(v[i]);
  }
}

/* ------------------------------------------------------ exact attention -- */

/* Causal GQA attention in float64 over f16 K/V values.  Column c (query token
 * at position pos0 + c) attends rows [0, pos0 + c + 1); q head h uses kv head
 * floor(h / (nH/nKV)); score = dot / sqrt(hd); max-subtracted softmax; o / L.
 * tests/test_attn_dec.js:72-82 (ref) and tests/unit/attn_tile_test.js:63-78.
 * gate (optional, f32 [n_cols][gate_stride], laid out like q): out *= 1 / (1 +
 * exp(-g)), tests/reference/ref_q38.mjs:59,191.
 * Rows at or past a column's limit are never read. */
PO_API void po_attn_f64(const float* q, uint64_t q_stride, const uint16_t* k_cache, const uint16_t* v_cache,
                        uint32_t n_heads, uint32_t n_kv, uint32_t hd, uint64_t pos0, uint32_t n_cols,
                        const float* gate, uint64_t gate_stride, double* out, uint64_t out_stride) {
  uint32_t G = n_heads / n_kv, kv_dim = n_kv * hd;
  double rs = sqrt((double)hd);
  int total = (int)(n_cols * n_heads);
#pragma omp parallel for schedule(dynamic, 1)
  for (int job = 0; job < total; job++) {
    uint32_t col = (uint32_t)job / n_heads, h = (uint32_t)job % n_heads;
    uint32_t g = h / G;
    uint64_t n = pos0 + col + 1;
    double* sc = (double*)malloc(sizeof(double) * n);
    const float* qh = q + col * q_stride + (size_t)h * hd;
    double M = -INFINITY;
    for (uint64_t t = 0; t < n; t++) {
      const uint16_t* kr = k_cache + t * kv_dim + (size_t)g * hd;
      double s = 0;
      for (uint32_t d = 0; d < hd; d++) s += (double)qh[d] * (double)po_h2f(kr[d]);
      sc[t] = s / rs;
      if (sc[t] > M) M = sc[t];
    }
    double L = 0;
    for (uint64_t t = 0; t < n; t++) { sc[t] = exp(sc[t] - M); L += sc[t]; }
    double* o = out + col * out_stride + (size_t)h * hd;
    for (uint32_t d = 0; d < hd; d++) o[d] = 0;
    for (uint64_t t = 0; t < n; t++) {
      const uint16_t* vr = v_cache + t * kv_dim + (size_t)g * hd;
      double w = sc[t];
      for (uint32_t d = 0; d < hd; d++) o[d] += w * (double)po_h2f(vr[d]);
    }
    for (uint32_t d = 0; d < hd; d++) {
      o[d] /= L;
      if (gate) { double gg = gate[col * gate_stride + (size_t)h * hd + d]; o[d] *= 1.0 / (1.0 + exp(-gg)); }
    }
    free(sc);
  }
}

/* ------------------------------------------- int8 and f32 caches (kvQ8, dense) -- */

/* kv_store_q8 (engine/wgsl/qwen35.js:908-946): n values (a multiple of 32) of a K or V row; per block of 32,
 * scale = max|x| / 127 in f32, inv = 1 / scale (0 for an all-zero block), value = clamp(round(x * inv), -127, 127)
 * with WGSL's round (ties to even).  attn_flash_q8 (engine/wgsl/qwen35.js:97-139) reads value * scale. */
PO_API void po_kv_store_q8(const float* x, uint32_t n, int8_t* q, float* scales) {
  for (uint32_t b = 0; b < n / 32; b++) {
    float a = 0.0f;
    for (int i = 0; i < 32; i++) { float v = fabsf(x[b * 32 + i]); if (v > a) a = v; }
    float sc = a / 127.0f;
    float inv = sc > 0.0f ? 1.0f / sc : 0.0f;
    scales[b] = sc;
    for (int i = 0; i < 32; i++) {
      float r = nearbyintf(x[b * 32 + i] * inv);
      if (r < -127.0f) r = -127.0f;
      if (r > 127.0f) r = 127.0f;
      q[b * 32 + i] = (int8_t)(int)r;
    }
  }
}
PO_API void po_dequant_q8(const int8_t* q, const float* scales, uint32_t n, float* x) {
  for (uint32_t i = 0; i < n; i++) x[i] = (float)q[i] * scales[i / 32];
}

/* po_attn_f64 over f32 K/V values (an f32 cache as the dense engine keeps, engine/wgsl/dense.js:22-136, or the
 * dequantised values of an int8 cache): the same float64 definition, tests/test_attn_dec.js:72-82. */
PO_API void po_attn_f64_kv32(const float* q, uint64_t q_stride, const float* k_cache, const float* v_cache,
                             uint32_t n_heads, uint32_t n_kv, uint32_t hd, uint64_t pos0, uint32_t n_cols,
                             const float* gate, uint64_t gate_stride, double* out, uint64_t out_stride) {
  uint32_t G = n_heads / n_kv, kv_dim = n_kv * hd;
  double rs = sqrt((double)hd);
  int total = (int)(n_cols * n_heads);
#pragma omp parallel for schedule(dynamic, 1)
  for (int job = 0; job < total; job++) {
    uint32_t col = (uint32_t)job / n_heads, h = (uint32_t)job % n_heads;
    uint32_t g = h / G;
    uint64_t n = pos0 + col + 1;
    double* sc = (double*)malloc(sizeof(double) * n);
    const float* qh = q + col * q_stride + (size_t)h * hd;
    double M = -INFINITY;
    for (uint64_t t = 0; t < n; t++) {
      const float* kr = k_cache + t * kv_dim + (size_t)g * hd;
      double s = 0;
      for (uint32_t d = 0; d < hd; d++) s += (double)qh[d] * (double)kr[d];
      sc[t] = s / rs;
      if (sc[t] > M) M = sc[t];
    }
    double L = 0;
    for (uint64_t t = 0; t < n; t++) { sc[t] = exp(sc[t] - M); L += sc[t]; }
    double* o = out + col * out_stride + (size_t)h * hd;
    for (uint32_t d = 0; d < hd; d++) o[d] = 0;
    for (uint64_t t = 0; t < n; t++) {
      const float* vr = v_cache + t * kv_dim + (size_t)g * hd;
      double w = sc[t];
      for (uint32_t d = 0; d < hd; d++) o[d] += w * (double)vr[d];
    }
    for (uint32_t d = 0; d < hd; d++) {
      o[d] /= L;
      if (gate) { double gg = gate[col * gate_stride + (size_t)h * hd + d]; o[d] *= 1.0 / (1.0 + exp(-gg)); }
    }
    free(sc);
  }
}

/* The model-level reference's form of the same attention: scores and weights
 * stored as f32 (Float32Array sc), JavaScript double arithmetic in between,
 * the output accumulated into an f32 array one position at a time, gate
 * multiplied into the f32 result.  tests/reference/ref_q38.mjs:171-191 (hybrid
 * models, gated) and tests/reference/ref_qwen.mjs:113-131 (dense models). */
PO_API void po_attn_f32ref(const float* q, uint64_t q_stride, const uint16_t* k_cache, const uint16_t* v_cache,
                           uint32_t n_heads, uint32_t n_kv, uint32_t hd, uint64_t pos0, uint32_t n_cols,
                           const float* gate, uint64_t gate_stride, float* out, uint64_t out_stride) {
  uint32_t G = n_heads / n_kv, kv_dim = n_kv * hd;
  int total = (int)(n_cols * n_heads);
#pragma omp parallel for schedule(dynamic, 1)
  for (int job = 0; job < total; job++) {
    uint32_t col = (uint32_t)job / n_heads, h = (uint32_t)job % n_heads;
    uint32_t g = h / G;
    uint64_t n = pos0 + col + 1;
    float* sc = (float*)malloc(sizeof(float) * n);
    const float* qh = q + col * q_stride + (size_t)h * hd;
    for (uint64_t t = 0; t < n; t++) {
      const uint16_t* kr = k_cache + t * kv_dim + (size_t)g * hd;
      double acc = 0;
      for (uint32_t d = 0; d < hd; d++) acc += (double)qh[d] * (double)po_h2f(kr[d]);
      sc[t] = (float)(acc / sqrt((double)hd));
    }
    double mx = -INFINITY;
    for (uint64_t t = 0; t < n; t++) if (sc[t] > mx) mx = sc[t];
    double sum = 0;
    for (uint64_t t = 0; t < n; t++) { sc[t] = (float)exp((double)sc[t] - mx); sum += sc[t]; }
    float* o = out + col * out_stride + (size_t)h * hd;
    for (uint32_t d = 0; d < hd; d++) o[d] = 0;
    for (uint64_t t = 0; t < n; t++) {
      const uint16_t* vr = v_cache + t * kv_dim + (size_t)g * hd;
      double wt = (double)sc[t] / sum;
      for (uint32_t d = 0; d < hd; d++) o[d] = (float)((double)o[d] + wt * (double)po_h2f(vr[d]));
    }
    if (gate)
      for (uint32_t d = 0; d < hd; d++) {
        double gg = gate[col * gate_stride + (size_t)h * hd + d];
        o[d] = (float)((double)o[d] * (1.0 / (1.0 + exp(-gg))));
      }
    free(sc);
  }
}

/* --------------------------------------------- timed CPU baseline (f32) -- */

/* The same attention with f32 accumulation over the f16 cache, one pass with an
 * online softmax, threaded over (column, head).  This is the "reference CPU
 * path" that is timed beside the GPU kernels; it is never used as the parity
 * checker (po_attn_f64 is). */
PO_API void po_attn_f32_fast(const float* q, uint64_t q_stride, const uint16_t* k_cache, const uint16_t* v_cache,
                             uint32_t n_heads, uint32_t n_kv, uint32_t hd, uint64_t pos0, uint32_t n_cols,
                             const float* gate, uint64_t gate_stride, float* out, uint64_t out_stride) {
  uint32_t G = n_heads / n_kv, kv_dim = n_kv * hd;
  float rs = 1.0f / sqrtf((float)hd);
  int total = (int)(n_cols * n_heads);
  /* With fewer (column, head) jobs than threads the sequence is cut into chunks as well, each job leaving an
   * unnormalised (acc, m, l) record that is merged afterwards: every host thread gets work. */
  int nthr = 1;
#ifdef _OPENMP
  nthr = omp_get_max_threads();
#endif
  int chunks = 1;
  if (total < nthr) { chunks = (nthr + total - 1) / total; if (chunks > 64) chunks = 64; }
  float* part = (float*)malloc((size_t)total * chunks * (hd + 2) * sizeof(float));
  if (!part) return;
#pragma omp parallel for schedule(dynamic, 1)
  for (int job = 0; job < total * chunks; job++) {
    int rc = job / chunks, ch = job % chunks;
    uint32_t col = (uint32_t)rc / n_heads, h = (uint32_t)rc % n_heads;
    uint32_t g = h / G;
    uint64_t n = pos0 + col + 1;
    uint64_t per = (n + chunks - 1) / chunks, t0 = per * ch, t1 = t0 + per < n ? t0 + per : n;
    const float* qh = q + col * q_stride + (size_t)h * hd;
    float acc[512];
    float kf[512];
    for (uint32_t d = 0; d < hd; d++) acc[d] = 0;
    float m = -3.0e38f, l = 0;
    for (uint64_t t = t0; t < t1; t++) {
      const uint16_t* kr = k_cache + t * kv_dim + (size_t)g * hd;
      const uint16_t* vr = v_cache + t * kv_dim + (size_t)g * hd;
      for (uint32_t d = 0; d < hd; d++) kf[d] = po_h2f(kr[d]);
      float s = 0;
      for (uint32_t d = 0; d < hd; d++) s += qh[d] * kf[d];
      s *= rs;
      if (s > m) {
        float a = expf(m - s);
        for (uint32_t d = 0; d < hd; d++) acc[d] *= a;
        l *= a; m = s;
      }
      float p = expf(s - m);
      l += p;
      for (uint32_t d = 0; d < hd; d++) acc[d] += p * po_h2f(vr[d]);
    }
    float* pr = part + (size_t)job * (hd + 2);
    for (uint32_t d = 0; d < hd; d++) pr[d] = acc[d];
    pr[hd] = m; pr[hd + 1] = l;
  }
  for (int rc = 0; rc < total; rc++) {
    uint32_t col = (uint32_t)rc / n_heads, h = (uint32_t)rc % n_heads;
    const float* pr = part + (size_t)rc * chunks * (hd + 2);
    float M = -3.0e38f, L = 0;
    for (int c = 0; c < chunks; c++) if (pr[(size_t)c * (hd + 2) + hd] > M) M = pr[(size_t)c * (hd + 2) + hd];
    float* o = out + col * out_stride + (size_t)h * hd;
    for (uint32_t d = 0; d < hd; d++) o[d] = 0;
    for (int c = 0; c < chunks; c++) {
      const float* r = pr + (size_t)c * (hd + 2);
      float w = r[hd + 1] > 0 ? expf(r[hd] - M) : 0.0f;
      L += r[hd + 1] * w;
      for (uint32_t d = 0; d < hd; d++) o[d] += r[d] * w;
    }
    for (uint32_t d = 0; d < hd; d++) {
      float r = o[d] / L;
      if (gate) r *= 1.0f / (1.0f + expf(-gate[col * gate_stride + (size_t)h * hd + d]));
      o[d] = r;
    }
  }
  free(part);
}

/* Number of host threads the threaded functions use from now on (0 or less: leave as is). */
PO_API void po_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

PO_API int po_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------ log-sum-exp merge of split partials -- */

/* out = sum_s o_s exp(m_s - M) / sum_s l_s exp(m_s - M), M = max_s m_s, in
 * float64 (engine/wgsl/attn_dec.js:255-276 computes the same in f32). */
PO_API void po_lse_merge(const double* o, const double* m, const double* l, uint32_t n_parts, uint32_t hd, double* out) {
  double M = -INFINITY, L = 0;
  for (uint32_t s = 0; s < n_parts; s++) if (m[s] > M) M = m[s];
  for (uint32_t d = 0; d < hd; d++) out[d] = 0;
  for (uint32_t s = 0; s < n_parts; s++) {
    double w = exp(m[s] - M);
    L += l[s] * w;
    for (uint32_t d = 0; d < hd; d++) out[d] += o[(size_t)s * hd + d] * w;
  }
  for (uint32_t d = 0; d < hd; d++) out[d] /= L;
}

/* ------------------------------ the reference tests' input generators -- */

/* tests/test_attn_dec.js:22-23: seed = (seed * 1664525 + 1013904223) >>> 0,
 * rnd = seed / 2^32 - 0.5.  The product stays below 2^53, so integer
 * arithmetic reproduces JavaScript's double arithmetic exactly. */
PO_API uint32_t po_lcg_dec_next(uint32_t* seed) {
  *seed = (uint32_t)(((uint64_t)*seed * 1664525ull + 1013904223ull) & 0xffffffffull);
  return *seed;
}
static inline double lcg_dec_rnd(uint32_t* seed) { return (double)po_lcg_dec_next(seed) / 4294967296.0 - 0.5; }

/* One run() of tests/test_attn_dec.js:38-45: K[i] = f16(rnd * 0.6), V[i] =
 * f16(rnd * 2) interleaved per element, then q[i] = f32(rnd * 4) for 4 columns.
 * The seed is carried between runs (:106-107). */
PO_API void po_gen_attn_dec(uint32_t* seed, uint64_t n_kv_elems, uint16_t* K, uint16_t* V, uint64_t n_q, float* q) {
  for (uint64_t i = 0; i < n_kv_elems; i++) {
    K[i] = po_f16_flush(lcg_dec_rnd(seed) * 0.6);
    V[i] = po_f16_flush(lcg_dec_rnd(seed) * 2.0);
  }
  for (uint64_t i = 0; i < n_q; i++) q[i] = (float)(lcg_dec_rnd(seed) * 4.0);
}

/* tests/unit/attn_tile_test.js:16-17: seed = (seed * 1103515245 + 12345) >>> 0
 * evaluated in IEEE double (the product exceeds 2^53 and is rounded before the
 * ToUint32 reduction), rnd = seed / 2^32. */
PO_API uint32_t po_lcg_tile_next(uint32_t* seed) {
  double x = (double)*seed * 1103515245.0 + 12345.0;  /* both operations round to double, as in JS */
  double r = fmod(x, 4294967296.0);
  *seed = (uint32_t)r;
  return *seed;
}
static inline double lcg_tile_rnd(uint32_t* seed) { return (double)po_lcg_tile_next(seed) / 4294967296.0; }

/* check() of tests/unit/attn_tile_test.js:43-52: for every row p < max_seq and
 * pair w: K elems 2w, 2w+1 = (rnd-0.5)*2, then V elems 2w, 2w+1 = rnd-0.5, all
 * through f32ToF16 (ties up); rows at or past seq_end hold the NaN pattern
 * 0x7e00 but their draws are still consumed; then q = (rnd-0.5)*3 as f32 for
 * n_cols * s0 values, s0 = nH*hd + 12. */
PO_API void po_gen_attn_tile(uint32_t* seed, uint32_t max_seq, uint32_t kv_dim, uint32_t seq_end,
                             uint16_t* K, uint16_t* V, uint64_t n_q, float* q) {
  for (uint32_t p = 0; p < max_seq; p++)
    for (uint32_t w = 0; w < kv_dim / 2; w++) {
      uint16_t k0 = po_f16_ties_up((float)((lcg_tile_rnd(seed) - 0.5) * 2.0));
      uint16_t k1 = po_f16_ties_up((float)((lcg_tile_rnd(seed) - 0.5) * 2.0));
      uint16_t v0 = po_f16_ties_up((float)(lcg_tile_rnd(seed) - 0.5));
      uint16_t v1 = po_f16_ties_up((float)(lcg_tile_rnd(seed) - 0.5));
      int live = p < seq_end;
      K[(size_t)p * kv_dim + 2 * w] = live ? k0 : 0x7e00;
      K[(size_t)p * kv_dim + 2 * w + 1] = live ? k1 : 0x7e00;
      V[(size_t)p * kv_dim + 2 * w] = live ? v0 : 0x7e00;
      V[(size_t)p * kv_dim + 2 * w + 1] = live ? v1 : 0x7e00;
    }
  for (uint64_t i = 0; i < n_q; i++) q[i] = (float)((lcg_tile_rnd(seed) - 0.5) * 3.0);
}
