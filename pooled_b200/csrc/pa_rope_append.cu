// RoPE (full or partial, NeoX pairing), the f16 KV-cache append and the standalone sigmoid gate.
//
// One small CTA per (column, head), or one CTA per column for prefill chunks.
//   PA_ROPE_F64    angle = pos * inv_freq[i] in float64 (inv_freq = theta^(-2i/n_rot) comes from the host's
//                  libm), cos / sin in float64, the two products and their difference / sum rounded one by
//                  one in float64, the result rounded to f32 — the arithmetic of pooled's CPU reference
//                  (tests/reference/ref_q38.mjs:67-79).  cos / sin come from a table that pa_angles_kernel fills
//                  once per (position, width) and every layer of the step reuses; the rotation itself is
//                  rot_exact(): the same bits as the float64 expression at f32 cost.
//   PA_ROPE_TABLE  cos / sin read from the caller's f32 table, products and sums rounded one by one in f32
//                  (the Flash engine's host table, engine/qwen4exp.js:549-553).
// K is rotated, rounded to f32 and then to f16 (round to nearest even) into row pos + col of the K cache;
// V is converted only.  Stands in for rope_part(_mc), kv_store and attn_glue_kv of pooled
// (engine/wgsl/qwen35.js:386-404, :858-906; engine/wgsl/layer_fuse.js:87-146).
#include "pa_params.cuh"

namespace pa {

__device__ __forceinline__ float ld_act(const void* p, uint64_t i, int f16) {
  return f16 ? __half2float(reinterpret_cast<const __half*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}

// f32 -> f16 round to nearest even with subnormals and overflow to inf (cvt.rn.f16.f32); NaN becomes the quiet
// pattern sign | 0x7e00 that pooled's f16_rne produces (engine/wgsl/f16.js:22), not the hardware's 0x7fff
__device__ __forceinline__ __half f16_rne(float x) {
  if (x != x) return __ushort_as_half((unsigned short)(((__float_as_uint(x) >> 16) & 0x8000u) | 0x7e00u));
  return __float2half_rn(x);
}

// grid (n_cols, q heads + k heads + v heads); one thread per pair of elements of the head.  Thread t < n_rot/2
// evaluates its own cos / sin and rotates dims (t, t + n_rot/2); the other threads pass dims n_rot + 2(t - n_rot/2),
// +1 through.  No shared memory and no barrier: every global load of the call is in flight at once, which is what
// the latency of a one-token call consists of.
__global__ void __launch_bounds__(128) pa_rope_append_kernel(const RopeParams p) {
  const uint32_t col = blockIdx.x, half = p.n_rot / 2, hd = p.hd, pr = threadIdx.x;
  // The kernel after this one may start fetching old cache rows while this one runs (it never touches the rows or
  // the rotated q written here before its own wait); this kernel itself writes nothing before its predecessor ends.
  // by-value angles go through shared memory: launch parameters indexed differently by every thread are served one
  // address at a time.  Done ahead of the wait, while the predecessor still runs.
  __shared__ Angle s_ang[64];
  if (p.trigger_early) pdl_trigger();
  if (p.n_ang) {
    if (threadIdx.x < p.n_ang * 2) reinterpret_cast<uint4*>(s_ang)[threadIdx.x] = reinterpret_cast<const uint4*>(p.ang)[threadIdx.x];
    __syncthreads();
  }
  // an angle this thread evaluates itself needs nothing of the predecessor's: ahead of the wait
  const uint32_t pos_c = p.n_items ? p.item_pos[col] : p.pos + col;
  Angle g_own;
  const bool own_angle = p.mode == PA_ROPE_F64 && !p.n_ang && !p.angles && pr < half && (p.q || p.k);
  if (own_angle) {
    double s, c;
    sincos(__dmul_rn((double)pos_c, p.inv_freq[pr]), &s, &c);
    g_own = make_angle(c, s);
  }
  pdl_wait();
  if (!p.trigger_early) pdl_trigger();
  if (pr >= hd / 2) return;
  const uint32_t nq = p.q ? p.q_heads : 0, nk = p.k ? p.kv_heads : 0;
  uint32_t slot = blockIdx.y;
  const uint64_t row_c = p.n_items ? p.item_row[col] : p.cache_row0 + col;
  if (slot >= nq && row_c == ~0ull) return;   // an item whose row another shard holds: nothing to append
  if (slot >= nq + nk) {
    // V head: conversion only
    const uint32_t head = slot - nq - nk, kvd = p.kv_heads * hd;
    const uint64_t so = (uint64_t)col * p.v_col_stride + (uint64_t)head * hd + 2 * pr;
    __half* dst = p.v_cache + row_c * (uint64_t)kvd + (uint64_t)head * hd + 2 * pr;
    dst[0] = f16_rne(ld_act(p.v, so, p.in_f16));
    dst[1] = f16_rne(ld_act(p.v, so + 1, p.in_f16));
    return;
  }
  const bool is_q = slot < nq;
  const uint32_t head = is_q ? slot : slot - nq;
  uint32_t d0, d1;
  const bool rot = p.mode != PA_ROPE_NONE && pr < half;
  if (pr < half) { d0 = pr; d1 = pr + half; } else { d0 = p.n_rot + 2 * (pr - half); d1 = d0 + 1; }
  const void* src = is_q ? p.q : p.k;
  const uint64_t sb = is_q ? (uint64_t)col * p.q_col_stride + (uint64_t)head * p.q_head_stride
                           : (uint64_t)col * p.kv_col_stride + (uint64_t)head * hd;
  const float a = ld_act(src, sb + d0, p.in_f16), b = ld_act(src, sb + d1, p.in_f16);
  float ra = a, rb = b;
  if (rot) {
    if (p.mode == PA_ROPE_F64) {
      Angle g;
      if (p.n_ang) g = s_ang[col * half + pr];
      else if (p.angles) g = p.angles[(uint64_t)col * half + pr];
      else g = g_own;
      ra = rot_exact(a, b, g, true);     // a cos - b sin
      rb = rot_exact(b, a, g, false);    // b cos + a sin
    } else {
      const float c = p.cs_table[(uint64_t)col * p.n_rot + 2 * pr], s = p.cs_table[(uint64_t)col * p.n_rot + 2 * pr + 1];
      ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
      rb = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
    }
  }
  if (is_q) {
    const uint64_t o = (uint64_t)col * p.q_out_col_stride + (uint64_t)head * hd;
    if (p.q_out_f16 == 2) {   // high and low f16 parts for the verify kernel's hi / lo rows
      __half* dst = reinterpret_cast<__half*>(p.q_out) + o;
      const __half ha = __float2half_rn(ra), hb = __float2half_rn(rb);
      dst[d0] = ha; dst[d1] = hb;
      dst[p.q_lo_offset + d0] = __float2half_rn(ra - __half2float(ha)); dst[p.q_lo_offset + d1] = __float2half_rn(rb - __half2float(hb));
    } else if (p.q_out_f16) { __half* dst = reinterpret_cast<__half*>(p.q_out) + o; dst[d0] = __float2half_rn(ra); dst[d1] = __float2half_rn(rb); }
    else { float* dst = reinterpret_cast<float*>(p.q_out) + o; dst[d0] = ra; dst[d1] = rb; }
  } else {
    __half* dst = p.k_cache + row_c * (uint64_t)(p.kv_heads * hd) + (uint64_t)head * hd;
    dst[d0] = f16_rne(ra); dst[d1] = f16_rne(rb);
  }
}

// Many columns (prefill chunks): one 256-thread CTA per column.  The column's n_rot/2 angles are evaluated once and
// shared by every head through shared memory; each thread then takes (head, pair) items four at a time so that its
// loads overlap.  Same arithmetic, element for element, as the per-head kernel above.
__global__ void __launch_bounds__(256) pa_rope_append_cols_kernel(const RopeParams p) {
  __shared__ Angle s_g[128];
  const uint32_t col = blockIdx.x, half = p.n_rot / 2, hd = p.hd, pairs = hd / 2;
  if (p.trigger_early) pdl_trigger();
  pdl_wait();
  if (!p.trigger_early) pdl_trigger();
  if (p.mode == PA_ROPE_F64) {
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
      if (p.n_ang) s_g[i] = p.ang[col * half + i];
      else if (p.angles) s_g[i] = p.angles[(uint64_t)col * half + i];
      else {
        double sv, cv;
        sincos(__dmul_rn((double)(p.pos + col), p.inv_freq[i]), &sv, &cv);
        s_g[i] = make_angle(cv, sv);
      }
    }
  }
  __syncthreads();
  const uint32_t nq = p.q ? p.q_heads * pairs : 0, nk = p.k ? p.kv_heads * pairs : 0, nv = p.v ? p.kv_heads * pairs : 0;
  const uint32_t total = nq + nk + nv, kvd = p.kv_heads * hd;
  for (uint32_t w0 = threadIdx.x; w0 < total; w0 += 4 * blockDim.x) {
    float a[4], b[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t w = w0 + u * blockDim.x;
      a[u] = b[u] = 0.f;
      if (w >= total) continue;
      if (w >= nq + nk) {                      // V: elements 2i, 2i+1
        const uint64_t so = (uint64_t)col * p.v_col_stride + 2 * (w - nq - nk);
        a[u] = ld_act(p.v, so, p.in_f16); b[u] = ld_act(p.v, so + 1, p.in_f16);
      } else {
        const bool is_q = w < nq;
        const uint32_t ww = is_q ? w : w - nq, head = ww / pairs, pr = ww % pairs;
        const uint32_t d0 = pr < half ? pr : p.n_rot + 2 * (pr - half), d1 = pr < half ? pr + half : d0 + 1;
        const uint64_t sb = is_q ? (uint64_t)col * p.q_col_stride + (uint64_t)head * p.q_head_stride : (uint64_t)col * p.kv_col_stride + (uint64_t)head * hd;
        a[u] = ld_act(is_q ? p.q : p.k, sb + d0, p.in_f16); b[u] = ld_act(is_q ? p.q : p.k, sb + d1, p.in_f16);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t w = w0 + u * blockDim.x;
      if (w >= total) continue;
      if (w >= nq + nk) {
        __half* dst = p.v_cache + (p.cache_row0 + col) * (uint64_t)kvd + 2 * (w - nq - nk);
        dst[0] = f16_rne(a[u]); dst[1] = f16_rne(b[u]);
        continue;
      }
      const bool is_q = w < nq;
      const uint32_t ww = is_q ? w : w - nq, head = ww / pairs, pr = ww % pairs;
      const uint32_t d0 = pr < half ? pr : p.n_rot + 2 * (pr - half), d1 = pr < half ? pr + half : d0 + 1;
      float ra = a[u], rb = b[u];
      if (p.mode != PA_ROPE_NONE && pr < half) {
        if (p.mode == PA_ROPE_F64) {
          const Angle g = s_g[pr];
          ra = rot_exact(a[u], b[u], g, true);
          rb = rot_exact(b[u], a[u], g, false);
        } else {
          const float c = p.cs_table[(uint64_t)col * p.n_rot + 2 * pr], sn = p.cs_table[(uint64_t)col * p.n_rot + 2 * pr + 1];
          ra = __fsub_rn(__fmul_rn(a[u], c), __fmul_rn(b[u], sn));
          rb = __fadd_rn(__fmul_rn(a[u], sn), __fmul_rn(b[u], c));
        }
      }
      if (is_q) {
        const uint64_t o = (uint64_t)col * p.q_out_col_stride + (uint64_t)head * hd;
        if (p.q_out_f16 == 2) {   // high and low f16 parts for the verify kernel's hi / lo rows
      __half* dst = reinterpret_cast<__half*>(p.q_out) + o;
      const __half ha = __float2half_rn(ra), hb = __float2half_rn(rb);
      dst[d0] = ha; dst[d1] = hb;
      dst[p.q_lo_offset + d0] = __float2half_rn(ra - __half2float(ha)); dst[p.q_lo_offset + d1] = __float2half_rn(rb - __half2float(hb));
    } else if (p.q_out_f16) { __half* dst = reinterpret_cast<__half*>(p.q_out) + o; dst[d0] = __float2half_rn(ra); dst[d1] = __float2half_rn(rb); }
        else { float* dst = reinterpret_cast<float*>(p.q_out) + o; dst[d0] = ra; dst[d1] = rb; }
      } else {
        __half* dst = p.k_cache + (p.cache_row0 + col) * (uint64_t)kvd + (uint64_t)head * hd;
        dst[d0] = f16_rne(ra); dst[d1] = f16_rne(rb);
      }
    }
  }
}


// Prefill chunks of f16 activations with the rotated q stored as f16 (what the prefill kernel consumes): the same
// arithmetic as the kernels above.  One CTA per column, two passes: the rotated dims two at a time (every lane of
// a warp does the same four rotations: mixed with copies, the few rotating lanes would hold their warps up), then
// 16-byte vectors of everything that is only copied (NaNs take the pattern the scalar path produces).
__device__ __forceinline__ uint32_t fix_nan2(uint32_t w, bool cache) {
  // per half: NaN -> 0x7fff (q, cvt.rn.f16.f32 of a NaN) or sign | 0x7e00 (cache, f16_rne)
  uint32_t out = w;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const uint32_t h = (w >> (16 * e)) & 0xffffu;
    if ((h & 0x7c00u) == 0x7c00u && (h & 0x03ffu)) {
      const uint32_t r = cache ? ((h & 0x8000u) | 0x7e00u) : 0x7fffu;
      out = (out & ~(0xffffu << (16 * e))) | (r << (16 * e));
    }
  }
  return out;
}
__global__ void __launch_bounds__(256) pa_rope_append_vec_kernel(const RopeParams p) {
  __shared__ Angle s_g[128];
  const uint32_t col = blockIdx.x, half = p.n_rot / 2, hd = p.hd;
  if (p.trigger_early) pdl_trigger();
  pdl_wait();
  if (!p.trigger_early) pdl_trigger();
  // the column's angles are requested now and go to shared memory after the first items' loads have been requested
  // too: one memory round trip for both (half <= 128 <= blockDim.x)
  Angle my_g;
  const bool has_g = threadIdx.x < half;
  if (has_g) my_g = p.n_ang ? p.ang[col * half + threadIdx.x] : p.angles[(uint64_t)col * half + threadIdx.x];
  bool g_staged = false;
  const uint32_t kvd = p.kv_heads * hd;
  const __half* qs = reinterpret_cast<const __half*>(p.q) + (uint64_t)col * p.q_col_stride;
  const __half* ks = reinterpret_cast<const __half*>(p.k) + (uint64_t)col * p.kv_col_stride;
  const __half* vs = reinterpret_cast<const __half*>(p.v) + (uint64_t)col * p.v_col_stride;
  __half* qd = reinterpret_cast<__half*>(p.q_out) + (uint64_t)col * p.q_out_col_stride;
  __half* kd = p.k_cache + (p.cache_row0 + col) * (uint64_t)kvd;
  __half* vd = p.v_cache + (p.cache_row0 + col) * (uint64_t)kvd;
  const uint32_t nqh = p.q ? p.q_heads : 0, nkh = p.k ? p.kv_heads : 0;

  // ---- rotated dims: an item is two adjacent dims (d, d + 1) with their partners (d + half, d + half + 1) of one
  //      head, so every lane of a warp carries the same four rotations ----
  {
    const uint32_t per = half / 2, total = (nqh + nkh) * per;
    for (uint32_t base = 0; base < total; base += 2 * blockDim.x) {   // (the same trips for every thread: a barrier sits inside)
      const uint32_t w0 = base + threadIdx.x;
      uint32_t A[2], B[2]; const __half* src[2]; __half* dst[2]; uint32_t dd[2]; int kind[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t w = w0 + u * blockDim.x;
        kind[u] = -1;
        if (w >= total) continue;
        const uint32_t head = w / per, d = 2 * (w % per);
        const bool is_q = head < nqh;
        kind[u] = is_q ? 0 : 1; dd[u] = d;
        src[u] = (is_q ? qs + (uint64_t)head * p.q_head_stride : ks + (uint64_t)(head - nqh) * hd) + d;
        dst[u] = (is_q ? qd + (uint64_t)head * hd : kd + (uint64_t)(head - nqh) * hd) + d;
        A[u] = *reinterpret_cast<const uint32_t*>(src[u]);
        B[u] = *reinterpret_cast<const uint32_t*>(src[u] + half);
      }
      if (!g_staged) {
        if (has_g) s_g[threadIdx.x] = my_g;
        __syncthreads();
        g_staged = true;
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (kind[u] < 0) continue;
        const bool cache = kind[u] != 0;
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&A[u])), b = __half22float2(*reinterpret_cast<const __half2*>(&B[u]));
        const Angle g0 = s_g[dd[u]], g1 = s_g[dd[u] + 1];
        const float ra0 = rot_exact(a.x, b.x, g0, true), ra1 = rot_exact(a.y, b.y, g1, true);
        const float rb0 = rot_exact(b.x, a.x, g0, false), rb1 = rot_exact(b.y, a.y, g1, false);
        auto h = [&](float x) -> uint32_t { return cache ? __half_as_ushort(f16_rne(x)) : __half_as_ushort(__float2half_rn(x)); };
        *reinterpret_cast<uint32_t*>(dst[u]) = h(ra0) | (h(ra1) << 16);
        *reinterpret_cast<uint32_t*>(dst[u] + half) = h(rb0) | (h(rb1) << 16);
      }
    }
  }
  // ---- everything else: 16-byte vectors of the unrotated dims of q and k, and all of v ----
  {
    const uint32_t cv = (hd - p.n_rot) / 8, vv = hd / 8;
    const uint32_t nq = p.q_rot_only ? 0u : nqh * cv, nk = nkh * cv, nv = p.v ? p.kv_heads * vv : 0, total = nq + nk + nv;
    for (uint32_t w0 = threadIdx.x; w0 < total; w0 += 4 * blockDim.x) {
      uint4 A[4]; __half* dst[4]; int kind[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t w = w0 + u * blockDim.x;
        kind[u] = -1;
        if (w >= total) continue;
        const __half* src;
        if (w >= nq + nk) {
          const uint32_t x = w - nq - nk;
          kind[u] = 1; src = vs + 8 * x; dst[u] = vd + 8 * x;
        } else {
          const bool is_q = w < nq;
          const uint32_t ww = is_q ? w : w - nq, head = ww / cv, d = p.n_rot + 8 * (ww % cv);
          kind[u] = is_q ? 0 : 1;
          src = (is_q ? qs + (uint64_t)head * p.q_head_stride : ks + (uint64_t)head * hd) + d;
          dst[u] = (is_q ? qd + (uint64_t)head * hd : kd + (uint64_t)head * hd) + d;
        }
        A[u] = *reinterpret_cast<const uint4*>(src);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (kind[u] < 0) continue;
        const bool cache = kind[u] != 0;
        uint4 o = A[u];
        o.x = fix_nan2(o.x, cache); o.y = fix_nan2(o.y, cache); o.z = fix_nan2(o.z, cache); o.w = fix_nan2(o.w, cache);
        *reinterpret_cast<uint4*>(dst[u]) = o;
      }
    }
  }
}

// cos / sin of every (column, rotary pair) of a call, evaluated once in float64 and shared by all layers of the step
// (the host keeps the table while position and width stay the same)
__global__ void __launch_bounds__(128) pa_angles_kernel(const AnglesParams p) {
  pdl_wait();        // an earlier kernel may still be reading the table
  pdl_trigger();
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.n_cols * p.half) return;
  double s, c;
  sincos(__dmul_rn((double)(p.pos0 + i / p.half), p.inv_freq[i % p.half]), &s, &c);
  p.out[i] = make_angle(c, s);
}

// QK head-norm (the step before RoPE in attn_glue, engine/wgsl/qwen35.js:1112-1122), with the arithmetic of the CPU
// reference (tests/reference/ref_q38.mjs:50-57): the sum of squares is accumulated in float64 in index order by one
// thread -- that order is part of the result -- then out = f32((x * inv) * w) with inv = 1 / sqrt(ss / hd + eps).
// grid (columns, heads), 64 threads.
__global__ void __launch_bounds__(64) pa_head_norm_kernel(const HeadNormParams p) {
  __shared__ float s_x[512];
  __shared__ double s_inv;
  const uint32_t col = blockIdx.x, hd = p.hd;
  const bool second = blockIdx.y >= p.n_first;
  const uint32_t head = second ? blockIdx.y - p.n_first : blockIdx.y;
  const void* x = second ? p.x2 : p.x;
  void* y = second ? p.y2 : p.y;
  const float* w = second ? p.w2 : p.w;
  pdl_wait();
  pdl_trigger();
  const uint64_t xo = (uint64_t)col * (second ? p.x2_col_stride : p.x_col_stride) + (uint64_t)head * (second ? p.x2_head_stride : p.x_head_stride);
  for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) s_x[i] = ld_act(x, xo + i, p.f16);
  __syncthreads();
  if (threadIdx.x == 0) {
    double ss = 0.0;
    for (uint32_t i = 0; i < hd; ++i) { const double v = (double)s_x[i]; ss = __dadd_rn(ss, __dmul_rn(v, v)); }
    s_inv = __ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(__ddiv_rn(ss, (double)hd), p.eps)));
  }
  __syncthreads();
  const double inv = s_inv;
  const uint64_t yo = (uint64_t)col * (second ? p.y2_col_stride : p.y_col_stride) + (uint64_t)head * (second ? p.y2_head_stride : p.y_head_stride);
  for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) {
    const float r = (float)__dmul_rn(__dmul_rn((double)s_x[i], inv), (double)w[i]);
    if (p.f16) reinterpret_cast<__half*>(y)[yo + i] = __float2half_rn(r);
    else reinterpret_cast<float*>(y)[yo + i] = r;
  }
}

__global__ void __launch_bounds__(256) pa_sigmoid_mul_kernel(const SigmoidParams p) {
  const uint32_t col = blockIdx.x, n = p.n_heads * p.hd;
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
    const uint32_t h = i / p.hd, d = i % p.hd;
    const uint64_t ao = (uint64_t)col * p.a_col_stride + i, go = (uint64_t)col * p.g_col_stride + (uint64_t)h * p.g_head_stride + d;
    const float gv = ld_act(p.g, go, p.f16);
    const float sg = 1.0f / (1.0f + expf(-gv));
    if (p.f16) reinterpret_cast<__half*>(p.a)[ao] = __float2half_rn(__half2float(reinterpret_cast<__half*>(p.a)[ao]) * sg);
    else reinterpret_cast<float*>(p.a)[ao] = reinterpret_cast<float*>(p.a)[ao] * sg;
  }
}

// whether a call goes to the vectorised kernel (the only one that knows q_rot_only)
bool rope_vec_applies(const RopeParams& p, uint32_t n_cols) {
  auto al16 = [](const void* x) { return ((uintptr_t)x & 15) == 0; };
  return !p.n_items && n_cols >= 16 && p.mode == PA_ROPE_F64 && (p.angles || p.n_ang) && p.in_f16 && p.n_rot % 16 == 0 && p.n_rot <= 256 && p.hd % 8 == 0 &&
         (!p.q || (p.q_out_f16 == 1 && al16(p.q) && al16(p.q_out) && p.q_col_stride % 8 == 0 && p.q_head_stride % 8 == 0 && p.q_out_col_stride % 8 == 0)) &&
         (!p.k || (p.v && al16(p.k) && al16(p.v) && p.kv_col_stride % 8 == 0 && p.v_col_stride % 8 == 0));
}

cudaError_t launch_rope_append(const RopeParams& p, uint32_t n_cols, cudaStream_t st) {
  if (rope_vec_applies(p, n_cols)) return launch_pdl(pa_rope_append_vec_kernel, dim3(n_cols), dim3(256), 0, st, p);
  if (n_cols >= 16 && !p.n_items) return launch_pdl(pa_rope_append_cols_kernel, dim3(n_cols), dim3(256), 0, st, p);
  const uint32_t slots = (p.q ? p.q_heads : 0) + (p.k ? p.kv_heads : 0) + (p.v ? p.kv_heads : 0);
  return launch_pdl(pa_rope_append_kernel, dim3(n_cols, slots), dim3(128), 0, st, p);
}
cudaError_t launch_angles(const AnglesParams& p, cudaStream_t st) {
  return launch_pdl(pa_angles_kernel, dim3((p.n_cols * p.half + 127) / 128), dim3(128), 0, st, p);
}
cudaError_t launch_head_norm(const HeadNormParams& p, uint32_t n_cols, uint32_t n_heads, cudaStream_t st) {
  return launch_pdl(pa_head_norm_kernel, dim3(n_cols, n_heads), dim3(64), 0, st, p);
}
cudaError_t launch_sigmoid_mul(const SigmoidParams& p, uint32_t n_cols, cudaStream_t st) {
  pa_sigmoid_mul_kernel<<<n_cols, 256, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace pa
