// RoPE (full or partial, NeoX pairing), the f16 KV-cache append and the standalone sigmoid gate.
//
// One small CTA per (column, head).  The cos / sin of an angle is evaluated by the thread that rotates the pair:
//   PA_ROPE_F64    angle = pos * inv_freq[i] in float64 (inv_freq = theta^(-2i/n_rot) comes from the host's
//                  libm), cos / sin in float64, the two products and their difference / sum rounded one by
//                  one in float64, the result rounded to f32 — the arithmetic of pooled's CPU reference
//                  (tests/reference/ref_q38.mjs:67-79).
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
#ifdef PA_TRACE
#define RTR(slot) do { if (p.trace && threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_)); p.trace[(224 + (blockIdx.y & 31)) * 256 + (slot)] = t_; } } while (0)
#else
#define RTR(slot) do {} while (0)
#endif
  RTR(0);
  if (p.trigger_early) pdl_trigger();
  pdl_wait();
  if (!p.trigger_early) pdl_trigger();
  RTR(1);
  if (pr >= hd / 2) return;
  const uint32_t nq = p.q ? p.q_heads : 0, nk = p.k ? p.kv_heads : 0;
  uint32_t slot = blockIdx.y;
  if (slot >= nq + nk) {
    // V head: conversion only
    const uint32_t head = slot - nq - nk, kvd = p.kv_heads * hd;
    const uint64_t so = (uint64_t)col * p.kv_col_stride + (uint64_t)head * hd + 2 * pr;
    __half* dst = p.v_cache + (p.cache_row0 + col) * (uint64_t)kvd + (uint64_t)head * hd + 2 * pr;
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
      const double ang = __dmul_rn((double)(p.pos + col), p.inv_freq[pr]);
      double s, c;
      sincos(ang, &s, &c);
      const double ad = (double)a, bd = (double)b;
      ra = (float)__dsub_rn(__dmul_rn(ad, c), __dmul_rn(bd, s));
      rb = (float)__dadd_rn(__dmul_rn(bd, c), __dmul_rn(ad, s));
    } else {
      const float c = p.cs_table[(uint64_t)col * p.n_rot + 2 * pr], s = p.cs_table[(uint64_t)col * p.n_rot + 2 * pr + 1];
      ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
      rb = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
    }
  }
  if (is_q) {
    const uint64_t o = (uint64_t)col * p.q_out_col_stride + (uint64_t)head * hd;
    if (p.q_out_f16) { __half* dst = reinterpret_cast<__half*>(p.q_out) + o; dst[d0] = __float2half_rn(ra); dst[d1] = __float2half_rn(rb); }
    else { float* dst = reinterpret_cast<float*>(p.q_out) + o; dst[d0] = ra; dst[d1] = rb; }
  } else {
    __half* dst = p.k_cache + (p.cache_row0 + col) * (uint64_t)(p.kv_heads * hd) + (uint64_t)head * hd;
    dst[d0] = f16_rne(ra); dst[d1] = f16_rne(rb);
  }
  RTR(2);
}

// Many columns (prefill chunks): one 256-thread CTA per column.  The column's n_rot/2 angles are evaluated once and
// shared by every head through shared memory; each thread then takes (head, pair) items four at a time so that its
// loads overlap.  Same arithmetic, element for element, as the per-head kernel above.
__global__ void __launch_bounds__(256) pa_rope_append_cols_kernel(const RopeParams p) {
  __shared__ double s_c[128], s_s[128];
  const uint32_t col = blockIdx.x, half = p.n_rot / 2, hd = p.hd, pairs = hd / 2;
  if (p.trigger_early) pdl_trigger();
  pdl_wait();
  if (!p.trigger_early) pdl_trigger();
  if (p.mode == PA_ROPE_F64) {
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
      double sv, cv;
      sincos(__dmul_rn((double)(p.pos + col), p.inv_freq[i]), &sv, &cv);
      s_c[i] = cv; s_s[i] = sv;
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
        const uint64_t so = (uint64_t)col * p.kv_col_stride + 2 * (w - nq - nk);
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
          const double c = s_c[pr], sn = s_s[pr], ad = (double)a[u], bd = (double)b[u];
          ra = (float)__dsub_rn(__dmul_rn(ad, c), __dmul_rn(bd, sn));
          rb = (float)__dadd_rn(__dmul_rn(bd, c), __dmul_rn(ad, sn));
        } else {
          const float c = p.cs_table[(uint64_t)col * p.n_rot + 2 * pr], sn = p.cs_table[(uint64_t)col * p.n_rot + 2 * pr + 1];
          ra = __fsub_rn(__fmul_rn(a[u], c), __fmul_rn(b[u], sn));
          rb = __fadd_rn(__fmul_rn(a[u], sn), __fmul_rn(b[u], c));
        }
      }
      if (is_q) {
        const uint64_t o = (uint64_t)col * p.q_out_col_stride + (uint64_t)head * hd;
        if (p.q_out_f16) { __half* dst = reinterpret_cast<__half*>(p.q_out) + o; dst[d0] = __float2half_rn(ra); dst[d1] = __float2half_rn(rb); }
        else { float* dst = reinterpret_cast<float*>(p.q_out) + o; dst[d0] = ra; dst[d1] = rb; }
      } else {
        __half* dst = p.k_cache + (p.cache_row0 + col) * (uint64_t)kvd + (uint64_t)head * hd;
        dst[d0] = f16_rne(ra); dst[d1] = f16_rne(rb);
      }
    }
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

cudaError_t launch_rope_append(const RopeParams& p, uint32_t n_cols, cudaStream_t st) {
  if (n_cols >= 16) return launch_pdl(pa_rope_append_cols_kernel, dim3(n_cols), dim3(256), 0, st, p);
  const uint32_t slots = (p.q ? p.q_heads : 0) + (p.k ? p.kv_heads : 0) + (p.v ? p.kv_heads : 0);
  return launch_pdl(pa_rope_append_kernel, dim3(n_cols, slots), dim3(128), 0, st, p);
}
cudaError_t launch_sigmoid_mul(const SigmoidParams& p, uint32_t n_cols, cudaStream_t st) {
  pa_sigmoid_mul_kernel<<<n_cols, 256, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace pa
