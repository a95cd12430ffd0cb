// RoPE (full or partial, NeoX pairing), the f16 KV-cache append and the standalone sigmoid gate.
//
// One CTA per column (token).  The cos / sin of the column's n_rot/2 angles are evaluated once per CTA
// and shared by every head:
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

__global__ void __launch_bounds__(256) pa_rope_append_kernel(const RopeParams p) {
  __shared__ double s_c[128], s_s[128];
  __shared__ float s_cf[128], s_sf[128];
  const uint32_t col = blockIdx.x, half = p.n_rot / 2;
  // The kernel after this one may start fetching old cache rows while this one runs (it never touches the rows or
  // the rotated q written here before its own wait); this kernel itself writes nothing before its predecessor ends.
  pdl_trigger();
  pdl_wait();
  if (p.mode == PA_ROPE_F64) {
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
      const double ang = __dmul_rn((double)(p.pos + col), p.inv_freq[i]);
      double sv, cv;
      sincos(ang, &sv, &cv);
      s_c[i] = cv; s_s[i] = sv;
    }
  } else if (p.mode == PA_ROPE_TABLE) {
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
      s_cf[i] = p.cs_table[(uint64_t)col * p.n_rot + 2 * i];
      s_sf[i] = p.cs_table[(uint64_t)col * p.n_rot + 2 * i + 1];
    }
  }
  __syncthreads();

  const uint32_t hd = p.hd, pairs = hd / 2;
  // work items: (head, pair) over q heads then k heads; pair < half rotates dims (pair, pair + half), the rest
  // pass dims n_rot + 2*(pair-half), +1 through
  const uint32_t nq = p.q ? p.q_heads * pairs : 0, nk = p.k ? p.kv_heads * pairs : 0;
  for (uint32_t w = threadIdx.x; w < nq + nk; w += blockDim.x) {
    const bool is_q = w < nq;
    const uint32_t ww = is_q ? w : w - nq;
    const uint32_t head = ww / pairs, pr = ww % pairs;
    uint32_t d0, d1;
    const bool rot = p.mode != PA_ROPE_NONE && pr < half;
    if (pr < half) { d0 = pr; d1 = pr + half; } else { d0 = p.n_rot + 2 * (pr - half); d1 = d0 + 1; }
    const void* src = is_q ? p.q : p.k;
    const uint64_t sb = is_q ? (uint64_t)col * p.q_col_stride + (uint64_t)head * p.q_head_stride
                             : (uint64_t)col * p.kv_col_stride + (uint64_t)head * hd;
    float a = ld_act(src, sb + d0, p.in_f16), b = ld_act(src, sb + d1, p.in_f16);
    float ra = a, rb = b;
    if (rot) {
      if (p.mode == PA_ROPE_F64) {
        const double c = s_c[pr], s = s_s[pr], ad = (double)a, bd = (double)b;
        ra = (float)__dsub_rn(__dmul_rn(ad, c), __dmul_rn(bd, s));
        rb = (float)__dadd_rn(__dmul_rn(bd, c), __dmul_rn(ad, s));
      } else {
        const float c = s_cf[pr], s = s_sf[pr];
        ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        rb = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
      }
    }
    if (is_q) {
      float* dst = p.q_out + (uint64_t)col * p.q_out_col_stride + (uint64_t)head * hd;
      dst[d0] = ra; dst[d1] = rb;
    } else {
      __half* dst = p.k_cache + (p.cache_row0 + col) * (uint64_t)(p.kv_heads * hd) + (uint64_t)head * hd;
      dst[d0] = f16_rne(ra); dst[d1] = f16_rne(rb);
    }
  }
  if (p.v) {
    const uint32_t kvd = p.kv_heads * hd;
    __half* dst = p.v_cache + (p.cache_row0 + col) * (uint64_t)kvd;
    for (uint32_t i = threadIdx.x; i < kvd; i += blockDim.x)
      dst[i] = f16_rne(ld_act(p.v, (uint64_t)col * p.kv_col_stride + i, p.in_f16));
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
  return launch_pdl(pa_rope_append_kernel, dim3(n_cols), dim3(256), 0, st, p);
}
cudaError_t launch_sigmoid_mul(const SigmoidParams& p, uint32_t n_cols, cudaStream_t st) {
  pa_sigmoid_mul_kernel<<<n_cols, 256, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace pa
