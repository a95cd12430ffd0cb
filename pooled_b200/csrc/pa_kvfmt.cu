// KV caches in the other two formats pooled's engines keep: int8 with one f32 scale per 32 values (kvQ8: kv_store_q8 +
// attn_flash_q8, engine/wgsl/qwen35.js:97-139, :908-946) and f32 (the dense engine, engine/wgsl/dense.js:22-136).
//
// The f16 cache has the TMA / tensor-core kernels of pa_decode.cu and pa_prefill.cu.  These two formats share one
// split-K kernel of the same outer shape (one CTA per (split, kv head, column), an unnormalised (o, m, l) record per
// (row, split) for pa_combine_kernel) built from plain vector loads: per chunk of 64 positions
//   scores   four threads per K row, a quarter of the head each, the G heads of the group per thread; q in shared memory
//   softmax  32 threads per head, online rescale across chunks (m starts at -3.0e38, as in the reference)
//   values   a thread per four dims and group of positions, the groups summed in a fixed order at the end
// A row of kv_dim values costs kv_dim * 1.125 bytes (int8) or kv_dim * 4 bytes (f32) against kv_dim * 2 for f16.
// int8 values are dequantised as f32(int8) * scale, the order of the reference (attn_flash_q8's dot and vread).
#include "pa_params.cuh"

namespace pa {

// ---- append -------------------------------------------------------------------------------------------------

// kv_store_q8 (engine/wgsl/qwen35.js:908-946), operation for operation: per block of 32 values scale = max|x| / 127,
// inv = 1 / scale (0 when the block is all zeros), value = clamp(round_to_nearest_even(x * inv), -127, 127).
// grid (kv_dim / 32 blocks, columns), one thread per (block, K or V).
__global__ void __launch_bounds__(64) pa_kv_store_q8_kernel(const KvStoreParams p) {
  pdl_wait();
  pdl_trigger();
  const uint32_t nb = p.kv_dim / 32, blk = blockIdx.x * 32 + (threadIdx.x & 31), col = blockIdx.y, which = threadIdx.x >> 5;
  if (blk >= nb) return;
  const void* src = which ? p.v : p.k;
  const uint64_t so = (uint64_t)col * (which ? p.v_col_stride : p.k_col_stride) + (uint64_t)blk * 32;
  float x[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) x[i] = (which ? p.v_f16 : p.k_f16) ? __half2float(reinterpret_cast<const __half*>(src)[so + i]) : reinterpret_cast<const float*>(src)[so + i];
  float a = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) a = fmaxf(a, fabsf(x[i]));
  const float sc = __fdiv_rn(a, 127.0f), inv = sc > 0.f ? __fdiv_rn(1.0f, sc) : 0.f;
  const uint64_t row = p.cache_row0 + col;
  (which ? p.vs : p.ks)[row * nb + blk] = sc;
  uint32_t* dst = reinterpret_cast<uint32_t*>((which ? p.v8 : p.k8) + row * p.kv_dim + (uint64_t)blk * 32);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t w = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int q = (int)fminf(fmaxf(rintf(__fmul_rn(x[4 * j + b], inv)), -127.0f), 127.0f);
      w |= ((uint32_t)q & 255u) << (8 * b);
    }
    dst[j] = w;
  }
}

// f32 cache rows: a copy (f16 activations widen exactly)
__global__ void __launch_bounds__(256) pa_kv_store_f32_kernel(const KvStoreParams p) {
  pdl_wait();
  pdl_trigger();
  const uint32_t col = blockIdx.y;
  const uint64_t row = p.cache_row0 + col;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < p.kv_dim; i += gridDim.x * blockDim.x) {
    const uint64_t ko = (uint64_t)col * p.k_col_stride + i, vo = (uint64_t)col * p.v_col_stride + i;
    p.k32[row * p.kv_dim + i] = p.k_f16 ? __half2float(reinterpret_cast<const __half*>(p.k)[ko]) : reinterpret_cast<const float*>(p.k)[ko];
    p.v32[row * p.kv_dim + i] = p.v_f16 ? __half2float(reinterpret_cast<const __half*>(p.v)[vo]) : reinterpret_cast<const float*>(p.v)[vo];
  }
}

cudaError_t launch_kv_store(const KvStoreParams& p, uint32_t n_cols, cudaStream_t st) {
  if (p.format == PA_KV_Q8) return launch_pdl(pa_kv_store_q8_kernel, dim3((p.kv_dim / 32 + 31) / 32, n_cols), dim3(64), 0, st, p);
  return launch_pdl(pa_kv_store_f32_kernel, dim3((p.kv_dim + 255) / 256, n_cols), dim3(256), 0, st, p);
}

// ---- split-K decode / verify / prefill over an int8 or f32 cache -----------------------------------------------

constexpr int kAnyChunk = 64;     // positions per chunk
constexpr int kAnyThreads = 256;
constexpr int kAnyMaxG = 16;      // query heads per kv head

template <int FMT> struct KvRead;
template <> struct KvRead<PA_KV_Q8> {
  // n consecutive values (n % 16 == 0) of a row starting at element e0 (e0 % 16 == 0)
  template <typename F> static __device__ __forceinline__ void span(const void* cache, const float* scales, uint64_t row, uint32_t kv_dim, uint32_t e0, uint32_t n, F&& f) {
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const int8_t*>(cache) + row * kv_dim + e0);
    const float* sc = scales + row * (kv_dim / 32);
    for (uint32_t c = 0; c < n / 16; ++c) {
      const uint4 w4 = src[c];
      const float s = sc[(e0 + 16 * c) / 32];
      const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int b = 0; b < 4; ++b) f(16 * c + 4 * j + b, __fmul_rn((float)(int8_t)(w[j] >> (8 * b)), s));
    }
  }
  static __device__ __forceinline__ float4 quad(const void* cache, const float* scales, uint64_t row, uint32_t kv_dim, uint32_t e0) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const int8_t*>(cache) + row * kv_dim + e0);
    const float s = scales[row * (kv_dim / 32) + e0 / 32];
    return make_float4(__fmul_rn((float)(int8_t)w, s), __fmul_rn((float)(int8_t)(w >> 8), s), __fmul_rn((float)(int8_t)(w >> 16), s), __fmul_rn((float)(int8_t)(w >> 24), s));
  }
};
template <> struct KvRead<PA_KV_F32> {
  template <typename F> static __device__ __forceinline__ void span(const void* cache, const float*, uint64_t row, uint32_t kv_dim, uint32_t e0, uint32_t n, F&& f) {
    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(cache) + row * kv_dim + e0);
    for (uint32_t c = 0; c < n / 4; ++c) {
      const float4 x = src[c];
      f(4 * c, x.x); f(4 * c + 1, x.y); f(4 * c + 2, x.z); f(4 * c + 3, x.w);
    }
  }
  static __device__ __forceinline__ float4 quad(const void* cache, const float*, uint64_t row, uint32_t kv_dim, uint32_t e0) {
    return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(cache) + row * kv_dim + e0);
  }
};

// grid (splits, kv heads, columns of one item).  Dynamic shared memory: q [G][hd] f32, then the chunk's scores /
// weights [G][64], then m, l, alpha [G] each, then the values phase's partial sums.
template <int FMT>
__global__ void __launch_bounds__(kAnyThreads) pa_decode_any_kernel(const AnyDecodeParams p) {
  extern __shared__ float sm[];
  const uint32_t hd = p.hd, G = p.G, split = blockIdx.x, g = blockIdx.y, c = blockIdx.z;
  float* q_s = sm;                               // [G][hd]
  float* s_s = q_s + G * hd;                     // [G][64]
  float* s_m = s_s + G * kAnyChunk;              // [G]
  float* s_l = s_m + G;
  float* s_a = s_l + G;
  float* s_red = sm + ((G * hd + G * kAnyChunk + 3 * G + 3) & ~3u);   // [position groups][G][hd] at the end (16-byte aligned)
  const int tid = threadIdx.x, lane = tid & 31;
  // rows this column sees, and this split's range of them (the plan is the item's: its last column's rows)
  const uint32_t lim = (uint32_t)min(max(p.lim0 + (int32_t)c, 0), (int32_t)p.n_rows);
  const uint32_t tiles = (p.n_rows + kAnyChunk - 1) / kAnyChunk;
  const uint32_t ns_eff = min(p.n_splits, max(1u, tiles / 2));
  const uint32_t tps = (tiles + ns_eff - 1) / max(ns_eff, 1u);
  const uint32_t t0 = split * tps * kAnyChunk, t1 = min(min(tiles, (split + 1) * tps) * kAnyChunk, lim);
  if (split * tps >= tiles) return;              // no record expected from this split
  pdl_wait();
  pdl_trigger();
  const uint64_t col = p.col0 + c;
  for (uint32_t i = tid; i < G * hd; i += kAnyThreads) {
    const uint64_t off = col * p.q_col_stride + (uint64_t)(g * G + i / hd) * p.q_head_stride + i % hd;
    q_s[i] = p.q_f16 ? __half2float(reinterpret_cast<const __half*>(p.q)[off]) : reinterpret_cast<const float*>(p.q)[off];
  }
  if ((uint32_t)tid < G) { s_m[tid] = -3.0e38f; s_l[tid] = 0.f; }
  // values phase: thread = (group of positions pg, four dims dq)
  const uint32_t quads = hd / 4, n_pg = kAnyThreads / quads, dq = tid % quads, pg = tid / quads;
  float acc[kAnyMaxG][4];
#pragma unroll
  for (int h = 0; h < kAnyMaxG; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
  const float rs = sqrtf((float)hd);
  const uint64_t row0 = (uint64_t)p.seq * p.max_seq;
  __syncthreads();
  for (uint32_t c0 = t0; c0 < t1; c0 += kAnyChunk) {
    const uint32_t n = min((uint32_t)kAnyChunk, t1 - c0);
    // ---- scores: thread (r, part) takes a quarter of row r for all G heads; the four parts are summed in lane order ----
    {
      const uint32_t r = tid >> 2, part = tid & 3, span = hd / 4;
      float s[kAnyMaxG];
#pragma unroll
      for (int h = 0; h < kAnyMaxG; ++h) s[h] = 0.f;
      if (r < n) {
        KvRead<FMT>::span(p.k, p.ks, row0 + c0 + r, p.kv_dim, g * hd + part * span, span, [&](uint32_t i, float kv) {
#pragma unroll
          for (int h = 0; h < kAnyMaxG; ++h) if ((uint32_t)h < G) s[h] = __fmaf_rn(q_s[h * hd + part * span + i], kv, s[h]);
        });
      }
#pragma unroll
      for (int h = 0; h < kAnyMaxG; ++h) {
        if ((uint32_t)h >= G) break;
        float v = s[h];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if (part == 0) s_s[h * kAnyChunk + r] = r < n ? v / rs : -INFINITY;
      }
    }
    __syncthreads();
    // ---- online softmax: warp w takes heads w, w + 8 ----
    for (uint32_t h = tid >> 5; h < G; h += kAnyThreads / 32) {
      const float a = s_s[h * kAnyChunk + lane], b = s_s[h * kAnyChunk + 32 + lane];
      float mx = fmaxf(a, b);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = s_m[h], m_new = fmaxf(m_old, mx);
      const float ea = expf(a - m_new), eb = expf(b - m_new);      // exp(-inf) = 0 for rows past the chunk's end
      s_s[h * kAnyChunk + lane] = ea; s_s[h * kAnyChunk + 32 + lane] = eb;
      float sum = ea + eb;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) {
        const float alpha = expf(m_old - m_new);
        s_m[h] = m_new; s_l[h] = s_l[h] * alpha + sum; s_a[h] = alpha;
      }
    }
    __syncthreads();
    // ---- values ----
#pragma unroll
    for (int h = 0; h < kAnyMaxG; ++h) {
      if ((uint32_t)h >= G) break;
      const float a = s_a[h];
      acc[h][0] *= a; acc[h][1] *= a; acc[h][2] *= a; acc[h][3] *= a;
    }
    for (uint32_t t = pg; t < n; t += n_pg) {
      const float4 v = KvRead<FMT>::quad(p.v, p.vs, row0 + c0 + t, p.kv_dim, g * hd + dq * 4);
#pragma unroll
      for (int h = 0; h < kAnyMaxG; ++h) {
        if ((uint32_t)h >= G) break;
        const float w = s_s[h * kAnyChunk + t];
        acc[h][0] = __fmaf_rn(w, v.x, acc[h][0]); acc[h][1] = __fmaf_rn(w, v.y, acc[h][1]);
        acc[h][2] = __fmaf_rn(w, v.z, acc[h][2]); acc[h][3] = __fmaf_rn(w, v.w, acc[h][3]);
      }
    }
    __syncthreads();
  }
  // ---- the position groups' sums, added in group order; one record per (row, split) ----
#pragma unroll
  for (int h = 0; h < kAnyMaxG; ++h) {
    if ((uint32_t)h >= G) break;
    *reinterpret_cast<float4*>(s_red + ((size_t)pg * G + h) * hd + dq * 4) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
  }
  __syncthreads();
  for (uint32_t i = tid; i < G * hd; i += kAnyThreads) {
    const uint32_t h = i / hd, d = i % hd;
    float o = s_red[(size_t)h * hd + d];
    for (uint32_t k = 1; k < n_pg; ++k) o += s_red[((size_t)k * G + h) * hd + d];
    const uint64_t prow = col * p.n_heads + g * G + h;
    p.part_o[(prow * p.n_splits + split) * hd + d] = o;
  }
  if ((uint32_t)tid < G) {
    const uint64_t prow = col * p.n_heads + g * G + tid;
    p.part_ml[(prow * p.n_splits + split) * 2] = s_m[tid];
    p.part_ml[(prow * p.n_splits + split) * 2 + 1] = s_l[tid];
  }
}

size_t any_decode_smem(uint32_t G, uint32_t hd) {
  const size_t n_pg = kAnyThreads / (hd / 4);
  return ((((size_t)G * hd + (size_t)G * kAnyChunk + 3 * G + 3) & ~(size_t)3) + n_pg * G * hd) * sizeof(float);
}

cudaError_t launch_decode_any(const AnyDecodeParams& p, int format, dim3 grid, cudaStream_t st) {
  const size_t smem = any_decode_smem(p.G, p.hd);
  static bool attr_set[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kq = pa_decode_any_kernel<PA_KV_Q8>;
  auto kf = pa_decode_any_kernel<PA_KV_F32>;
  const int fi = format == PA_KV_Q8 ? 0 : 1;
  if (!attr_set[fi][dev & 63]) {
    cudaError_t e = fi == 0 ? cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                            : cudaFuncSetAttribute(kf, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_set[fi][dev & 63] = true;
  }
  return fi == 0 ? launch_pdl(kq, grid, dim3(kAnyThreads), smem, st, p) : launch_pdl(kf, grid, dim3(kAnyThreads), smem, st, p);
}

}  // namespace pa
