// C ABI of libpooled_attn.so: contexts, layer caches, tensor maps and the entry points declared in
// include/pooled_attn.h.  No exceptions cross the boundary; every failure is a status code plus a message.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <new>

#include "pa_common.cuh"

#include "pa_params.cuh"

namespace pa {
cudaError_t launch_decode(const pa_layer* L, const DecodeParams& p, dim3 grid, int nt, cudaStream_t st);
cudaError_t launch_combine(int head_dim, const CombineParams& p, uint32_t rows, cudaStream_t st);
cudaError_t launch_rope_append(const RopeParams& p, uint32_t n_cols, cudaStream_t st);
cudaError_t launch_sigmoid_mul(const SigmoidParams& p, uint32_t n_cols, cudaStream_t st);
cudaError_t launch_angles(const AnglesParams& p, cudaStream_t st);
bool rope_vec_applies(const RopeParams& p, uint32_t n_cols);
cudaError_t launch_epoch_bump(unsigned int* ctr, cudaStream_t st);
cudaError_t launch_head_norm(const HeadNormParams& p, uint32_t n_cols, uint32_t n_heads, cudaStream_t st);
int prefill_supported(const pa_ctx* ctx);
cudaError_t launch_prefill(const pa_layer* L, const PrefillParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_q,
                           const CUtensorMap& tm_o, const CUtensorMap& tm_q2, cudaStream_t st);
cudaError_t launch_verify(const pa_layer* L, const PrefillParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v, uint32_t n_kv, cudaStream_t st);
cudaError_t launch_kv_store(const KvStoreParams& p, uint32_t n_cols, cudaStream_t st);
cudaError_t launch_decode_any(const AnyDecodeParams& p, int format, dim3 grid, cudaStream_t st);
}  // namespace pa

using namespace pa;

static thread_local std::string g_err;  // for failures before a context exists

static int fail(pa_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf; else g_err = buf;
  return code;
}
#define CU_TRY(ctx, expr)                                                                         \
  do {                                                                                            \
    cudaError_t e_ = (expr);                                                                      \
    if (e_ != cudaSuccess) {                                                                      \
      (ctx)->failed = true;                                                                       \
      return fail((ctx), PA_ECUDA, "%s failed: %s", #expr, cudaGetErrorString(e_));               \
    }                                                                                             \
  } while (0)

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode() {
  static encode_tiled_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<encode_tiled_fn>(p);
  }
  return fn;
}

// View of an f16 cache [rows][kv_dim] as {64 elements, rows, kv_dim/64 chunks}; a box of {64, box_rows,
// head_dim/64} lands in shared memory as [chunk][row][128 bytes] with the 128-byte swizzle.
static int make_cache_map(pa_ctx* ctx, CUtensorMap* tm, void* base, uint64_t rows, uint32_t kv_dim, uint32_t hd, uint32_t box_rows) {
  encode_tiled_fn enc = get_encode();
  if (!enc) return fail(ctx, PA_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {64, rows, kv_dim / 64};
  cuuint64_t strides[2] = {(cuuint64_t)kv_dim * 2, 128};
  cuuint32_t box[3] = {64, box_rows, hd / 64};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ctx, PA_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return PA_OK;
}

static uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

// ------------------------------------------------------------------------------ host mirrors --

extern "C" uint32_t pa_dec_config(uint32_t head_dim, uint32_t G, uint32_t n_kv, uint32_t splits) {
  if (head_dim != 256 || G < 1 || G > 8 || n_kv < 1) return 0;
  if (splits > 0) return splits;
  uint32_t s = 256 / n_kv;
  return s > 16 ? s : 16;
}
extern "C" uint32_t pa_dec_split_len(uint32_t s, uint32_t S) {
  uint32_t l = ceil_div(ceil_div(s, S), 64) * 64;
  return l > 64 ? l : 64;
}
extern "C" uint32_t pa_dec_splits(uint32_t s, uint32_t S) { return ceil_div(s, pa_dec_split_len(s, S)); }
extern "C" uint32_t pa_tile_split_len(uint32_t seq_end, uint32_t fa_split, uint32_t fa_splits, uint32_t target) {
  auto up64 = [](uint32_t x) { return ceil_div(x, 64) * 64; };
  if (target < 1) target = 1;
  uint32_t m = 64;
  uint32_t a = up64(ceil_div(seq_end, target)), b = up64(ceil_div(seq_end, fa_splits));
  if (a > m) m = a;
  if (b > m) m = b;
  return m < fa_split ? m : fa_split;
}

// Splits per (item, kv head): enough CTAs to give every SM one, never more than one wave, at least two
// 64-row tiles each.  Depends on the call's longest column and item count only.
static uint32_t plan_splits(const pa_ctx* ctx, uint32_t n_rows, uint32_t n_items, uint32_t total_cols = 0, uint32_t groups = 1) {
  const uint32_t tiles = ceil_div(n_rows, 64);
  if (!total_cols) total_cols = n_items;
  uint32_t want = ctx->cfg.splits ? ctx->cfg.splits : (uint32_t)ctx->sm_count / (ctx->cfg.n_kv_heads * n_items);
  if (want < 1) want = 1;
  uint32_t cap = tiles / 2;
  if (cap < 1) cap = 1;
  if (want > cap) want = cap;
  if (want > ctx->max_splits) want = ctx->max_splits;
  const uint32_t fit = (uint32_t)(ctx->part_slots / ((size_t)total_cols * ctx->cfg.n_heads * groups));   // records: one per (row, split, consumer group)
  if (want > fit) want = fit;
  return want;
}
extern "C" uint32_t pa_plan_splits(pa_ctx* ctx, uint32_t n_rows, uint32_t n_items) {
  if (!ctx || n_items < 1) return 0;
  return plan_splits(ctx, n_rows, n_items);
}

// ------------------------------------------------------------------------------ lifetime --

extern "C" const char* pa_version(void) { return "pooled_attn 0.1 (sm_100a)"; }
extern "C" const char* pa_last_error(pa_ctx* ctx) { return ctx ? ctx->err.c_str() : g_err.c_str(); }

extern "C" int pa_create(int device, const pa_config* cfg, pa_ctx** out) {
  if (!cfg || !out) return fail(nullptr, PA_EINVAL, "pa_create: null argument");
  *out = nullptr;
  if (cfg->n_heads < 1 || cfg->n_kv_heads < 1 || cfg->n_heads % cfg->n_kv_heads)
    return fail(nullptr, PA_EINVAL, "pa_create: n_heads %u must be a multiple of n_kv_heads %u", cfg->n_heads, cfg->n_kv_heads);
  if (cfg->head_dim != 64 && cfg->head_dim != 128 && cfg->head_dim != 256)
    return fail(nullptr, PA_EUNSUPPORTED, "pa_create: head_dim %u is not supported (64, 128 or 256)", cfg->head_dim);
  if (cfg->n_rot > cfg->head_dim || (cfg->n_rot & 1) || (cfg->rope_mode != PA_ROPE_NONE && cfg->n_rot < 2))
    return fail(nullptr, PA_EINVAL, "pa_create: n_rot %u must be even and at most head_dim", cfg->n_rot);
  if (cfg->rope_mode > PA_ROPE_TABLE || cfg->act_dtype > PA_F16) return fail(nullptr, PA_EINVAL, "pa_create: bad rope_mode or act_dtype");
  if (cfg->max_cols < 1) return fail(nullptr, PA_EINVAL, "pa_create: max_cols must be at least 1");
  int n_dev = 0;
  if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev)
    return fail(nullptr, PA_ECUDA, "pa_create: CUDA device %d is not available (%d visible); there is no CPU fallback", device, n_dev);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return fail(nullptr, PA_ECUDA, "pa_create: cannot query device %d", device);
  if (prop.major != 10)
    return fail(nullptr, PA_EUNSUPPORTED, "pa_create: device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
  pa_ctx* ctx = new (std::nothrow) pa_ctx();
  if (!ctx) return fail(nullptr, PA_ENOMEM, "pa_create: out of host memory");
  ctx->device = device;
  ctx->cfg = *cfg;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->smem_optin = (int)prop.sharedMemPerBlockOptin;
  ctx->G = cfg->n_heads / cfg->n_kv_heads;
  ctx->q_dim = cfg->n_heads * cfg->head_dim;
  ctx->kv_dim = cfg->n_kv_heads * cfg->head_dim;
  ctx->max_splits = 256;
  if (const char* e = getenv("POOLED_ATTN_PRE_STAGES")) ctx->tune.pre_stages = atoi(e) < 0 ? 0 : atoi(e);
  if (const char* e = getenv("POOLED_ATTN_NEXT_TILES")) ctx->tune.next_tiles = atoi(e) < 0 ? 0 : atoi(e);
  ctx->tune.no_fuse = getenv("POOLED_ATTN_NO_FUSE") != nullptr;
  ctx->tune.verify_mma_sync = getenv("POOLED_ATTN_VERIFY_MMA_SYNC") != nullptr;
  ctx->tune.no_merge = getenv("POOLED_ATTN_NO_MERGE") != nullptr;
  if (const char* e = getenv("POOLED_ATTN_OWN_PREFETCH")) ctx->tune.own_prefetch = atoi(e);
  if (const char* e = getenv("POOLED_ATTN_XCH_PREFETCH")) ctx->tune.xch_prefetch = atoi(e);
  if (const char* e = getenv("POOLED_ATTN_KV_EVICT_FIRST")) ctx->tune.kv_evict_first = atoi(e) != 0;
  if (const char* e = getenv("POOLED_ATTN_NO_Q_TMA")) ctx->tune.no_q_tma = atoi(e) != 0;
  if (const char* e = getenv("POOLED_ATTN_OLD_TAIL")) ctx->tune.old_tail = atoi(e) != 0;
  if (const char* e = getenv("POOLED_ATTN_NO_OUT_TMA")) ctx->tune.no_out_tma = atoi(e) != 0;
  auto bail = [&](int code, const char* what, cudaError_t e) {
    std::string msg = std::string("pa_create: ") + what + ": " + cudaGetErrorString(e);
    pa_destroy(ctx);
    return fail(nullptr, code, "%s", msg.c_str());
  };
  cudaError_t e;
  if ((e = cudaSetDevice(device)) != cudaSuccess) return bail(PA_ECUDA, "cudaSetDevice", e);
  const uint32_t half = cfg->n_rot / 2;
  if (half) {
    double host[128];
    for (uint32_t i = 0; i < half; ++i) host[i] = pow(cfg->rope_theta, -(2.0 * (double)i) / (double)cfg->n_rot);
    memcpy(ctx->inv_freq_host, host, half * sizeof(double));
    if ((e = cudaMalloc(&ctx->inv_freq, half * sizeof(double))) != cudaSuccess) return bail(PA_ENOMEM, "cudaMalloc(inv_freq)", e);
    if ((e = cudaMemcpy(ctx->inv_freq, host, half * sizeof(double), cudaMemcpyHostToDevice)) != cudaSuccess) return bail(PA_ECUDA, "cudaMemcpy(inv_freq)", e);
  }
  if (half && (e = cudaMalloc(&ctx->angles, (size_t)cfg->max_cols * half * sizeof(Angle))) != cudaSuccess) return bail(PA_ENOMEM, "cudaMalloc(angles)", e);
  if ((e = cudaMalloc(&ctx->q_rot, (size_t)cfg->max_cols * cfg->n_heads * cfg->head_dim * 4)) != cudaSuccess) return bail(PA_ENOMEM, "cudaMalloc(q_rot)", e);
  // split partials: one (o, m, l) record per (query row, split).  A call uses rows * splits of them, about
  // 64 rows x one CTA per SM; the split planner keeps every call inside this capacity.
  ctx->part_slots = 16384;
  if ((e = cudaMalloc(&ctx->part_o, ctx->part_slots * cfg->head_dim * 4)) != cudaSuccess) return bail(PA_ENOMEM, "cudaMalloc(part_o)", e);
  if ((e = cudaMalloc(&ctx->part_ml, ctx->part_slots * 2 * 4)) != cudaSuccess) return bail(PA_ENOMEM, "cudaMalloc(part_ml)", e);
  ctx->merge_slots = 2u * kMaxItems * cfg->n_kv_heads;
  if ((e = cudaMalloc(&ctx->merge_ctr, ctx->merge_slots * 4)) != cudaSuccess) return bail(PA_ENOMEM, "cudaMalloc(merge counters)", e);
  if ((e = cudaMemset(ctx->merge_ctr, 0, ctx->merge_slots * 4)) != cudaSuccess) return bail(PA_ECUDA, "cudaMemset(merge counters)", e);
  if ((e = cudaMalloc(&ctx->dev_err, 4)) != cudaSuccess) return bail(PA_ENOMEM, "cudaMalloc(err)", e);
  if ((e = cudaMemset(ctx->dev_err, 0, 4)) != cudaSuccess) return bail(PA_ECUDA, "cudaMemset(err)", e);
  if ((e = cudaMallocHost(&ctx->host_err, 4)) != cudaSuccess) return bail(PA_ENOMEM, "cudaMallocHost(err)", e);
  *ctx->host_err = 0;
  *out = ctx;
  return PA_OK;
}

extern "C" int pa_destroy(pa_ctx* ctx) {
  if (!ctx) return PA_OK;
  cudaSetDevice(ctx->device);
  cudaFree(ctx->inv_freq); cudaFree(ctx->angles); cudaFree(ctx->norm_q); cudaFree(ctx->norm_k); cudaFree(ctx->q_rot); cudaFree(ctx->k_rot); cudaFree(ctx->part_o); cudaFree(ctx->part_ml); cudaFree(ctx->dev_err); cudaFree(ctx->merge_ctr);
  cudaFree(ctx->stage_dev);
  for (cudaEvent_t e : ctx->ev) cudaEventDestroy(e);
  if (ctx->host_err) cudaFreeHost(ctx->host_err);
  if (ctx->stage_host) cudaFreeHost(ctx->stage_host);
  delete ctx;
  return PA_OK;
}

// bytes of one cache row and of one row of scales in a layer's format
static size_t row_bytes_of(const pa_ctx* ctx, int fmt) { return (size_t)ctx->kv_dim * (fmt == PA_KV_Q8 ? 1 : fmt == PA_KV_F32 ? 4 : 2); }
static size_t scale_row_bytes_of(const pa_ctx* ctx, int fmt) { return fmt == PA_KV_Q8 ? (size_t)ctx->kv_dim / 32 * 4 : 0; }

extern "C" int pa_layer_create_fmt(pa_ctx* ctx, uint32_t n_seqs, uint32_t max_seq, int kv_format, pa_layer** out) {
  if (!ctx || !out) return fail(ctx, PA_EINVAL, "pa_layer_create: null argument");
  *out = nullptr;
  if (n_seqs < 1 || max_seq < 1) return fail(ctx, PA_EINVAL, "pa_layer_create: n_seqs and max_seq must be positive");
  if (kv_format != PA_KV_F16 && kv_format != PA_KV_Q8 && kv_format != PA_KV_F32) return fail(ctx, PA_EINVAL, "pa_layer_create: unknown cache format %d", kv_format);
  if (kv_format != PA_KV_F16 && ctx->G > 16) return fail(ctx, PA_EUNSUPPORTED, "pa_layer_create: int8 / f32 caches take at most 16 query heads per kv head");
  const uint64_t rows = (uint64_t)n_seqs * max_seq;
  if (rows >= (1ull << 31)) return fail(ctx, PA_EUNSUPPORTED, "pa_layer_create: %llu cache rows exceed the 2^31 row limit of one layer", (unsigned long long)rows);
  pa_layer* L = new (std::nothrow) pa_layer();
  if (!L) return fail(ctx, PA_ENOMEM, "pa_layer_create: out of host memory");
  L->ctx = ctx; L->n_seqs = n_seqs; L->max_seq = max_seq; L->kv_format = kv_format;
  cudaSetDevice(ctx->device);
  const size_t bytes = rows * row_bytes_of(ctx, kv_format), sbytes = rows * scale_row_bytes_of(ctx, kv_format);
  size_t free_b = 0, total_b = 0;
  cudaMemGetInfo(&free_b, &total_b);
  void *kp = nullptr, *vp = nullptr;
  bool ok = cudaMalloc(&kp, bytes) == cudaSuccess && cudaMalloc(&vp, bytes) == cudaSuccess;
  if (ok && sbytes) ok = cudaMalloc(&L->k_scale, sbytes) == cudaSuccess && cudaMalloc(&L->v_scale, sbytes) == cudaSuccess;
  if (ok && kv_format != PA_KV_F16 && !ctx->k_rot) ok = cudaMalloc(&ctx->k_rot, (size_t)ctx->cfg.max_cols * ctx->kv_dim * 4) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    cudaFree(kp); cudaFree(vp); cudaFree(L->k_scale); cudaFree(L->v_scale);
    delete L;
    return fail(ctx, PA_ENOMEM, "context %u x %u sequences needs two %.0f MiB KV buffers for this layer; the device has %.0f MiB free (ask for a shorter context or fewer sequences)",
                max_seq, n_seqs, bytes / 1048576.0, free_b / 1048576.0);
  }
  if (kv_format == PA_KV_F16) {
    L->k = (__half*)kp; L->v = (__half*)vp;
    int rc = make_cache_map(ctx, &L->tm_k64, L->k, rows, ctx->kv_dim, ctx->cfg.head_dim, 64);
    if (!rc) rc = make_cache_map(ctx, &L->tm_v64, L->v, rows, ctx->kv_dim, ctx->cfg.head_dim, 64);
    if (rc) { cudaFree(L->k); cudaFree(L->v); delete L; return rc; }
  } else {
    L->k_alt = kp; L->v_alt = vp;
  }
  *out = L;
  return PA_OK;
}
extern "C" int pa_layer_create(pa_ctx* ctx, uint32_t n_seqs, uint32_t max_seq, pa_layer** out) {
  return pa_layer_create_fmt(ctx, n_seqs, max_seq, PA_KV_F16, out);
}

extern "C" int pa_layer_destroy(pa_layer* L) {
  if (!L) return PA_OK;
  cudaSetDevice(L->ctx->device);
  cudaFree(L->k); cudaFree(L->v); cudaFree(L->k_alt); cudaFree(L->v_alt); cudaFree(L->k_scale); cudaFree(L->v_scale);
  delete L;
  return PA_OK;
}

extern "C" int pa_layer_set_origin(pa_layer* L, uint32_t origin) {
  if (!L) return PA_EINVAL;
  L->origin = origin;
  return PA_OK;
}

extern "C" int pa_layer_set_next(pa_layer* L, pa_layer* next) {
  if (!L) return PA_EINVAL;
  if (next && next->ctx != L->ctx) return fail(L->ctx, PA_EINVAL, "pa_layer_set_next: the layers belong to different contexts");
  L->next = next;
  return PA_OK;
}

extern "C" int pa_layer_set_head_norm(pa_layer* L, const float* q_w, const float* k_w, double eps) {
  if (!L) return PA_EINVAL;
  pa_ctx* ctx = L->ctx;
  if ((q_w == nullptr) != (k_w == nullptr)) return fail(ctx, PA_EINVAL, "pa_layer_set_head_norm: give both weights or neither");
  if (q_w && !(eps >= 0.0)) return fail(ctx, PA_EINVAL, "pa_layer_set_head_norm: eps must be a non-negative number");
  if (q_w && ctx->cfg.head_dim > 512) return fail(ctx, PA_EUNSUPPORTED, "pa_layer_set_head_norm: head_dim above 512");
  if (q_w && !ctx->norm_q) {   // scratch for the normed q and k of one layer call, made once
    cudaSetDevice(ctx->device);
    const size_t es = ctx->cfg.act_dtype == PA_F16 ? 2 : 4;
    if (cudaMalloc(&ctx->norm_q, (size_t)ctx->cfg.max_cols * ctx->q_dim * es) != cudaSuccess ||
        cudaMalloc(&ctx->norm_k, (size_t)ctx->cfg.max_cols * ctx->kv_dim * es) != cudaSuccess) {
      cudaGetLastError();
      cudaFree(ctx->norm_q); ctx->norm_q = nullptr;
      return fail(ctx, PA_ENOMEM, "pa_layer_set_head_norm: scratch for the normed q and k does not fit on the device");
    }
  }
  L->qnorm_w = q_w; L->knorm_w = k_w; L->norm_eps = eps;
  return PA_OK;
}

extern "C" void* pa_cache_ptr(pa_layer* L, int which) {
  if (!L) return nullptr;
  if (which == 2) return L->k_scale;
  if (which == 3) return L->v_scale;
  if (L->kv_format != PA_KV_F16) return which ? L->v_alt : L->k_alt;
  return which ? (void*)L->v : (void*)L->k;
}

extern "C" int pa_sync(pa_ctx* ctx, void* stream) {
  if (!ctx) return PA_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  CU_TRY(ctx, cudaMemcpyAsync(ctx->host_err, ctx->dev_err, 4, cudaMemcpyDeviceToHost, st));
  CU_TRY(ctx, cudaStreamSynchronize(st));
  if (*ctx->host_err) {
    ctx->failed = true;
    return fail(ctx, PA_ETIMEOUT, "a device-side wait ran out (code %u); call pa_reset() before the next step", *ctx->host_err);
  }
  return PA_OK;
}

extern "C" int pa_reset(pa_ctx* ctx) {
  if (!ctx) return PA_EINVAL;
  cudaGetLastError();
  if (cudaDeviceSynchronize() != cudaSuccess || cudaMemset(ctx->dev_err, 0, 4) != cudaSuccess ||
      cudaMemset(ctx->merge_ctr, 0, ctx->merge_slots * 4) != cudaSuccess)
    return fail(ctx, PA_ECUDA, "pa_reset: the device does not answer");
  *ctx->host_err = 0;
  ctx->failed = false;
  ctx->err.clear();
  // nothing cached survives a failed step: the angle table is refilled, no early fetch is assumed safe
  ctx->angles_valid = false; ctx->scope_active = false; ctx->scope_fresh = false;
  ctx->inflight_layer = nullptr;
  return PA_OK;
}

extern "C" int pa_get_stats(pa_ctx* ctx, pa_stats* out) {
  if (!ctx || !out) return PA_EINVAL;
  *out = ctx->stats;
  return PA_OK;
}

extern "C" int pa_set_core_only(pa_ctx* ctx, int on) {
  if (!ctx) return PA_EINVAL;
  ctx->core_only = on != 0;
  return PA_OK;
}
extern "C" int pa_timing_begin(pa_ctx* ctx, uint32_t max_events) {
  if (!ctx || max_events < 1) return PA_EINVAL;
  cudaSetDevice(ctx->device);
  while (ctx->ev.size() < 2 * (size_t)max_events) {
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) return fail(ctx, PA_ECUDA, "pa_timing_begin: cudaEventCreate failed");
    ctx->ev.push_back(e);
  }
  ctx->ev_used = 0;
  ctx->timing = true;
  return PA_OK;
}
extern "C" int pa_timing_end(pa_ctx* ctx, double* core_ms, uint64_t* core_launches) {
  if (!ctx || !core_ms || !core_launches) return PA_EINVAL;
  ctx->timing = false;
  double total = 0;
  for (size_t i = 0; i + 1 < ctx->ev_used; i += 2) {
    CU_TRY(ctx, cudaEventSynchronize(ctx->ev[i + 1]));
    float ms = 0;
    CU_TRY(ctx, cudaEventElapsedTime(&ms, ctx->ev[i], ctx->ev[i + 1]));
    total += ms;
  }
  *core_ms = total;
  *core_launches = ctx->ev_used / 2;
  ctx->ev_used = 0;
  return PA_OK;
}
static inline void timing_mark(pa_ctx* ctx, cudaStream_t st, int end) {
  if (!ctx->timing) return;
  if (!end && ctx->ev_used + 2 > ctx->ev.size()) { ctx->timing = false; return; }
  cudaEventRecord(ctx->ev[ctx->ev_used++], st);
}

extern "C" int pa_alloc(pa_ctx* ctx, size_t bytes, void** p) {
  if (!ctx || !p) return PA_EINVAL;
  if (cudaMalloc(p, bytes) != cudaSuccess) { cudaGetLastError(); return fail(ctx, PA_ENOMEM, "pa_alloc: %zu bytes do not fit on the device", bytes); }
  return PA_OK;
}
extern "C" int pa_free(pa_ctx* ctx, void* p) { (void)ctx; cudaFree(p); return PA_OK; }
extern "C" int pa_alloc_host(pa_ctx* ctx, size_t bytes, void** p) {
  if (!ctx || !p) return PA_EINVAL;
  if (cudaMallocHost(p, bytes) != cudaSuccess) { cudaGetLastError(); return fail(ctx, PA_ENOMEM, "pa_alloc_host: cannot pin %zu bytes", bytes); }
  return PA_OK;
}
extern "C" int pa_free_host(pa_ctx* ctx, void* p) { (void)ctx; cudaFreeHost(p); return PA_OK; }
extern "C" int pa_upload(pa_ctx* ctx, void* d, const void* h, size_t n, void* stream) {
  if (!ctx) return PA_EINVAL;
  CU_TRY(ctx, cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return PA_OK;
}
extern "C" int pa_download(pa_ctx* ctx, void* h, const void* d, size_t n, void* stream) {
  if (!ctx) return PA_EINVAL;
  CU_TRY(ctx, cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return PA_OK;
}

// ------------------------------------------------------------------------------ the path --

#define GUARD(ctx)                                                                                       \
  do {                                                                                                   \
    if (!(ctx)) return PA_EINVAL;                                                                        \
    if ((ctx)->failed) return fail((ctx), PA_ESTATE, "an earlier step failed (%s); call pa_reset() first", (ctx)->err.c_str()); \
  } while (0)

// own_rows: the call writes or reads rows pos .. pos+n_cols-1 themselves, which must lie inside this layer's cache
// (for a shard: inside [origin, origin + max_seq)); otherwise any position at or past the origin's sequence is fine
static int check_cols(pa_layer* L, uint32_t seq, uint32_t pos, uint32_t n_cols, const char* who, bool own_rows = true) {
  pa_ctx* ctx = L->ctx;
  if (seq >= L->n_seqs) return fail(ctx, PA_EINVAL, "%s: sequence %u of %u", who, seq, L->n_seqs);
  if (n_cols < 1 || n_cols > ctx->cfg.max_cols) return fail(ctx, PA_EINVAL, "%s: %u columns, the context was created for at most %u", who, n_cols, ctx->cfg.max_cols);
  if ((uint64_t)pos + n_cols >= (1ull << 31)) return fail(ctx, PA_EINVAL, "%s: position %u is out of range", who, pos);
  if (own_rows && (pos < L->origin || (uint64_t)pos + n_cols > (uint64_t)L->origin + L->max_seq))
    return fail(ctx, PA_EINVAL, "%s: positions %u..%u pass the layer's max_seq %u (rows %u..%u)", who, pos, pos + n_cols - 1, L->max_seq,
                L->origin, L->origin + L->max_seq - 1);
  return PA_OK;
}


// cos / sin of a call of at most 64 angles, evaluated by the host's libm and kept while the position repeats (every
// layer of a step asks for the same ones)
static const Angle* host_angles(pa_ctx* ctx, uint32_t pos, uint32_t n_cols) {
  const uint32_t half = ctx->cfg.n_rot / 2;
  if (ctx->host_ang_n != n_cols * half || ctx->host_ang_pos != pos) {
    for (uint32_t c = 0; c < n_cols; ++c)
      for (uint32_t i = 0; i < half; ++i) {
        const double ang = (double)(pos + c) * ctx->inv_freq_host[i];
        ctx->host_ang[c * half + i] = make_angle(cos(ang), sin(ang));
      }
    ctx->host_ang_n = n_cols * half; ctx->host_ang_pos = pos;
  }
  return ctx->host_ang;
}

// Makes ctx->angles hold cos / sin for columns pos .. pos + n_cols - 1, launching pa_angles_kernel unless the table
// already does (same position and width, same capture, and no graph replay can have rewritten it since).
static int ensure_angles(pa_ctx* ctx, uint32_t pos, uint32_t n_cols, cudaStream_t st) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  unsigned long long cap = 0;
  if (cudaStreamGetCaptureInfo(st, &cs, &cap) != cudaSuccess) { cudaGetLastError(); cs = cudaStreamCaptureStatusNone; }
  if (cs != cudaStreamCaptureStatusActive) cap = 0;
  else ctx->ever_captured = true;
  const bool same = ctx->angles_valid && ctx->angles_pos0 == pos && ctx->angles_n == n_cols && ctx->angles_capture == cap;
  const bool trusted = cap != 0 || !ctx->ever_captured || (ctx->scope_active && ctx->scope_fresh);
  if (same && trusted) return PA_OK;
  AnglesParams a{};
  a.out = ctx->angles; a.inv_freq = ctx->inv_freq; a.pos0 = pos; a.n_cols = n_cols; a.half = ctx->cfg.n_rot / 2;
  CU_TRY(ctx, launch_angles(a, st));
  ctx->stats.kernel_launches++;
  ctx->angles_valid = true; ctx->angles_pos0 = pos; ctx->angles_n = n_cols; ctx->angles_capture = cap;
  if (ctx->scope_active) ctx->scope_fresh = true;
  return PA_OK;
}

static int rope_append_impl(pa_layer* L, pa_ctx* ctx, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* q, uint64_t qcs, uint64_t qhs,
                            uint32_t q_heads, void* q_out, uint64_t q_out_cs, const void* k, const void* v, uint64_t kvcs, const float* cs_table,
                            uint32_t mode, int in_f16, cudaStream_t st, int q_out_f16 = 0, bool in_layer_call = false, uint64_t vcs = 0,
                            bool* q_rot_only = nullptr) {   // in: write only the rotated dims of q if the kernel can; out: whether it will
  if (L && L->kv_format != PA_KV_F16) {
    // int8 / f32 caches: q rotated as usual; k rotated into the context's f32 scratch (the rotation kernel's q path,
    // with the kv heads as its heads), then the format's own store kernel -- attn_glue followed by kv_store_q8
    if (n_cols > ctx->cfg.max_cols) return fail(ctx, PA_EINVAL, "rope: %u columns exceed max_cols %u", n_cols, ctx->cfg.max_cols);
    if (q)
      if (int rc = rope_append_impl(nullptr, ctx, seq, pos, n_cols, q, qcs, qhs, q_heads, q_out, q_out_cs, nullptr, nullptr, 0, cs_table, mode, in_f16, st, q_out_f16, in_layer_call))
        return rc;
    if (!k) return PA_OK;
    KvStoreParams sp{};
    sp.format = L->kv_format; sp.kv_dim = ctx->kv_dim; sp.cache_row0 = (uint64_t)seq * L->max_seq + (pos - L->origin);
    sp.k8 = (int8_t*)L->k_alt; sp.v8 = (int8_t*)L->v_alt; sp.ks = L->k_scale; sp.vs = L->v_scale; sp.k32 = (float*)L->k_alt; sp.v32 = (float*)L->v_alt;
    sp.v = v; sp.v_col_stride = vcs ? vcs : kvcs; sp.v_f16 = in_f16;
    if (mode == PA_ROPE_NONE) { sp.k = k; sp.k_col_stride = kvcs; sp.k_f16 = in_f16; }
    else {
      if (int rc = rope_append_impl(nullptr, ctx, seq, pos, n_cols, k, kvcs, ctx->cfg.head_dim, ctx->cfg.n_kv_heads, ctx->k_rot, ctx->kv_dim, nullptr, nullptr, 0, cs_table,
                                    mode, in_f16, st, 0, false))
        return rc;
      sp.k = ctx->k_rot; sp.k_col_stride = ctx->kv_dim; sp.k_f16 = 0;
    }
    CU_TRY(ctx, launch_kv_store(sp, n_cols, st));
    ctx->stats.kernel_launches++;
    ctx->inflight_layer = nullptr;
    return PA_OK;
  }
  RopeParams p{};
  p.q_out_f16 = q_out_f16;
  if (q_out_f16 == 2) p.q_lo_offset = (uint64_t)ctx->cfg.max_cols * ctx->q_dim;   // second half of the f32-sized q_rot buffer
  p.trigger_early = in_layer_call ? 1u : 0u;
  p.q = q; p.q_col_stride = qcs; p.q_head_stride = qhs; p.q_heads = q_heads; p.q_out = q_out; p.q_out_col_stride = q_out_cs;
  p.k = k; p.v = v; p.kv_col_stride = kvcs; p.v_col_stride = vcs ? vcs : kvcs; p.kv_heads = ctx->cfg.n_kv_heads;
  if (L) { p.k_cache = L->k; p.v_cache = L->v; p.cache_row0 = (uint64_t)seq * L->max_seq + (pos - L->origin); }
  p.hd = ctx->cfg.head_dim; p.n_rot = ctx->cfg.n_rot; p.pos = pos; p.mode = mode; p.in_f16 = in_f16;
  p.inv_freq = ctx->inv_freq; p.cs_table = cs_table;
  if (mode == PA_ROPE_TABLE && !cs_table) return fail(ctx, PA_EINVAL, "rope: PA_ROPE_TABLE needs a cos/sin table");
  const uint32_t half = ctx->cfg.n_rot / 2;
  if (mode == PA_ROPE_F64 && half && (q || k)) {
    if (n_cols * half <= 64) {
      // few angles: the host's libm evaluates them (the very values the CPU reference uses) and they travel by value
      p.n_ang = n_cols * half;
      memcpy(p.ang, host_angles(ctx, pos, n_cols), (size_t)p.n_ang * sizeof(Angle));
    } else if (ctx->angles && n_cols <= ctx->cfg.max_cols) {
      if (int rc = ensure_angles(ctx, pos, n_cols, st)) return rc;
      p.angles = ctx->angles;
    }
  }
  if (q_rot_only) {
    *q_rot_only = *q_rot_only && rope_vec_applies(p, n_cols);
    p.q_rot_only = *q_rot_only ? 1u : 0u;
  }
  CU_TRY(ctx, launch_rope_append(p, n_cols, st));
  ctx->stats.kernel_launches++;
  if (L && k) {
    uint32_t r0 = pos - L->origin;
    if (ctx->inflight_layer == L && ctx->inflight_row0 < r0) r0 = ctx->inflight_row0;
    ctx->inflight_layer = L; ctx->inflight_row0 = r0;
  }
  return PA_OK;
}

extern "C" int pa_rope(pa_ctx* ctx, const void* x, uint64_t col_stride, uint64_t head_stride, uint32_t n_heads_x, uint32_t pos, uint32_t n_cols,
                       const float* cs_table, float* y, uint64_t y_col_stride, void* stream) {
  GUARD(ctx);
  if (!x || !y || n_cols < 1 || n_heads_x < 1) return fail(ctx, PA_EINVAL, "pa_rope: null or empty argument");
  cudaSetDevice(ctx->device);
  return rope_append_impl(nullptr, ctx, 0, pos, n_cols, x, col_stride, head_stride, n_heads_x, y, y_col_stride, nullptr, nullptr, 0, cs_table,
                          ctx->cfg.rope_mode, ctx->cfg.act_dtype == PA_F16, (cudaStream_t)stream);
}

extern "C" int pa_kv_append(pa_layer* L, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* k, const void* v, uint64_t col_stride, int dtype,
                            void* stream) {
  if (!L) return PA_EINVAL;
  pa_ctx* ctx = L->ctx;
  GUARD(ctx);
  if (!k || !v) return fail(ctx, PA_EINVAL, "pa_kv_append: null k or v");
  if (int rc = check_cols(L, seq, pos, n_cols, "pa_kv_append")) return rc;
  cudaSetDevice(ctx->device);
  return rope_append_impl(L, ctx, seq, pos, n_cols, nullptr, 0, 0, 0, nullptr, 0, k, v, col_stride, nullptr, PA_ROPE_NONE, dtype == PA_F16,
                          (cudaStream_t)stream);
}

extern "C" int pa_rope_append(pa_layer* L, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* q, uint64_t q_col_stride, uint64_t q_head_stride,
                              const void* k, const void* v, uint64_t kv_col_stride, const float* cs_table, float* q_rot, void* stream) {
  if (!L) return PA_EINVAL;
  pa_ctx* ctx = L->ctx;
  GUARD(ctx);
  if (!q || !k || !v) return fail(ctx, PA_EINVAL, "pa_rope_append: null q, k or v");
  if (int rc = check_cols(L, seq, pos, n_cols, "pa_rope_append")) return rc;
  cudaSetDevice(ctx->device);
  return rope_append_impl(L, ctx, seq, pos, n_cols, q, q_col_stride, q_head_stride, ctx->cfg.n_heads, q_rot ? q_rot : ctx->q_rot, ctx->q_dim, k, v,
                          kv_col_stride, cs_table, ctx->cfg.rope_mode, ctx->cfg.act_dtype == PA_F16, (cudaStream_t)stream);
}

static int rope_append_items_impl(pa_layer* L, const pa_item* items, uint32_t n_items, const void* q, uint64_t q_col_stride, uint64_t q_head_stride,
                                  const void* k, const void* v, uint64_t kv_col_stride, uint64_t v_col_stride, float* q_rot, void* stream) {
  pa_ctx* ctx = L->ctx;
  if (!q || !k || !v || !items) return fail(ctx, PA_EINVAL, "pa_rope_append_items: null q, k, v or items");
  if (n_items < 1 || n_items > 32) return fail(ctx, PA_EINVAL, "pa_rope_append_items: 1 to 32 items per call");
  if (n_items > ctx->cfg.max_cols && !q_rot) return fail(ctx, PA_EINVAL, "pa_rope_append_items: %u items exceed max_cols %u", n_items, ctx->cfg.max_cols);
  if (ctx->cfg.rope_mode == PA_ROPE_TABLE) return fail(ctx, PA_EUNSUPPORTED, "pa_rope_append_items: PA_ROPE_TABLE takes one table per call; use pa_rope_append per sequence");
  cudaSetDevice(ctx->device);
  RopeParams p{};
  p.q = q; p.q_col_stride = q_col_stride; p.q_head_stride = q_head_stride; p.q_heads = ctx->cfg.n_heads;
  p.q_out = q_rot ? q_rot : ctx->q_rot; p.q_out_col_stride = ctx->q_dim;
  p.k = k; p.v = v; p.kv_col_stride = kv_col_stride; p.v_col_stride = v_col_stride; p.kv_heads = ctx->cfg.n_kv_heads;
  p.k_cache = L->k; p.v_cache = L->v;
  p.hd = ctx->cfg.head_dim; p.n_rot = ctx->cfg.n_rot; p.mode = ctx->cfg.rope_mode; p.in_f16 = ctx->cfg.act_dtype == PA_F16;
  p.inv_freq = ctx->inv_freq;
  p.n_items = n_items;
  const uint32_t half = ctx->cfg.n_rot / 2;
  uint32_t row0 = 0xffffffffu;
  for (uint32_t i = 0; i < n_items; ++i) {
    const pa_item& it = items[i];
    if (it.n_cols != 1) return fail(ctx, PA_EINVAL, "pa_rope_append_items: item %u has %u columns; one token per item", i, it.n_cols);
    if (it.seq >= L->n_seqs) return fail(ctx, PA_EINVAL, "pa_rope_append_items: item %u: sequence %u of %u", i, it.seq, L->n_seqs);
    p.item_pos[i] = it.pos;
    const bool owns = it.pos >= L->origin && it.pos - L->origin < L->max_seq;
    p.item_row[i] = owns ? (uint64_t)it.seq * L->max_seq + (it.pos - L->origin) : ~0ull;
    if (owns && it.pos - L->origin < row0) row0 = it.pos - L->origin;
    if (p.mode == PA_ROPE_F64 && n_items * half <= 64)
      for (uint32_t j = 0; j < half; ++j) {
        const double ang = (double)it.pos * ctx->inv_freq_host[j];
        p.ang[i * half + j] = make_angle(cos(ang), sin(ang));
      }
  }
  if (p.mode == PA_ROPE_F64 && n_items * half <= 64) p.n_ang = n_items * half;
  CU_TRY(ctx, launch_rope_append(p, n_items, (cudaStream_t)stream));
  ctx->stats.kernel_launches++;
  // what the kernel just launched may still be writing: rows from row0 on (none on a shard that owns no item's row)
  if (ctx->inflight_layer == L && ctx->inflight_row0 < row0) row0 = ctx->inflight_row0;
  ctx->inflight_layer = L; ctx->inflight_row0 = row0;
  return PA_OK;
}

extern "C" int pa_rope_append_items(pa_layer* L, const pa_item* items, uint32_t n_items, const void* q, uint64_t q_col_stride, uint64_t q_head_stride,
                                    const void* k, const void* v, uint64_t kv_col_stride, float* q_rot, void* stream) {
  if (!L) return PA_EINVAL;
  GUARD(L->ctx);
  if (L->kv_format != PA_KV_F16) return fail(L->ctx, PA_EUNSUPPORTED, "pa_rope_append_items: f16 caches only; use pa_rope_append per sequence");
  return rope_append_items_impl(L, items, n_items, q, q_col_stride, q_head_stride, k, v, kv_col_stride, kv_col_stride, q_rot, stream);
}

static int build_items(pa_layer* L, const pa_item* items, uint32_t n_items, ItemList* il, uint32_t* total_cols, uint32_t* max_rows, uint32_t* max_cols,
                       uint64_t* kv_bytes, const char* who, bool sharded_ok) {
  pa_ctx* ctx = L->ctx;
  if (!items || n_items < 1 || n_items > (uint32_t)kMaxItems) return fail(ctx, PA_EINVAL, "%s: between 1 and %d items per call", who, kMaxItems);
  uint32_t cols = 0, mr = 0, mc = 0;
  uint64_t bytes = 0;
  for (uint32_t i = 0; i < n_items; ++i) {
    if (int rc = check_cols(L, items[i].seq, items[i].pos, items[i].n_cols, who, sharded_ok ? false : true)) return rc;
    if (items[i].n_cols * ctx->G > (uint32_t)kMaxRows)
      return fail(ctx, PA_EUNSUPPORTED, "%s: %u columns x %u heads per kv head exceed the %d query rows one pass carries; use pa_prefill", who,
                  items[i].n_cols, ctx->G, kMaxRows);
    const int64_t end = (int64_t)items[i].pos + items[i].n_cols - (int64_t)L->origin;
    const uint32_t rows = (uint32_t)(end < 0 ? 0 : end > (int64_t)L->max_seq ? L->max_seq : end);
    il->seq[i] = items[i].seq; il->n_cols[i] = items[i].n_cols; il->col0[i] = cols; il->pos[i] = items[i].pos;
    il->lim0[i] = (int32_t)((int64_t)items[i].pos + 1 - (int64_t)L->origin); il->n_rows[i] = rows;
    cols += items[i].n_cols;
    if (rows > mr) mr = rows;
    if (items[i].n_cols > mc) mc = items[i].n_cols;
    bytes += 2ull * rows * ctx->kv_dim * 2;
  }
  if (cols > ctx->cfg.max_cols || (size_t)cols * ctx->cfg.n_heads > ctx->part_slots)
    return fail(ctx, PA_EINVAL, "%s: %u columns in one call exceed the context's max_cols %u", who, cols, ctx->cfg.max_cols);
  *total_cols = cols; *max_rows = mr; *max_cols = mc; *kv_bytes = bytes;
  return PA_OK;
}


// the tokens' unrotated k / v rows for the fused front of the decode kernel: one item at `pos` (cos / sin from the
// host), or one token of each of several items (kv_stride elements between their rows; cos / sin on the device)
struct FusedFront { const void* k; const void* v; uint32_t append_mask; uint32_t pos; uint64_t k_stride = 0, v_stride = 0; bool device_angles = false; };

// a gathered call: the columns' row lists on the device, one list of `stride` words per column
struct GatherLists { const uint32_t* lists; uint32_t stride; };

// Decode / verify / prefill over an int8 or f32 cache: per item, blocks of columns small enough for the record buffers;
// each block is one launch of the plain split-K kernel (a CTA per (split, kv head, column)) and one combine.
static int decode_any_impl(pa_layer* L, const pa_item* items, uint32_t n_items, const void* q, int q_dtype, uint64_t qcs, uint64_t qhs, const void* gate,
                           uint64_t gcs, uint64_t ghs, void* out, uint64_t ocs, cudaStream_t st, const char* who) {
  pa_ctx* ctx = L->ctx;
  if (!q || !out) return fail(ctx, PA_EINVAL, "%s: null q or output", who);
  if (!items || n_items < 1) return fail(ctx, PA_EINVAL, "%s: no items", who);
  cudaSetDevice(ctx->device);
  const size_t qes = q_dtype == PA_F16 ? 2 : 4, aes = ctx->cfg.act_dtype == PA_F16 ? 2 : 4;
  const uint32_t hd = ctx->cfg.head_dim, nH = ctx->cfg.n_heads;
  const uint32_t block = std::max<uint32_t>(1u, (uint32_t)(ctx->part_slots / (4ull * nH)));   // columns per launch: room for four splits at least
  uint64_t col = 0;
  for (uint32_t i = 0; i < n_items; ++i) {
    if (int rc = check_cols(L, items[i].seq, items[i].pos, items[i].n_cols, who)) return rc;
    for (uint32_t c0 = 0; c0 < items[i].n_cols; c0 += block) {
      const uint32_t nc = std::min(block, items[i].n_cols - c0);
      const uint32_t pos0 = items[i].pos + c0;
      const uint32_t rows = pos0 + nc - L->origin;                 // rows the block's last column sees
      const uint32_t ns = plan_splits(ctx, rows, 1, nc, 1);
      AnyDecodeParams a{};
      a.q = reinterpret_cast<const uint8_t*>(q) + (col + c0) * qcs * qes; a.q_f16 = q_dtype == PA_F16; a.q_col_stride = qcs; a.q_head_stride = qhs;
      a.k = L->k_alt; a.v = L->v_alt; a.ks = L->k_scale; a.vs = L->v_scale;
      a.kv_dim = ctx->kv_dim; a.hd = hd; a.G = ctx->G; a.n_heads = nH; a.max_seq = L->max_seq; a.n_splits = ns;
      a.seq = items[i].seq; a.lim0 = (int32_t)(pos0 + 1 - L->origin); a.n_rows = rows; a.col0 = 0;
      a.part_o = ctx->part_o; a.part_ml = ctx->part_ml;
      timing_mark(ctx, st, 0);
      CU_TRY(ctx, launch_decode_any(a, L->kv_format, dim3(ns, ctx->cfg.n_kv_heads, nc), st));
      timing_mark(ctx, st, 1);
      CombineParams c{};
      c.o = ctx->part_o; c.ml = ctx->part_ml;
      c.o_row_stride = (uint64_t)ns * hd; c.o_part_stride = hd; c.ml_row_stride = (uint64_t)ns * 2; c.ml_part_stride = 2;
      c.n_heads = nH; c.fixed_parts = 0; c.n_splits = ns; c.groups = 1;
      c.gate = gate ? reinterpret_cast<const uint8_t*>(gate) + (col + c0) * gcs * aes : nullptr; c.gate_col_stride = gcs; c.gate_head_stride = ghs;
      c.out = reinterpret_cast<uint8_t*>(out) + (col + c0) * ocs * aes; c.out_col_stride = ocs; c.act_f16 = ctx->cfg.act_dtype == PA_F16;
      c.items.seq[0] = items[i].seq; c.items.lim0[0] = a.lim0; c.items.n_rows[0] = rows; c.items.n_cols[0] = nc; c.items.col0[0] = 0; c.n_items = 1;
      c.err = ctx->dev_err;
      if (!ctx->core_only) CU_TRY(ctx, launch_combine((int)hd, c, nc * nH, st));
      ctx->stats.kernel_launches += ctx->core_only ? 1 : 2;
      ctx->stats.kv_bytes_streamed += 2ull * rows * (row_bytes_of(ctx, L->kv_format) + scale_row_bytes_of(ctx, L->kv_format));
    }
    col += items[i].n_cols;
  }
  ctx->stats.calls++;
  ctx->inflight_layer = nullptr;
  return PA_OK;
}

static int decode_impl(pa_layer* L, const pa_item* items, uint32_t n_items, const void* q, int q_dtype, uint64_t qcs, uint64_t qhs, const void* gate,
                       uint64_t gcs, uint64_t ghs, void* out, uint64_t ocs, float* partial, cudaStream_t st, const char* who, bool after_own_append = false,
                       bool exchange = false, const FusedFront* fz = nullptr, const void* q_lo = nullptr, const GatherLists* gl = nullptr) {
  pa_ctx* ctx = L->ctx;
  if (L->kv_format != PA_KV_F16) {
    if (partial || exchange || gl) return fail(ctx, PA_EUNSUPPORTED, "%s: partial records, the peer exchange and row lists are for f16 caches", who);
    return decode_any_impl(L, items, n_items, q, q_dtype, qcs, qhs, gate, gcs, ghs, out, ocs, st, who);
  }
  if (!q || (!out && !partial)) return fail(ctx, PA_EINVAL, "%s: null q or output", who);
  if ((qcs & 1) || (qhs & 1) || ((uintptr_t)q & 7)) return fail(ctx, PA_EINVAL, "%s: q strides must be even and q 8-byte aligned", who);
  DecodeParams p{};
  uint32_t total_cols, max_rows, max_cols; uint64_t kv_bytes;
  // partial records may come from a shard that holds only part (or none) of the rows the columns see
  if (int rc = build_items(L, items, n_items, &p.items, &total_cols, &max_rows, &max_cols, &kv_bytes, who, partial != nullptr || exchange)) return rc;
  if (exchange) {
    if (!ctx->xc.world) return fail(ctx, PA_EINVAL, "%s: call pa_exchange_init first", who);
    if ((uint64_t)total_cols * ctx->cfg.n_heads > ctx->xc.max_rows)
      return fail(ctx, PA_EUNSUPPORTED, "%s: %u query rows exceed the %u rows of the exchange buffers", who, total_cols * ctx->cfg.n_heads, ctx->xc.max_rows);
  }
  cudaSetDevice(ctx->device);
  const int nt = (int)ceil_div(max_cols * ctx->G, 8);
  // One sequence with more than 8 query rows per kv head (a k-token verify block) goes to the tensor-core split-K
  // kernel; single tokens and batches of sequences stay on the streaming mma.sync kernel.
  const bool verify_tc = n_items == 1 && nt > 1 && max_rows > 0 && !ctx->tune.verify_mma_sync && !gl && ctx->cfg.head_dim >= 128;
  const uint32_t groups = 1u;   // records per split: one, whatever the number of consumer groups
  uint32_t ns = plan_splits(ctx, max_rows, n_items, total_cols, groups);
  if (gl) {
    // the lists' lengths live on the device: the grid is sized for the longest list possible and each CTA derives its
    // own column's plan (plan_splits' rule without the cap by the row count, which the kernel applies)
    ns = plan_splits(ctx, 0x40000000u, n_items, total_cols, groups);
    const uint32_t most = std::max(1u, ceil_div(gl->stride - 1, 64) / 2);
    if (ns > most) ns = most;
    p.gather = gl->lists; p.gather_stride = gl->stride; p.k_cache = L->k; p.v_cache = L->v;
  }
  if (n_items == 1 && max_cols * ctx->G > 8) { const uint32_t fit = (uint32_t)(ctx->part_slots / (2ull * total_cols * ctx->cfg.n_heads)); if (ns > fit) ns = fit; if (ns > 256) ns = 256; if (ns < 1) ns = 1; }
  p.q = q; p.q_f16 = q_dtype == PA_F16; p.q_col_stride = qcs; p.q_head_stride = qhs;
  p.part_o = ctx->part_o; p.part_ml = ctx->part_ml; p.n_splits = ns;
  p.n_heads = ctx->cfg.n_heads; p.G = ctx->G; p.max_seq = L->max_seq;
  p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)ctx->cfg.head_dim));
  p.err = ctx->dev_err;
  // after this library's own RoPE/append kernel the only rows in flux are the call's new ones: older rows may be
  // fetched while that kernel still runs
  p.prefetch_old_rows = after_own_append ? 1u : 0u;
  p.early_limit = (after_own_append && ctx->inflight_layer == L) ? ctx->inflight_row0 : 0xffffffffu;
  p.pre_stages = (uint32_t)ctx->tune.pre_stages;
  p.kv_evict_first = ctx->tune.kv_evict_first ? 1u : 0u;
  // tiles beyond the ring asked into L2 ahead of the wait: on a shard the wait spans the cross-GPU exchange of the call
  // before, a window in which HBM would otherwise idle
  p.own_prefetch = (uint32_t)std::max(0, exchange ? ctx->tune.xch_prefetch : ctx->tune.own_prefetch);
  p.next_tiles = (L->next && L->next->ctx == ctx) ? (uint32_t)ctx->tune.next_tiles : 0u;
  if (fz) {
    p.fused = fz->device_angles ? 2u : 1u; p.append = fz->append_mask; p.k_new = fz->k; p.v_new = fz->v;
    p.k_new_stride = fz->k_stride; p.v_new_stride = fz->v_stride; p.inv_freq = ctx->inv_freq;
    p.k_cache = L->k; p.v_cache = L->v;
    if (!fz->device_angles) memcpy(p.rope_ang, host_angles(ctx, fz->pos, 1), (size_t)(ctx->cfg.n_rot / 2) * sizeof(Angle));
  }
  CUtensorMap tm_k, tm_v;
  PrefillParams vp{};
  if (verify_tc) {
    const uint64_t seq_off = (uint64_t)items[0].seq * L->max_seq * ctx->kv_dim;
    if (int rc = make_cache_map(ctx, &tm_k, L->k + seq_off, max_rows, ctx->kv_dim, ctx->cfg.head_dim, 64)) return rc;
    if (int rc = make_cache_map(ctx, &tm_v, L->v + seq_off, max_rows, ctx->kv_dim, ctx->cfg.head_dim, 64)) return rc;
    vp.q = q; vp.q_f16 = q_dtype == PA_F16; vp.q_col_stride = qcs; vp.q_head_stride = qhs; vp.q_lo = q_lo;
    vp.n_cols = items[0].n_cols; vp.n_heads = ctx->cfg.n_heads; vp.G = ctx->G; vp.max_seq = L->max_seq;
    vp.scale_log2 = p.scale_log2; vp.err = ctx->dev_err;
    vp.prefetch_old_rows = after_own_append ? 1u : 0u; vp.early_limit = p.early_limit; vp.pre_stages = p.pre_stages; vp.kv_evict_first = p.kv_evict_first;
    vp.part_o = ctx->part_o; vp.part_ml = ctx->part_ml; vp.n_splits = ns; vp.lim0 = p.items.lim0[0]; vp.n_rows = max_rows; vp.col0 = 0;
    const uint64_t am = q_dtype == PA_F16 ? 7 : 3;
    if ((qcs & am) || (qhs & am) || ((uintptr_t)q & 15)) return fail(ctx, PA_EINVAL, "%s: a multi-column block needs q strides that are multiples of 16 bytes and q 16-byte aligned", who);
  }
  // One kernel per call where the merge can be shared out among the call's own CTAs: all of them resident at once (one
  // wave at one CTA per SM), and at least half as many CTAs per (item, kv head) as there are (row, 64-dim slice) units.
  // Not on a KV-sequence shard: there the combine kernel, whose small CTAs wait for the other GPUs beside the next
  // call's decode CTAs (already fetching their first tiles), measured faster than decode CTAs that hold their SMs
  // through the exchange.
  const uint32_t units = max_cols * ctx->G * (ctx->cfg.head_dim / 64);
  bool all_rows = true;   // on a shard an item may have no row here: its CTAs never run, so its units must be the combine kernel's
  for (uint32_t i = 0; i < n_items; ++i) all_rows = all_rows && p.items.n_rows[i] > 0;
  const bool merge = !partial && !exchange && !verify_tc && nt <= 2 && all_rows && !ctx->core_only && !ctx->tune.no_merge && max_rows > 0 &&
                     (uint64_t)ns * ctx->cfg.n_kv_heads * n_items <= (uint64_t)ctx->sm_count && 2 * ns >= units;
  if (merge) {
    p.merge = ctx->tune.old_tail ? 1u : 2u; p.merge_ctr = ctx->merge_ctr;
    p.gate = gate; p.gate_col_stride = gcs; p.gate_head_stride = ghs; p.out = out; p.out_col_stride = ocs; p.act_f16 = ctx->cfg.act_dtype == PA_F16;
  }
  // an exchanging call numbers itself ahead of its combine kernel: in the decode kernel where that runs
  const bool decode_runs = !verify_tc && max_rows > 0;
  if (exchange && !ctx->core_only) {
    if (decode_runs) p.xch_ctr = ctx->xc.ctr;
    else { CU_TRY(ctx, launch_epoch_bump(ctx->xc.ctr, st)); ctx->stats.kernel_launches++; }
  }
  timing_mark(ctx, st, 0);
  if (verify_tc) CU_TRY(ctx, launch_verify(L, vp, tm_k, tm_v, ctx->cfg.n_kv_heads, st));
  else if (max_rows > 0) CU_TRY(ctx, launch_decode(L, p, dim3(ns, ctx->cfg.n_kv_heads, n_items), nt, st));
  timing_mark(ctx, st, 1);
  CombineParams c{};
  c.o = ctx->part_o; c.ml = ctx->part_ml;
  const uint32_t rs = ns * groups;
  c.o_row_stride = (uint64_t)rs * ctx->cfg.head_dim; c.o_part_stride = ctx->cfg.head_dim;
  c.ml_row_stride = (uint64_t)rs * 2; c.ml_part_stride = 2;
  c.n_heads = ctx->cfg.n_heads; c.fixed_parts = 0; c.n_splits = ns; c.groups = groups;
  c.gather = p.gather; c.gather_stride = p.gather_stride;
  c.gate = gate; c.gate_col_stride = gcs; c.gate_head_stride = ghs; c.out = out; c.out_col_stride = ocs;
  c.act_f16 = ctx->cfg.act_dtype == PA_F16;
  c.partial_out = partial; c.partial_rows = (uint64_t)total_cols * ctx->cfg.n_heads;
  c.exchange = exchange ? 1 : 0; c.xc = ctx->xc; c.err = ctx->dev_err;
  c.xch_sweeps = ctx->tune.wait_polls ? ctx->tune.wait_polls : (1u << 20);
  c.items = p.items; c.n_items = n_items;
  if (!ctx->core_only && !merge) CU_TRY(ctx, launch_combine((int)ctx->cfg.head_dim, c, total_cols * ctx->cfg.n_heads, st));
  ctx->stats.kernel_launches += (ctx->core_only || merge) ? 1 : 2; ctx->stats.kv_bytes_streamed += kv_bytes; ctx->stats.calls++;
  // this call's kernel waited for everything before it; what it appends itself is what may still be in flight
  if (fz && fz->append_mask) {
    uint32_t r0 = 0xffffffffu;
    for (uint32_t i = 0; i < n_items; ++i)
      if ((fz->append_mask >> i) & 1u) r0 = std::min(r0, p.items.n_rows[i] ? p.items.n_rows[i] - 1 : 0u);
    ctx->inflight_layer = L; ctx->inflight_row0 = r0;
  } else ctx->inflight_layer = nullptr;
  return PA_OK;
}

extern "C" int pa_decode(pa_layer* L, const pa_item* items, uint32_t n_items, const void* q, int q_dtype, uint64_t q_col_stride, uint64_t q_head_stride,
                         const void* gate, uint64_t gate_col_stride, uint64_t gate_head_stride, void* out, uint64_t out_col_stride, void* stream) {
  if (!L) return PA_EINVAL;
  GUARD(L->ctx);
  if (!out) return fail(L->ctx, PA_EINVAL, "pa_decode: null out");
  if (!q) {   // the rotated q a preceding pa_rope_append / pa_rope_append_items left in the context (q_rot = NULL there)
    q = L->ctx->q_rot; q_dtype = PA_F32; q_col_stride = L->ctx->q_dim; q_head_stride = L->ctx->cfg.head_dim;
  }
  // straight after this library's own append into the layer (the kernel before this one on the stream), rows older
  // than the appended ones may be fetched while that kernel still runs
  return decode_impl(L, items, n_items, q, q_dtype, q_col_stride, q_head_stride, gate, gate_col_stride, gate_head_stride, out, out_col_stride, nullptr,
                     (cudaStream_t)stream, "pa_decode", L->ctx->inflight_layer == L);
}

extern "C" int pa_decode_gather(pa_layer* L, uint32_t seq, uint32_t n_cols, const uint32_t* row_lists, uint32_t list_stride, const void* q, int q_dtype,
                                uint64_t q_col_stride, uint64_t q_head_stride, const void* gate, uint64_t gate_col_stride, uint64_t gate_head_stride,
                                void* out, uint64_t out_col_stride, void* stream) {
  if (!L) return PA_EINVAL;
  pa_ctx* ctx = L->ctx;
  GUARD(ctx);
  if (!out || !row_lists) return fail(ctx, PA_EINVAL, "pa_decode_gather: null out or row lists");
  if (n_cols < 1 || n_cols > (uint32_t)kMaxItems) return fail(ctx, PA_EINVAL, "pa_decode_gather: 1 to %d columns per call", kMaxItems);
  if (list_stride < 2 || ((uintptr_t)row_lists & 3)) return fail(ctx, PA_EINVAL, "pa_decode_gather: list_stride must be at least 2 (the length word and one row)");
  if (seq >= L->n_seqs) return fail(ctx, PA_EINVAL, "pa_decode_gather: sequence %u of %u", seq, L->n_seqs);
  if (ctx->G > 8) return fail(ctx, PA_EUNSUPPORTED, "pa_decode_gather: more than 8 query heads per kv head");
  // every column is its own item (its list is its own K/V stream); positions are list positions, all of them visible
  pa_item items[kMaxItems];
  const uint32_t longest = std::min<uint32_t>(list_stride - 1, L->max_seq);
  for (uint32_t c = 0; c < n_cols; ++c) items[c] = pa_item{seq, L->origin + longest - 1, 1, 0};
  GatherLists gl{row_lists, list_stride};
  return decode_impl(L, items, n_cols, q, q_dtype, q_col_stride, q_head_stride, gate, gate_col_stride, gate_head_stride, out, out_col_stride, nullptr,
                     (cudaStream_t)stream, "pa_decode_gather", false, false, nullptr, nullptr, &gl);
}

extern "C" int pa_decode_partial(pa_layer* L, const pa_item* items, uint32_t n_items, const void* q, int q_dtype, uint64_t q_col_stride,
                                 uint64_t q_head_stride, float* partial, void* stream) {
  if (!L) return PA_EINVAL;
  GUARD(L->ctx);
  if (!partial) return fail(L->ctx, PA_EINVAL, "pa_decode_partial: null partial");
  return decode_impl(L, items, n_items, q, q_dtype, q_col_stride, q_head_stride, nullptr, 0, 0, nullptr, 0, partial, (cudaStream_t)stream,
                     "pa_decode_partial");
}

extern "C" int pa_merge(pa_ctx* ctx, const float* parts, uint32_t n_parts, uint32_t n_cols, const void* gate, uint64_t gate_col_stride,
                        uint64_t gate_head_stride, void* out, uint64_t out_col_stride, void* stream) {
  GUARD(ctx);
  if (!parts || !out || n_parts < 1 || n_parts > 512 || n_cols < 1) return fail(ctx, PA_EINVAL, "pa_merge: null argument, or n_parts outside 1..512");
  cudaSetDevice(ctx->device);
  const uint64_t rows = (uint64_t)n_cols * ctx->cfg.n_heads, hd = ctx->cfg.head_dim;
  CombineParams c{};
  c.o = parts; c.ml = parts + rows * hd;
  c.o_row_stride = hd; c.o_part_stride = rows * (hd + 2);
  c.ml_row_stride = 2; c.ml_part_stride = rows * (hd + 2);
  c.n_heads = ctx->cfg.n_heads; c.fixed_parts = n_parts; c.n_splits = 1;
  c.gate = gate; c.gate_col_stride = gate_col_stride; c.gate_head_stride = gate_head_stride; c.out = out; c.out_col_stride = out_col_stride;
  c.act_f16 = ctx->cfg.act_dtype == PA_F16;
  c.err = ctx->dev_err;
  CU_TRY(ctx, launch_combine((int)hd, c, (uint32_t)rows, (cudaStream_t)stream));
  ctx->stats.kernel_launches++;
  return PA_OK;
}

// the caller's own (unrotated) f16 q of a layer call whose RoPE kernel wrote only the rotated dims of the rotated q
struct PlainQ { const void* q; uint64_t cs, hs; };

static bool q_tma_ok(const pa_ctx* ctx, int q_dtype, uint64_t qcs, uint64_t qhs, const void* q) {
  return q_dtype == PA_F16 && ctx->cfg.head_dim == 256 && !(qcs & 63) && !(qhs & 63) && !((uintptr_t)q & 15) && !ctx->tune.no_q_tma;
}

static int prefill_impl(pa_layer* L, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* q, int q_dtype, uint64_t qcs, uint64_t qhs, const void* gate,
                        uint64_t gcs, uint64_t ghs, void* out, uint64_t ocs, cudaStream_t st, const PlainQ* plain = nullptr) {
  pa_ctx* ctx = L->ctx;
  if (!q || !out) return fail(ctx, PA_EINVAL, "pa_prefill: null q or out");
  if (L->kv_format != PA_KV_F16) {   // every column attended on its own, as the reference's kernels for these formats do
    if (n_cols < 1 || n_cols > ctx->cfg.max_cols) return fail(ctx, PA_EINVAL, "pa_prefill: %u columns, the context was created for at most %u", n_cols, ctx->cfg.max_cols);
    pa_item it{seq, pos, n_cols, 0};
    return decode_any_impl(L, &it, 1, q, q_dtype, qcs, qhs, gate, gcs, ghs, out, ocs, st, "pa_prefill");
  }
  if (int rc = check_cols(L, seq, pos, n_cols, "pa_prefill")) return rc;
  if (!prefill_supported(ctx)) return fail(ctx, PA_EUNSUPPORTED, "pa_prefill: head_dim %u is outside the tiled prefill kernel's shapes", ctx->cfg.head_dim);
  const uint64_t qm = q_dtype == PA_F16 ? 7 : 3, om = ctx->cfg.act_dtype == PA_F16 ? 7 : 3;   // 16-byte vector accesses
  if ((qcs & qm) || (qhs & qm) || ((uintptr_t)q & 15)) return fail(ctx, PA_EINVAL, "pa_prefill: q strides must be multiples of 16 bytes and q 16-byte aligned");
  if ((ocs & om) || ((uintptr_t)out & 15)) return fail(ctx, PA_EINVAL, "pa_prefill: the out column stride must be a multiple of 16 bytes and out 16-byte aligned");
  cudaSetDevice(ctx->device);
  PrefillParams p{};
  p.q = q; p.q_f16 = q_dtype == PA_F16; p.q_col_stride = qcs; p.q_head_stride = qhs;
  p.gate = gate; p.gate_col_stride = gcs; p.gate_head_stride = ghs; p.out = out; p.out_col_stride = ocs;
  p.act_f16 = ctx->cfg.act_dtype == PA_F16;
  p.seq = seq; p.pos = pos - L->origin; p.n_cols = n_cols; p.n_heads = ctx->cfg.n_heads; p.G = ctx->G; p.max_seq = L->max_seq;
  p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)ctx->cfg.head_dim));
  p.err = ctx->dev_err;
  // Tensor maps of this call: the sequence's rows [0, pos + n_cols) only, so that a K/V tile reaching past the last
  // appended row is zero-filled by TMA instead of carrying whatever the cache holds there (0 * NaN is NaN).
  CUtensorMap tm_k, tm_v;
  const uint64_t seq_off = (uint64_t)seq * L->max_seq * ctx->kv_dim;
  if (int rc = make_cache_map(ctx, &tm_k, L->k + seq_off, (uint64_t)p.pos + n_cols, ctx->kv_dim, ctx->cfg.head_dim, 64)) return rc;
  if (int rc = make_cache_map(ctx, &tm_v, L->v + seq_off, (uint64_t)p.pos + n_cols, ctx->kv_dim, ctx->cfg.head_dim, 64)) return rc;
  // f16 query rows at head_dim 256 travel by TMA: a map of q as [n_cols][q_col_stride] in 64-element chunks, the same
  // shape of map as a cache's (rows past n_cols read as zeros)
  CUtensorMap tm_q = tm_k, tm_q2 = tm_k;
  if (plain) {
    // the rotated chunks of a head from the rotated q, the others from the caller's q (the caller checked q_tma_ok for both)
    const uint32_t rot = ctx->cfg.n_rot;
    if (int rc = make_cache_map(ctx, &tm_q, const_cast<void*>(q), n_cols, (uint32_t)qcs, rot, 128)) return rc;
    if (int rc = make_cache_map(ctx, &tm_q2, const_cast<void*>(plain->q), n_cols, (uint32_t)plain->cs, ctx->cfg.head_dim - rot, 128)) return rc;
    p.q_tma = 2; p.q_rot_chunks = rot / 64; p.q2_head_stride = plain->hs;
  } else if (q_tma_ok(ctx, q_dtype, qcs, qhs, q)) {
    if (int rc = make_cache_map(ctx, &tm_q, const_cast<void*>(q), n_cols, (uint32_t)qcs, ctx->cfg.head_dim, 128)) return rc;
    p.q_tma = 1;
  }
  // ... and f16 output tiles leave by TMA (any head_dim the kernel takes; gate, if any, f16 with 16-byte aligned rows)
  CUtensorMap tm_o = tm_k;
  if (ctx->cfg.act_dtype == PA_F16 && !(ocs & 63) && !ctx->tune.no_out_tma && (!gate || (!(gcs & 7) && !(ghs & 7) && !((uintptr_t)gate & 15)))) {
    if (int rc = make_cache_map(ctx, &tm_o, out, n_cols, (uint32_t)ocs, ctx->cfg.head_dim, 128)) return rc;
    p.out_tma = 1;
  }
  timing_mark(ctx, st, 0);
  CU_TRY(ctx, launch_prefill(L, p, tm_k, tm_v, tm_q, tm_o, tm_q2, st));
  timing_mark(ctx, st, 1);
  ctx->stats.kernel_launches++; ctx->stats.calls++;
  ctx->stats.kv_bytes_streamed += 2ull * (pos + n_cols) * ctx->kv_dim * 2;
  ctx->inflight_layer = nullptr;   // the prefill kernel waits for its RoPE/append kernel before it lets anything follow
  return PA_OK;
}

extern "C" int pa_prefill(pa_layer* L, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* q, int q_dtype, uint64_t q_col_stride,
                          uint64_t q_head_stride, const void* gate, uint64_t gate_col_stride, uint64_t gate_head_stride, void* out, uint64_t out_col_stride,
                          void* stream) {
  if (!L) return PA_EINVAL;
  GUARD(L->ctx);
  return prefill_impl(L, seq, pos, n_cols, q, q_dtype, q_col_stride, q_head_stride, gate, gate_col_stride, gate_head_stride, out, out_col_stride,
                      (cudaStream_t)stream);
}

extern "C" int pa_head_norm(pa_ctx* ctx, const void* x, uint64_t col_stride, uint64_t head_stride, uint32_t n_heads_x, uint32_t n_cols, const float* w,
                            double eps, void* y, uint64_t y_col_stride, uint64_t y_head_stride, void* stream) {
  GUARD(ctx);
  if (!x || !y || !w) return fail(ctx, PA_EINVAL, "pa_head_norm: null x, y or w");
  if (n_cols == 0 || n_heads_x == 0) return PA_OK;
  if (n_heads_x > 65535) return fail(ctx, PA_EINVAL, "pa_head_norm: at most 65535 heads per call");
  if (ctx->cfg.head_dim > 512) return fail(ctx, PA_EUNSUPPORTED, "pa_head_norm: head_dim above 512");
  if (!(eps >= 0.0)) return fail(ctx, PA_EINVAL, "pa_head_norm: eps must be a non-negative number");
  cudaSetDevice(ctx->device);
  HeadNormParams p{};
  p.x = x; p.x_col_stride = col_stride; p.x_head_stride = head_stride; p.y = y; p.y_col_stride = y_col_stride; p.y_head_stride = y_head_stride;
  p.w = w; p.eps = eps; p.hd = ctx->cfg.head_dim; p.f16 = ctx->cfg.act_dtype == PA_F16; p.n_first = n_heads_x;
  CU_TRY(ctx, launch_head_norm(p, n_cols, n_heads_x, (cudaStream_t)stream));
  ctx->stats.kernel_launches++;
  return PA_OK;
}

extern "C" int pa_sigmoid_mul(pa_ctx* ctx, void* a, uint64_t a_col_stride, const void* g, uint64_t g_col_stride, uint64_t g_head_stride, uint32_t n_cols,
                              void* stream) {
  GUARD(ctx);
  if (!a || !g || n_cols < 1) return fail(ctx, PA_EINVAL, "pa_sigmoid_mul: null or empty argument");
  cudaSetDevice(ctx->device);
  SigmoidParams p{};
  p.a = a; p.a_col_stride = a_col_stride; p.g = g; p.g_col_stride = g_col_stride; p.g_head_stride = g_head_stride;
  p.n_heads = ctx->cfg.n_heads; p.hd = ctx->cfg.head_dim; p.f16 = ctx->cfg.act_dtype == PA_F16;
  CU_TRY(ctx, launch_sigmoid_mul(p, n_cols, (cudaStream_t)stream));
  ctx->stats.kernel_launches++;
  return PA_OK;
}

// ------------------------------------------------------------------------------ one call --

// One token of a model with head_dim 256 and 64 rotary dims, or head_dim 128 rotated in full (at most 8 heads per kv
// head): the rotation of q and k and the append ride inside the decode kernel (attn_glue_kv folded into attn_dec, in
// the reference's terms).
static bool can_fuse_front(const pa_ctx* ctx, uint32_t n_cols, const void* q, uint64_t qcs, uint64_t qhs, const void* k, const void* v) {
  const uint32_t nr = ctx->cfg.n_rot, hd = ctx->cfg.head_dim;
  return !ctx->core_only && n_cols == 1 && ctx->cfg.rope_mode == PA_ROPE_F64 && ((hd == 256 && nr == 64) || (hd == 128 && nr == 128)) && ctx->G <= 8 &&
         !(qcs & 1) && !(qhs & 1) && !((uintptr_t)q & 7) && !((uintptr_t)k & 7) && !((uintptr_t)v & 7) && !ctx->tune.no_fuse;
}

static int layer_impl(pa_layer* L, uint32_t seq, uint32_t pos, uint32_t n_cols, int mode, const void* q, uint64_t qcs, uint64_t qhs, const void* k,
                      const void* v, uint64_t kvcs, const void* gate, uint64_t gcs, uint64_t ghs, const float* cs_table, void* out, uint64_t ocs,
                      cudaStream_t st, bool sharded = false) {
  pa_ctx* ctx = L->ctx;
  if (!q || !k || !v || !out) return fail(ctx, PA_EINVAL, "pa_attn_layer: null q, k, v or out");
  if (int rc = check_cols(L, seq, pos, n_cols, "pa_attn_layer", !sharded)) return rc;
  cudaSetDevice(ctx->device);
  // QK head-norm of the layer, if it has one: q and k in one launch into the context's scratch, which the rest of the
  // call then reads (head_norm precedes RoPE in attn_glue, engine/wgsl/qwen35.js:1112-1131).  The gate keeps pointing
  // into the caller's q_full.
  uint64_t kcs = kvcs;   // k's column stride (v keeps the caller's)
  if (L->qnorm_w && !ctx->core_only) {
    if (n_cols > ctx->cfg.max_cols) return fail(ctx, PA_EINVAL, "pa_attn_layer: %u columns exceed max_cols %u", n_cols, ctx->cfg.max_cols);
    HeadNormParams hp{};
    hp.x = q; hp.x_col_stride = qcs; hp.x_head_stride = qhs; hp.y = ctx->norm_q; hp.y_col_stride = ctx->q_dim; hp.y_head_stride = ctx->cfg.head_dim;
    hp.w = L->qnorm_w; hp.n_first = ctx->cfg.n_heads;
    hp.x2 = k; hp.x2_col_stride = kvcs; hp.x2_head_stride = ctx->cfg.head_dim; hp.y2 = ctx->norm_k; hp.y2_col_stride = ctx->kv_dim;
    hp.y2_head_stride = ctx->cfg.head_dim; hp.w2 = L->knorm_w;
    hp.eps = L->norm_eps; hp.hd = ctx->cfg.head_dim; hp.f16 = ctx->cfg.act_dtype == PA_F16;
    CU_TRY(ctx, launch_head_norm(hp, n_cols, ctx->cfg.n_heads + ctx->cfg.n_kv_heads, st));
    ctx->stats.kernel_launches++;
    q = ctx->norm_q; qcs = ctx->q_dim; qhs = ctx->cfg.head_dim;
    k = ctx->norm_k; kcs = ctx->kv_dim;
  }
  // A k-token block on the tensor-core split-K kernel in its hi/lo form takes q as two f16 planes (high and low parts),
  // which the RoPE kernel writes directly: nothing is left to convert in the attention kernel's prologue.
  const bool planes = mode != PA_MODE_PREFILL && n_cols * ctx->G > 8 && n_cols * ctx->G <= (uint32_t)kMaxRows && !(ctx->cfg.flags & PA_FLAG_FAST) &&
                      !ctx->tune.verify_mma_sync && ctx->cfg.head_dim >= 128;
  if (L->kv_format != PA_KV_F16) {
    if (sharded) return fail(ctx, PA_EUNSUPPORTED, "pa_attn_layer_sharded: the peer exchange is for f16 caches");
    if (n_cols > ctx->cfg.max_cols) return fail(ctx, PA_EINVAL, "pa_attn_layer: %u columns exceed max_cols %u", n_cols, ctx->cfg.max_cols);
    if (!ctx->core_only)
      if (int rc = rope_append_impl(L, ctx, seq, pos, n_cols, q, qcs, qhs, ctx->cfg.n_heads, ctx->q_rot, ctx->q_dim, k, v, kcs, cs_table, ctx->cfg.rope_mode,
                                    ctx->cfg.act_dtype == PA_F16, st, 0, true, kvcs))
        return rc;
    pa_item it{seq, pos, n_cols, 0};
    return decode_any_impl(L, &it, 1, ctx->q_rot, PA_F32, ctx->q_dim, ctx->cfg.head_dim, gate, gcs, ghs, out, ocs, st, "pa_attn_layer");
  }
  if (sharded) {
    // this rank appends only if the new rows fall into its shard; every rank rotates q and decodes what it holds
    const bool owns = pos >= L->origin && (uint64_t)pos + n_cols <= (uint64_t)L->origin + L->max_seq;
    if (can_fuse_front(ctx, n_cols, q, qcs, qhs, k, v)) {
      FusedFront fz{k, v, owns ? 1u : 0u, pos};
      pa_item it{seq, pos, 1, 0};
      return decode_impl(L, &it, 1, q, (int)ctx->cfg.act_dtype, qcs, qhs, gate, gcs, ghs, out, ocs, nullptr, st, "pa_attn_layer_sharded", true, true, &fz);
    }
    // columns [c_lo, c_hi) of the block fall into this shard; a block may straddle a shard boundary, in which case
    // each rank appends its own columns (q is rotated for all of them everywhere)
    const uint64_t s_lo = L->origin, s_hi = (uint64_t)L->origin + L->max_seq;
    const uint32_t c_lo = pos >= s_lo ? 0u : (uint32_t)std::min<uint64_t>(s_lo - pos, n_cols);
    const uint32_t c_hi = (uint64_t)pos + n_cols <= s_hi ? n_cols : (pos >= s_hi ? 0u : (uint32_t)(s_hi - pos));
    const bool some = c_lo < c_hi, straddles = some && !owns;
    if (!ctx->core_only)
      if (int rc = rope_append_impl(owns ? L : nullptr, ctx, seq, pos, n_cols, q, qcs, qhs, ctx->cfg.n_heads, ctx->q_rot, ctx->q_dim, owns ? k : nullptr,
                                    owns ? v : nullptr, kcs, cs_table, ctx->cfg.rope_mode, ctx->cfg.act_dtype == PA_F16, st, planes ? 2 : 0, true, kvcs))
        return rc;
    if (straddles && !ctx->core_only) {
      const size_t es = ctx->cfg.act_dtype == PA_F16 ? 2 : 4;
      const uint8_t* k2 = reinterpret_cast<const uint8_t*>(k) + (size_t)c_lo * kcs * es;
      const uint8_t* v2 = reinterpret_cast<const uint8_t*>(v) + (size_t)c_lo * kvcs * es;
      const float* t2 = cs_table ? cs_table + (size_t)c_lo * ctx->cfg.n_rot : nullptr;
      if (int rc = rope_append_impl(L, ctx, seq, pos + c_lo, c_hi - c_lo, nullptr, 0, 0, 0, nullptr, 0, k2, v2, kcs, t2, ctx->cfg.rope_mode,
                                    ctx->cfg.act_dtype == PA_F16, st, 0, true, kvcs))
        return rc;
    }
    pa_item it{seq, pos, n_cols, 0};
    if (planes)
      return decode_impl(L, &it, 1, ctx->q_rot, PA_F16, ctx->q_dim, ctx->cfg.head_dim, gate, gcs, ghs, out, ocs, nullptr, st, "pa_attn_layer_sharded", true, true,
                         nullptr, reinterpret_cast<const __half*>(ctx->q_rot) + (size_t)ctx->cfg.max_cols * ctx->q_dim);
    return decode_impl(L, &it, 1, ctx->q_rot, PA_F32, ctx->q_dim, ctx->cfg.head_dim, gate, gcs, ghs, out, ocs, nullptr, st, "pa_attn_layer_sharded", true, true);
  }
  // the decode / verify kernel carries at most 64 query rows per kv head; wider passes are prefill chunks
  // (the reference takes the tiled kernel on full-width non-verify passes, engine/qwen35.js:2489)
  const bool prefill = mode == PA_MODE_PREFILL || (mode == PA_MODE_AUTO && n_cols * ctx->G > (uint32_t)kMaxRows);
  if (!prefill && can_fuse_front(ctx, n_cols, q, qcs, qhs, k, v)) {
    FusedFront fz{k, v, 1u, pos};
    pa_item it{seq, pos, 1, 0};
    return decode_impl(L, &it, 1, q, (int)ctx->cfg.act_dtype, qcs, qhs, gate, gcs, ghs, out, ocs, nullptr, st, "pa_attn_layer", true, false, &fz);
  }
  // the prefill kernel feeds q to the tensor cores as f16, so its rotated q is stored as f16 (half the traffic); and
  // where that kernel fetches its query rows by TMA, the dims no rotation touches (192 of 256 in the hybrid models)
  // are not copied at all: the kernel takes those chunks from the caller's q and only the rotated chunk from q_rot
  const uint32_t rot = ctx->cfg.n_rot;
  bool rot_only = prefill && !ctx->core_only && ctx->cfg.act_dtype == PA_F16 && ctx->cfg.rope_mode == PA_ROPE_F64 && rot >= 64 && rot % 64 == 0 &&
                  rot < ctx->cfg.head_dim && q_tma_ok(ctx, PA_F16, qcs, qhs, q) && q_tma_ok(ctx, PA_F16, ctx->q_dim, ctx->cfg.head_dim, ctx->q_rot);
  if (!ctx->core_only)
    if (int rc = rope_append_impl(L, ctx, seq, pos, n_cols, q, qcs, qhs, ctx->cfg.n_heads, ctx->q_rot, ctx->q_dim, k, v, kcs, cs_table, ctx->cfg.rope_mode,
                                  ctx->cfg.act_dtype == PA_F16, st, prefill ? 1 : (planes ? 2 : 0), true, kvcs, &rot_only))
      return rc;
  if (prefill) {
    const PlainQ plain{q, qcs, qhs};
    return prefill_impl(L, seq, pos, n_cols, ctx->q_rot, PA_F16, ctx->q_dim, ctx->cfg.head_dim, gate, gcs, ghs, out, ocs, st, rot_only ? &plain : nullptr);
  }
  pa_item it{seq, pos, n_cols, 0};
  if (planes)
    return decode_impl(L, &it, 1, ctx->q_rot, PA_F16, ctx->q_dim, ctx->cfg.head_dim, gate, gcs, ghs, out, ocs, nullptr, st, "pa_attn_layer", true, false, nullptr,
                       reinterpret_cast<const __half*>(ctx->q_rot) + (size_t)ctx->cfg.max_cols * ctx->q_dim);
  return decode_impl(L, &it, 1, ctx->q_rot, PA_F32, ctx->q_dim, ctx->cfg.head_dim, gate, gcs, ghs, out, ocs, nullptr, st, "pa_attn_layer", true);
}

extern "C" int pa_attn_layer(pa_layer* L, uint32_t seq, uint32_t pos, uint32_t n_cols, int mode, const void* q, uint64_t q_col_stride,
                             uint64_t q_head_stride, const void* k, const void* v, uint64_t kv_col_stride, const void* gate, uint64_t gate_col_stride,
                             uint64_t gate_head_stride, const float* cs_table, void* out, uint64_t out_col_stride, void* stream) {
  if (!L) return PA_EINVAL;
  GUARD(L->ctx);
  return layer_impl(L, seq, pos, n_cols, mode, q, q_col_stride, q_head_stride, k, v, kv_col_stride, gate, gate_col_stride, gate_head_stride, cs_table, out,
                    out_col_stride, (cudaStream_t)stream);
}

extern "C" int pa_attn_layer_host(pa_layer* L, uint32_t seq, uint32_t pos, uint32_t n_cols, int mode, const void* q, uint64_t qcs, uint64_t qhs,
                                  const void* k, const void* v, uint64_t kvcs, const void* gate, uint64_t gcs, uint64_t ghs, const float* cs_table,
                                  void* out, uint64_t ocs, void* stream) {
  if (!L) return PA_EINVAL;
  pa_ctx* ctx = L->ctx;
  GUARD(ctx);
  if (!q || !k || !v || !out) return fail(ctx, PA_EINVAL, "pa_attn_layer_host: null q, k, v or out");
  if (int rc = check_cols(L, seq, pos, n_cols, "pa_attn_layer_host")) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  cudaSetDevice(ctx->device);
  const size_t es = ctx->cfg.act_dtype == PA_F16 ? 2 : 4;
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  // bytes of each host array as the strides describe it (last column only up to its last element)
  const size_t q_last = (size_t)(ctx->cfg.n_heads - 1) * qhs + ctx->cfg.head_dim;
  const size_t qb = up(((size_t)(n_cols - 1) * qcs + q_last) * es), kb = up(((size_t)(n_cols - 1) * kvcs + ctx->kv_dim) * es);
  const size_t g_last = (size_t)(ctx->cfg.n_heads - 1) * ghs + ctx->cfg.head_dim;
  const size_t gb = gate ? up(((size_t)(n_cols - 1) * gcs + g_last) * es) : 0;
  const size_t ob = up(((size_t)(n_cols - 1) * ocs + ctx->q_dim) * es);
  const size_t tb = cs_table ? up((size_t)n_cols * ctx->cfg.n_rot * 4) : 0;
  // a gate that lives inside the q buffer (interleaved q_full) is not copied twice
  const uint8_t* qh = (const uint8_t*)q; const uint8_t* gh = (const uint8_t*)gate;
  const bool gate_in_q = gate && gh >= qh && gh < qh + qb;
  const size_t need = qb + 2 * kb + (gate_in_q ? 0 : gb) + ob + tb;
  if (need > ctx->stage_bytes) {
    CU_TRY(ctx, cudaStreamSynchronize(st));
    cudaFree(ctx->stage_dev); ctx->stage_dev = nullptr; ctx->stage_bytes = 0;
    if (cudaMalloc(&ctx->stage_dev, need) != cudaSuccess) { cudaGetLastError(); return fail(ctx, PA_ENOMEM, "pa_attn_layer_host: %zu staging bytes do not fit on the device", need); }
    ctx->stage_bytes = need;
  }
  uint8_t* d = (uint8_t*)ctx->stage_dev;
  uint8_t *dq = d, *dk = dq + qb, *dv = dk + kb, *dg = dv + kb, *dout = dg + (gate_in_q ? 0 : gb), *dt = dout + ob;
  CU_TRY(ctx, cudaMemcpyAsync(dq, q, ((size_t)(n_cols - 1) * qcs + q_last) * es, cudaMemcpyHostToDevice, st));
  CU_TRY(ctx, cudaMemcpyAsync(dk, k, ((size_t)(n_cols - 1) * kvcs + ctx->kv_dim) * es, cudaMemcpyHostToDevice, st));
  CU_TRY(ctx, cudaMemcpyAsync(dv, v, ((size_t)(n_cols - 1) * kvcs + ctx->kv_dim) * es, cudaMemcpyHostToDevice, st));
  const void* dgate = nullptr;
  if (gate_in_q) dgate = dq + (gh - qh);
  else if (gate) { CU_TRY(ctx, cudaMemcpyAsync(dg, gate, ((size_t)(n_cols - 1) * gcs + g_last) * es, cudaMemcpyHostToDevice, st)); dgate = dg; }
  if (cs_table) CU_TRY(ctx, cudaMemcpyAsync(dt, cs_table, (size_t)n_cols * ctx->cfg.n_rot * 4, cudaMemcpyHostToDevice, st));
  if (int rc = layer_impl(L, seq, pos, n_cols, mode, dq, qcs, qhs, dk, dv, kvcs, dgate, gcs, ghs, cs_table ? (const float*)dt : nullptr, dout, ocs, st)) return rc;
  if (ocs == ctx->q_dim) {
    CU_TRY(ctx, cudaMemcpyAsync(out, dout, (size_t)n_cols * ctx->q_dim * es, cudaMemcpyDeviceToHost, st));
  } else {
    CU_TRY(ctx, cudaMemcpy2DAsync(out, ocs * es, dout, ocs * es, ctx->q_dim * es, n_cols, cudaMemcpyDeviceToHost, st));
  }
  return pa_sync(ctx, stream);
}

// One token step over several layers with HOST buffers: one upload per array, the layers back to back, one download.
extern "C" int pa_attn_step_host(pa_layer* const* layers, uint32_t n_layers, uint32_t seq, uint32_t pos, uint32_t n_cols, int mode, const void* q,
                                 uint64_t q_layer_stride, uint64_t qcs, uint64_t qhs, const void* k, const void* v, uint64_t kv_layer_stride, uint64_t kvcs,
                                 const void* gate, uint64_t gate_layer_stride, uint64_t gcs, uint64_t ghs, void* out, uint64_t out_layer_stride, uint64_t ocs,
                                 void* stream) {
  if (!layers || n_layers < 1 || !layers[0]) return PA_EINVAL;
  pa_ctx* ctx = layers[0]->ctx;
  GUARD(ctx);
  if (!q || !k || !v || !out) return fail(ctx, PA_EINVAL, "pa_attn_step_host: null q, k, v or out");
  for (uint32_t l = 0; l < n_layers; ++l) {
    if (!layers[l] || layers[l]->ctx != ctx) return fail(ctx, PA_EINVAL, "pa_attn_step_host: layer %u belongs to another context", l);
    if (int rc = check_cols(layers[l], seq, pos, n_cols, "pa_attn_step_host")) return rc;
  }
  cudaStream_t st = (cudaStream_t)stream;
  cudaSetDevice(ctx->device);
  const size_t es = ctx->cfg.act_dtype == PA_F16 ? 2 : 4;
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  const size_t qb = up((size_t)n_layers * q_layer_stride * es), kb = up((size_t)n_layers * kv_layer_stride * es);
  const size_t gb = gate ? up((size_t)n_layers * gate_layer_stride * es) : 0, ob = up((size_t)n_layers * out_layer_stride * es);
  const uint8_t* qh = (const uint8_t*)q; const uint8_t* gh = (const uint8_t*)gate;
  const bool gate_in_q = gate && gh >= qh && gh < qh + qb;     // interleaved q_full: the gate rides in the q upload
  const size_t need = qb + 2 * kb + (gate_in_q ? 0 : gb) + ob;
  if (need > ctx->stage_bytes) {
    CU_TRY(ctx, cudaStreamSynchronize(st));
    cudaFree(ctx->stage_dev); ctx->stage_dev = nullptr; ctx->stage_bytes = 0;
    if (cudaMalloc(&ctx->stage_dev, need) != cudaSuccess) { cudaGetLastError(); return fail(ctx, PA_ENOMEM, "pa_attn_step_host: %zu staging bytes do not fit on the device", need); }
    ctx->stage_bytes = need;
  }
  uint8_t* d = (uint8_t*)ctx->stage_dev;
  uint8_t *dq = d, *dk = dq + qb, *dv = dk + kb, *dg = dv + kb, *dout = dg + (gate_in_q ? 0 : gb);
  CU_TRY(ctx, cudaMemcpyAsync(dq, q, (size_t)n_layers * q_layer_stride * es, cudaMemcpyHostToDevice, st));
  CU_TRY(ctx, cudaMemcpyAsync(dk, k, (size_t)n_layers * kv_layer_stride * es, cudaMemcpyHostToDevice, st));
  CU_TRY(ctx, cudaMemcpyAsync(dv, v, (size_t)n_layers * kv_layer_stride * es, cudaMemcpyHostToDevice, st));
  const uint8_t* dgate = nullptr;
  if (gate_in_q) dgate = dq + (gh - qh);
  else if (gate) { CU_TRY(ctx, cudaMemcpyAsync(dg, gate, (size_t)n_layers * gate_layer_stride * es, cudaMemcpyHostToDevice, st)); dgate = dg; }
  ctx->scope_active = true; ctx->scope_fresh = false;   // all layers of this call may share one cos / sin table
  for (uint32_t l = 0; l < n_layers; ++l) {
    if (int rc = layer_impl(layers[l], seq, pos, n_cols, mode, dq + l * q_layer_stride * es, qcs, qhs, dk + l * kv_layer_stride * es,
                            dv + l * kv_layer_stride * es, kvcs, dgate ? dgate + l * gate_layer_stride * es : nullptr, gcs, ghs, nullptr,
                            dout + l * out_layer_stride * es, ocs, st)) {
      ctx->scope_active = false;
      return rc;
    }
  }
  ctx->scope_active = false;
  CU_TRY(ctx, cudaMemcpyAsync(out, dout, (size_t)n_layers * out_layer_stride * es, cudaMemcpyDeviceToHost, st));
  return pa_sync(ctx, stream);
}


// ------------------------------------------------------------------------------ cache export / import, slots --

// rows of [pos0, pos1) this layer's shard holds: first global position and count
static uint32_t shard_span(const pa_layer* L, uint32_t pos0, uint32_t pos1, uint32_t* first) {
  const uint64_t lo = std::max<uint64_t>(pos0, L->origin), hi = std::min<uint64_t>(pos1, (uint64_t)L->origin + L->max_seq);
  *first = (uint32_t)lo;
  return hi > lo ? (uint32_t)(hi - lo) : 0u;
}
static int cache_copy(pa_layer* L, uint32_t seq, uint32_t pos0, uint32_t pos1, int which, void* host, bool to_host, uint32_t* rows_out, void* stream,
                      const char* who) {
  if (!L) return PA_EINVAL;
  pa_ctx* ctx = L->ctx;
  GUARD(ctx);
  if (rows_out) *rows_out = 0;
  const bool scales = which == 2 || which == 3;
  if (!host || which < 0 || which > 3 || (scales && L->kv_format != PA_KV_Q8))
    return fail(ctx, PA_EINVAL, "%s: null host buffer, or `which` is not 0 (K), 1 (V) or, on an int8 layer, 2 / 3 (their scales)", who);
  if (seq >= L->n_seqs || pos1 < pos0) return fail(ctx, PA_EINVAL, "%s: sequence %u of %u, positions [%u, %u)", who, seq, L->n_seqs, pos0, pos1);
  uint32_t first;
  const uint32_t n = shard_span(L, pos0, pos1, &first);
  if (rows_out) *rows_out = n;
  if (!n) return PA_OK;
  cudaSetDevice(ctx->device);
  const size_t row_bytes = scales ? scale_row_bytes_of(ctx, L->kv_format) : row_bytes_of(ctx, L->kv_format);
  uint8_t* dev = reinterpret_cast<uint8_t*>(pa_cache_ptr(L, which)) + ((size_t)seq * L->max_seq + (first - L->origin)) * row_bytes;
  uint8_t* h = reinterpret_cast<uint8_t*>(host) + (size_t)(first - pos0) * row_bytes;
  if (to_host) CU_TRY(ctx, cudaMemcpyAsync(h, dev, (size_t)n * row_bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  else {
    CU_TRY(ctx, cudaMemcpyAsync(dev, h, (size_t)n * row_bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    ctx->inflight_layer = nullptr;   // a copy is ordered by the stream like any kernel, but it is no PDL predecessor:
  }                                  // nothing of the next call may start ahead of it (see decode_impl)
  return PA_OK;
}
extern "C" int pa_cache_export(pa_layer* L, uint32_t seq, uint32_t pos0, uint32_t pos1, int which, void* host_dst, uint32_t* rows_copied, void* stream) {
  return cache_copy(L, seq, pos0, pos1, which, host_dst, true, rows_copied, stream, "pa_cache_export");
}
extern "C" int pa_cache_import(pa_layer* L, uint32_t seq, uint32_t pos0, uint32_t pos1, int which, const void* host_src, uint32_t* rows_copied,
                               void* stream) {
  return cache_copy(L, seq, pos0, pos1, which, const_cast<void*>(host_src), false, rows_copied, stream, "pa_cache_import");
}

struct pa_slot {
  pa_ctx* ctx = nullptr;
  uint32_t pos = 0, first = 0, rows = 0;   // positions [0, pos) were saved; this shard held `rows` of them from `first`
  size_t row_bytes = 0;
  uint8_t* k = nullptr;
  uint8_t* v = nullptr;
};
extern "C" int pa_slot_save(pa_layer* L, uint32_t seq, uint32_t pos, pa_slot** out, void* stream) {
  if (!L || !out) return PA_EINVAL;
  pa_ctx* ctx = L->ctx;
  GUARD(ctx);
  *out = nullptr;
  if (L->kv_format != PA_KV_F16) return fail(ctx, PA_EUNSUPPORTED, "pa_slot_save: slots are for f16 caches (use pa_cache_export / pa_cache_import)");
  if (seq >= L->n_seqs) return fail(ctx, PA_EINVAL, "pa_slot_save: sequence %u of %u", seq, L->n_seqs);
  pa_slot* s = new (std::nothrow) pa_slot();
  if (!s) return fail(ctx, PA_ENOMEM, "pa_slot_save: out of host memory");
  s->ctx = ctx; s->pos = pos; s->row_bytes = (size_t)ctx->kv_dim * 2;
  s->rows = shard_span(L, 0, pos, &s->first);
  cudaSetDevice(ctx->device);
  if (s->rows) {
    const size_t bytes = (size_t)s->rows * s->row_bytes;
    if (cudaMalloc(&s->k, bytes) != cudaSuccess || cudaMalloc(&s->v, bytes) != cudaSuccess) {
      cudaGetLastError(); cudaFree(s->k); delete s;
      return fail(ctx, PA_ENOMEM, "pa_slot_save: two copies of %u rows (%.0f MiB each) do not fit on the device", pos, bytes / 1048576.0);
    }
    const size_t off = ((size_t)seq * L->max_seq + (s->first - L->origin)) * s->row_bytes;
    CU_TRY(ctx, cudaMemcpyAsync(s->k, reinterpret_cast<uint8_t*>(L->k) + off, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    CU_TRY(ctx, cudaMemcpyAsync(s->v, reinterpret_cast<uint8_t*>(L->v) + off, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  }
  *out = s;
  return PA_OK;
}
extern "C" int pa_slot_load(pa_layer* L, uint32_t seq, const pa_slot* s, uint32_t* pos_out, void* stream) {
  if (!L || !s) return PA_EINVAL;
  pa_ctx* ctx = L->ctx;
  GUARD(ctx);
  if (s->ctx != ctx || s->row_bytes != (size_t)ctx->kv_dim * 2 || L->kv_format != PA_KV_F16)
    return fail(ctx, PA_EINVAL, "pa_slot_load: the slot was saved from another context or cache format");
  if (seq >= L->n_seqs) return fail(ctx, PA_EINVAL, "pa_slot_load: sequence %u of %u", seq, L->n_seqs);
  uint32_t first;
  const uint32_t rows = shard_span(L, 0, s->pos, &first);
  if (rows != s->rows || (rows && first != s->first)) return fail(ctx, PA_EINVAL, "pa_slot_load: the slot holds rows %u..%u, this layer's shard would hold %u..%u",
                                                                  s->first, s->first + s->rows, first, first + rows);
  cudaSetDevice(ctx->device);
  if (rows) {
    const size_t bytes = (size_t)rows * s->row_bytes, off = ((size_t)seq * L->max_seq + (first - L->origin)) * s->row_bytes;
    CU_TRY(ctx, cudaMemcpyAsync(reinterpret_cast<uint8_t*>(L->k) + off, s->k, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    CU_TRY(ctx, cudaMemcpyAsync(reinterpret_cast<uint8_t*>(L->v) + off, s->v, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    ctx->inflight_layer = nullptr;
  }
  if (pos_out) *pos_out = s->pos;
  return PA_OK;
}
extern "C" int pa_slot_export(const pa_slot* s, int which, void* host_dst, void* stream) {
  if (!s || !host_dst || (which != 0 && which != 1)) return PA_EINVAL;
  pa_ctx* ctx = s->ctx;
  cudaSetDevice(ctx->device);
  if (s->rows) CU_TRY(ctx, cudaMemcpyAsync(host_dst, which ? s->v : s->k, (size_t)s->rows * s->row_bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return PA_OK;
}
extern "C" int pa_slot_info(const pa_slot* s, uint32_t* pos, uint32_t* first_row, uint32_t* rows) {
  if (!s) return PA_EINVAL;
  if (pos) *pos = s->pos;
  if (first_row) *first_row = s->first;
  if (rows) *rows = s->rows;
  return PA_OK;
}
extern "C" int pa_slot_drop(pa_slot* s) {
  if (!s) return PA_OK;
  cudaSetDevice(s->ctx->device);
  cudaFree(s->k); cudaFree(s->v);
  delete s;
  return PA_OK;
}

// ------------------------------------------------------------------------------ peer exchange --

extern "C" size_t pa_exchange_bytes(pa_ctx* ctx, uint32_t world, uint32_t max_rows) {
  if (!ctx || world < 1 || world > 8 || max_rows < 1) return 0;
  const size_t n_slices = ctx->cfg.head_dim / 64;
  const size_t blk = (size_t)max_rows * (ctx->cfg.head_dim + 2 * n_slices) * 8;   // {value, tag} entries: o rows + (m, l) per (row, slice)
  return 2 * (size_t)world * blk;                                                  // two parities x world source ranks
}

extern "C" int pa_shared_alloc(pa_ctx* ctx, size_t bytes, void** dev_ptr, void* ipc_handle_out) {
  if (!ctx || !dev_ptr || !ipc_handle_out || !bytes) return PA_EINVAL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "ipc handle size");
  cudaSetDevice(ctx->device);
  if (cudaMalloc(dev_ptr, bytes) != cudaSuccess) { cudaGetLastError(); return fail(ctx, PA_ENOMEM, "pa_shared_alloc: %zu bytes do not fit on the device", bytes); }
  CU_TRY(ctx, cudaMemset(*dev_ptr, 0, bytes));
  CU_TRY(ctx, cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(ipc_handle_out), *dev_ptr));
  return PA_OK;
}
extern "C" int pa_shared_open(pa_ctx* ctx, const void* ipc_handle, void** dev_ptr) {
  if (!ctx || !ipc_handle || !dev_ptr) return PA_EINVAL;
  cudaSetDevice(ctx->device);
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof h);
  cudaError_t e = cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { cudaGetLastError(); return fail(ctx, PA_ECUDA, "pa_shared_open: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e)); }
  return PA_OK;
}
extern "C" int pa_shared_close(pa_ctx* ctx, void* dev_ptr) {
  if (!ctx) return PA_EINVAL;
  cudaSetDevice(ctx->device);
  cudaIpcCloseMemHandle(dev_ptr);
  return PA_OK;
}
extern "C" int pa_exchange_init(pa_ctx* ctx, uint32_t rank, uint32_t world, void* const* bufs, uint32_t max_rows) {
  if (!ctx || !bufs || world < 1 || world > 8 || rank >= world || max_rows < 1) return fail(ctx, PA_EINVAL, "pa_exchange_init: bad rank / world (1..8) / buffers");
  cudaSetDevice(ctx->device);
  ExchangeView x{};
  for (uint32_t r = 0; r < world; ++r) { if (!bufs[r]) return fail(ctx, PA_EINVAL, "pa_exchange_init: null buffer of rank %u", r); x.peer[r] = (float*)bufs[r]; }
  x.world = world; x.rank = rank; x.max_rows = max_rows; x.hd = ctx->cfg.head_dim;
  if (!ctx->xc.ctr) {
    if (cudaMalloc(&x.ctr, 8) != cudaSuccess) { cudaGetLastError(); return fail(ctx, PA_ENOMEM, "pa_exchange_init: out of device memory"); }
  } else x.ctr = ctx->xc.ctr;
  // A fresh session: call counter 0 and no entry in this rank's buffer that could carry a tag of the new session (the
  // buffer may have served an earlier one).  The peers write into it only after the barrier that follows set-up.
  CU_TRY(ctx, cudaDeviceSynchronize());
  CU_TRY(ctx, cudaMemset(x.ctr, 0, 8));
  CU_TRY(ctx, cudaMemset(bufs[rank], 0, pa_exchange_bytes(ctx, world, max_rows)));
  CU_TRY(ctx, cudaDeviceSynchronize());
  ctx->xc = x;
  return PA_OK;
}
extern "C" int pa_set_wait_limit(pa_ctx* ctx, uint32_t sweeps) {
  if (!ctx) return PA_EINVAL;
  ctx->tune.wait_polls = sweeps;
  return PA_OK;
}
extern "C" int pa_decode_exchange(pa_layer* L, const pa_item* items, uint32_t n_items, const void* q, int q_dtype, uint64_t q_col_stride,
                                  uint64_t q_head_stride, const void* gate, uint64_t gate_col_stride, uint64_t gate_head_stride, void* out,
                                  uint64_t out_col_stride, void* stream) {
  if (!L) return PA_EINVAL;
  GUARD(L->ctx);
  if (!out) return fail(L->ctx, PA_EINVAL, "pa_decode_exchange: null out");
  if (L->kv_format != PA_KV_F16) return fail(L->ctx, PA_EUNSUPPORTED, "pa_decode_exchange: the peer exchange is for f16 caches");
  return decode_impl(L, items, n_items, q, q_dtype, q_col_stride, q_head_stride, gate, gate_col_stride, gate_head_stride, out, out_col_stride, nullptr,
                     (cudaStream_t)stream, "pa_decode_exchange", L->ctx->inflight_layer == L, true);
}

// One token of each of several sequences through a whole layer: the fused front of the decode kernel for every item
// (each CTA rotates its item's q, the CTA on an item's last tile rotates and appends its k / v row), or the
// RoPE/append kernel for all items followed by the decode, where the fused front does not apply.
extern "C" int pa_attn_items(pa_layer* L, const pa_item* items, uint32_t n_items, const void* q, uint64_t q_col_stride, uint64_t q_head_stride,
                             const void* k, const void* v, uint64_t kv_col_stride, const void* gate, uint64_t gate_col_stride, uint64_t gate_head_stride,
                             void* out, uint64_t out_col_stride, int exchange, void* stream) {
  if (!L) return PA_EINVAL;
  pa_ctx* ctx = L->ctx;
  GUARD(ctx);
  if (!q || !k || !v || !out || !items) return fail(ctx, PA_EINVAL, "pa_attn_items: null q, k, v, out or items");
  if (n_items < 1 || n_items > (uint32_t)kMaxItems) return fail(ctx, PA_EINVAL, "pa_attn_items: 1 to %d items per call", kMaxItems);
  if (n_items > ctx->cfg.max_cols) return fail(ctx, PA_EINVAL, "pa_attn_items: %u items exceed max_cols %u", n_items, ctx->cfg.max_cols);
  if (L->kv_format != PA_KV_F16) return fail(ctx, PA_EUNSUPPORTED, "pa_attn_items: f16 caches only; use pa_attn_layer per sequence");
  if (ctx->cfg.rope_mode == PA_ROPE_TABLE) return fail(ctx, PA_EUNSUPPORTED, "pa_attn_items: PA_ROPE_TABLE takes one table per call; use pa_attn_layer per sequence");
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t mask = 0;
  for (uint32_t i = 0; i < n_items; ++i) {
    if (items[i].n_cols != 1) return fail(ctx, PA_EINVAL, "pa_attn_items: item %u has %u columns; one token per item", i, items[i].n_cols);
    if (int rc = check_cols(L, items[i].seq, items[i].pos, 1, "pa_attn_items", !exchange)) return rc;
    if (items[i].pos >= L->origin && items[i].pos - L->origin < L->max_seq) mask |= 1u << i;
  }
  cudaSetDevice(ctx->device);
  uint64_t qcs = q_col_stride, qhs = q_head_stride, kcs = kv_col_stride;
  if (L->qnorm_w && !ctx->core_only) {   // QK head-norm first, item i as column i (as pa_attn_layer does for its columns)
    HeadNormParams hp{};
    hp.x = q; hp.x_col_stride = qcs; hp.x_head_stride = qhs; hp.y = ctx->norm_q; hp.y_col_stride = ctx->q_dim; hp.y_head_stride = ctx->cfg.head_dim;
    hp.w = L->qnorm_w; hp.n_first = ctx->cfg.n_heads;
    hp.x2 = k; hp.x2_col_stride = kv_col_stride; hp.x2_head_stride = ctx->cfg.head_dim; hp.y2 = ctx->norm_k; hp.y2_col_stride = ctx->kv_dim;
    hp.y2_head_stride = ctx->cfg.head_dim; hp.w2 = L->knorm_w;
    hp.eps = L->norm_eps; hp.hd = ctx->cfg.head_dim; hp.f16 = ctx->cfg.act_dtype == PA_F16;
    CU_TRY(ctx, launch_head_norm(hp, n_items, ctx->cfg.n_heads + ctx->cfg.n_kv_heads, st));
    ctx->stats.kernel_launches++;
    q = ctx->norm_q; qcs = ctx->q_dim; qhs = ctx->cfg.head_dim;
    k = ctx->norm_k; kcs = ctx->kv_dim;
  }
  if (can_fuse_front(ctx, 1, q, qcs, qhs, k, v) && !(kcs & 1) && !(kv_col_stride & 1)) {
    // one item: cos / sin from the host's libm, as pa_attn_layer; several: each CTA evaluates its own item's
    FusedFront fz{k, v, mask, items[0].pos, kcs, kv_col_stride, n_items > 1};
    return decode_impl(L, items, n_items, q, (int)ctx->cfg.act_dtype, qcs, qhs, gate, gate_col_stride, gate_head_stride, out, out_col_stride, nullptr, st,
                       "pa_attn_items", true, exchange != 0, &fz);
  }
  if (!ctx->core_only)
    if (int rc = rope_append_items_impl(L, items, n_items, q, qcs, qhs, k, v, kcs, kv_col_stride, ctx->q_rot, st)) return rc;
  return decode_impl(L, items, n_items, ctx->q_rot, PA_F32, ctx->q_dim, ctx->cfg.head_dim, gate, gate_col_stride, gate_head_stride, out, out_col_stride, nullptr,
                     st, "pa_attn_items", true, exchange != 0);
}

extern "C" int pa_attn_layer_sharded(pa_layer* L, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* q, uint64_t q_col_stride,
                                     uint64_t q_head_stride, const void* k, const void* v, uint64_t kv_col_stride, const void* gate,
                                     uint64_t gate_col_stride, uint64_t gate_head_stride, const float* cs_table, void* out, uint64_t out_col_stride,
                                     void* stream) {
  if (!L) return PA_EINVAL;
  GUARD(L->ctx);
  return layer_impl(L, seq, pos, n_cols, PA_MODE_DECODE, q, q_col_stride, q_head_stride, k, v, kv_col_stride, gate, gate_col_stride, gate_head_stride,
                    cs_table, out, out_col_stride, (cudaStream_t)stream, true);
}
