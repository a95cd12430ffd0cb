// pa_decode_static: the split-K decode + combine for callers that must not allocate.
//
// Who this is for: code that runs where device allocation is off the table — inside a region a host framework is
// capturing, on a real-time thread that may not block on the allocator, in a process whose memory pool is owned by
// someone else, or in an embedding that was handed raw device pointers and nothing more.  Such a caller cannot
// create a pa_ctx / pa_layer (both allocate their caches and work buffers); it already owns its K/V caches, q, gate
// and out, and passes them here as plain pointers.
//
// What is different from pa_decode: the per-split partial records (o, m, l) that the decode kernel writes and the
// combine kernel reads live in a fixed array inside the library image instead of in a context's buffer.  The array
// exists once per GPU that loads the library and stays until the process exits.  Consequences a caller must know:
//   - capacity: PA_STATIC_RECORDS records.  A call uses n_cols * n_heads * splits of them; the split count is
//     lowered to fit, and a call that does not fit even unsplit is refused with PA_EUNSUPPORTED.
//   - every call on a device shares the array.  Two calls that overlap on the GPU (different streams, or different
//     threads / processes sharing the context) race on it; keep calls on one stream or order them with events.
//   - the array keeps the previous call's contents.  Records are fully rewritten before they are read, so nothing
//     needs clearing except the status word the bounded device-side waits report into; the entry point clears that
//     word on the stream before the kernels.
//   - the first call on a device looks up the array's device address (cudaGetSymbolAddress) and sets the kernel's
//     shared-memory attribute.  Make that first call outside any stream capture.
// Nothing here calls cudaMalloc, cudaFree, cudaMallocHost or any library routine that allocates.
#include <math.h>
#include <stdio.h>

#include <mutex>

#include "pa_params.cuh"

namespace pa {
cudaError_t launch_decode(const pa_layer* L, const DecodeParams& p, dim3 grid, int nt, cudaStream_t st);
cudaError_t launch_combine(int head_dim, const CombineParams& p, uint32_t rows, cudaStream_t st);
}  // namespace pa

using namespace pa;

#define PA_STATIC_RECORDS 2048   // (query row, split) records; 2048 * (256 + 2) floats + the status word = 2.1 MB per GPU

// [0]: status word of the bounded waits (padded to 64 floats); then PA_STATIC_RECORDS * 256 floats of o; then
// PA_STATIC_RECORDS * 2 floats of (m, l).  In host code this name is only a handle for cudaGetSymbolAddress: passing
// it to a kernel as if it were a pointer would hand the GPU a host address.
static __device__ __align__(256) float g_static_scratch[64 + PA_STATIC_RECORDS * 256 + PA_STATIC_RECORDS * 2];

static float* g_scratch_dev[64] = {};   // per device: the array's device address, looked up once (under g_setup_mu)
static std::mutex g_setup_mu;
static int g_smem_optin[64] = {};
static int g_sm_count[64] = {};

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int say(char* msg, size_t len, int code, const char* text) {
  if (msg && len) snprintf(msg, len, "%s", text);
  return code;
}

static int encode_map(CUtensorMap* tm, const void* base, uint64_t rows, uint32_t kv_dim, uint32_t hd) {
  static encode_tiled_fn enc = nullptr;
  if (!enc) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return -1;
    enc = reinterpret_cast<encode_tiled_fn>(f);
  }
  cuuint64_t dims[3] = {64, rows, kv_dim / 64};
  cuuint64_t strides[2] = {(cuuint64_t)kv_dim * 2, 128};
  cuuint32_t box[3] = {64, 64, hd / 64};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -1;
}

extern "C" PA_API int pa_decode_static(int device, const void* k_cache, const void* v_cache, uint32_t cache_rows, uint32_t n_heads,
                                       uint32_t n_kv_heads, uint32_t head_dim, uint32_t pos, uint32_t n_cols, const float* q, const float* gate,
                                       float* out, void* stream, char* msg, size_t msg_len) {
  if (!k_cache || !v_cache || !q || !out) return say(msg, msg_len, PA_EINVAL, "pa_decode_static: null cache, q or out");
  if (device < 0 || device >= 64) return say(msg, msg_len, PA_EINVAL, "pa_decode_static: device index outside 0..63");
  if (head_dim != 128 && head_dim != 256) return say(msg, msg_len, PA_EUNSUPPORTED, "pa_decode_static: head_dim must be 128 or 256");
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads) return say(msg, msg_len, PA_EINVAL, "pa_decode_static: n_heads must be a multiple of n_kv_heads");
  const uint32_t G = n_heads / n_kv_heads;
  if (n_cols < 1 || n_cols * G > (uint32_t)kMaxRows)
    return say(msg, msg_len, PA_EUNSUPPORTED, "pa_decode_static: n_cols * (n_heads / n_kv_heads) must be between 1 and 64");
  if ((uint64_t)pos + n_cols > cache_rows || cache_rows >= (1u << 31)) return say(msg, msg_len, PA_EINVAL, "pa_decode_static: pos + n_cols passes cache_rows");
  const int nt = (int)((n_cols * G + 7) / 8);
  const uint32_t groups = 1;   // the decode kernel leaves one record per (row, split)
  const uint32_t rows = n_cols * n_heads;
  if (rows * groups > PA_STATIC_RECORDS) {
    char b[160];
    snprintf(b, sizeof b, "pa_decode_static: %u query rows need more than the %d records of the built-in scratch array", rows, PA_STATIC_RECORDS);
    return say(msg, msg_len, PA_EUNSUPPORTED, b);
  }
  if (((uintptr_t)q & 7) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return say(msg, msg_len, PA_EINVAL, "pa_decode_static: misaligned pointer");
  if (cudaSetDevice(device) != cudaSuccess) return say(msg, msg_len, PA_ECUDA, "pa_decode_static: cudaSetDevice failed (there is no CPU path)");
  std::unique_lock<std::mutex> setup_lock(g_setup_mu);
  if (!g_scratch_dev[device]) {
    // one-time set-up for this device, with the device current: the array's address on THIS device
    float* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_static_scratch) != cudaSuccess || !ptr) {
      cudaGetLastError();
      return say(msg, msg_len, PA_ECUDA, "pa_decode_static: cudaGetSymbolAddress failed for the built-in scratch array");
    }
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) return say(msg, msg_len, PA_ECUDA, "pa_decode_static: cannot query the device");
    g_smem_optin[device] = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return say(msg, msg_len, PA_ECUDA, "pa_decode_static: cannot query the device");
    g_sm_count[device] = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess || v != 10)
      return say(msg, msg_len, PA_EUNSUPPORTED, "pa_decode_static: this library is built for sm_100a only");
    g_scratch_dev[device] = ptr;
  }
  setup_lock.unlock();
  float* scratch = g_scratch_dev[device];
  uint32_t* err = reinterpret_cast<uint32_t*>(scratch);
  float* part_o = scratch + 64;
  float* part_ml = part_o + (size_t)PA_STATIC_RECORDS * 256;
  cudaStream_t st = (cudaStream_t)stream;

  // host-side stand-ins for the handles the launchers read (plain structs on the stack; nothing is allocated)
  pa_ctx ctx;
  ctx.device = device; ctx.sm_count = g_sm_count[device]; ctx.smem_optin = g_smem_optin[device];
  ctx.cfg.n_heads = n_heads; ctx.cfg.n_kv_heads = n_kv_heads; ctx.cfg.head_dim = head_dim; ctx.cfg.flags = 0;
  ctx.G = G; ctx.q_dim = n_heads * head_dim; ctx.kv_dim = n_kv_heads * head_dim;
  pa_layer layer;
  layer.ctx = &ctx; layer.n_seqs = 1; layer.max_seq = cache_rows;
  if (encode_map(&layer.tm_k64, k_cache, cache_rows, ctx.kv_dim, head_dim) || encode_map(&layer.tm_v64, v_cache, cache_rows, ctx.kv_dim, head_dim))
    return say(msg, msg_len, PA_ECUDA, "pa_decode_static: cuTensorMapEncodeTiled failed");

  const uint32_t n_rows = pos + n_cols, tiles = (n_rows + 63) / 64;
  uint32_t ns = (uint32_t)ctx.sm_count / n_kv_heads;
  if (ns < 1) ns = 1;
  if (ns > (tiles / 2 > 1 ? tiles / 2 : 1)) ns = tiles / 2 > 1 ? tiles / 2 : 1;
  if (ns > PA_STATIC_RECORDS / (rows * groups)) ns = PA_STATIC_RECORDS / (rows * groups);   // fit the records into the fixed array
  if (ns > 256) ns = 256;

  DecodeParams p{};
  p.q = q; p.q_f16 = 0; p.q_col_stride = ctx.q_dim; p.q_head_stride = head_dim;
  p.part_o = part_o; p.part_ml = part_ml; p.n_splits = ns;
  p.n_heads = n_heads; p.G = G; p.max_seq = cache_rows;
  p.prefetch_old_rows = 0;
  p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)head_dim));
  p.err = err;
  p.items.seq[0] = 0; p.items.lim0[0] = (int32_t)pos + 1; p.items.n_rows[0] = n_rows; p.items.n_cols[0] = n_cols; p.items.col0[0] = 0;

  // the one thing that must start at zero: the status word (the records are rewritten before they are read)
  if (cudaMemsetAsync(err, 0, 4, st) != cudaSuccess) return say(msg, msg_len, PA_ECUDA, "pa_decode_static: cudaMemsetAsync failed");
  if (launch_decode(&layer, p, dim3(ns, n_kv_heads, 1), nt, st) != cudaSuccess) {
    cudaGetLastError();
    return say(msg, msg_len, PA_ECUDA, "pa_decode_static: launching the decode kernel failed");
  }
  CombineParams c{};
  c.o = part_o; c.ml = part_ml;
  c.o_row_stride = (uint64_t)ns * groups * head_dim; c.o_part_stride = head_dim; c.ml_row_stride = (uint64_t)ns * groups * 2; c.ml_part_stride = 2;
  c.n_heads = n_heads; c.fixed_parts = 0; c.n_splits = ns; c.groups = groups;
  c.gate = gate; c.gate_col_stride = ctx.q_dim; c.gate_head_stride = head_dim; c.out = out; c.out_col_stride = ctx.q_dim; c.act_f16 = 0;
  c.partial_out = nullptr; c.partial_rows = rows; c.items = p.items; c.n_items = 1;
  if (launch_combine((int)head_dim, c, rows, st) != cudaSuccess) {
    cudaGetLastError();
    return say(msg, msg_len, PA_ECUDA, "pa_decode_static: launching the combine kernel failed");
  }
  return PA_OK;
}

// The status word of the bounded device-side waits of the calls made so far on `stream` (0: every wait was satisfied).
// A 4-byte copy out of the built-in array followed by a wait for the stream: allocates nothing.
extern "C" PA_API int pa_decode_static_status(int device, void* stream, uint32_t* word) {
  if (!word || device < 0 || device >= 64) return PA_EINVAL;
  *word = 0;
  float* scratch;
  {
    std::lock_guard<std::mutex> g(g_setup_mu);
    scratch = g_scratch_dev[device];
  }
  if (!scratch) return PA_OK;   // no call has run on this device yet
  if (cudaSetDevice(device) != cudaSuccess) return PA_ECUDA;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemcpyAsync(word, scratch, 4, cudaMemcpyDeviceToHost, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) {
    cudaGetLastError();
    return PA_ECUDA;
  }
  return *word ? PA_ETIMEOUT : PA_OK;
}
