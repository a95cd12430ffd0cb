// Shared device helpers for the sm_100a attention kernels: PTX wrappers for mbarrier, TMA, ldmatrix and
// mma.sync, the bounded-wait rule, and the internal context layout.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cstdlib>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/pooled_attn.h"

namespace pa {

// Every device-side wait is bounded: after this many polls the waiter records PA_WAIT_* in the context's
// error word and carries on as if the wait had succeeded, so control flow stays uniform, every thread
// reaches the end of the kernel and the host reports PA_ETIMEOUT instead of a hung GPU.
constexpr uint32_t kWaitPolls = 1u << 24;  // with 32..64 ns back-off: well under a second

enum : uint32_t { WAIT_KFULL = 1, WAIT_VFULL = 2, WAIT_EMPTY = 3, WAIT_MMA = 4, WAIT_TMEM = 5, WAIT_QFULL = 6, WAIT_PEER = 7, WAIT_MERGE = 8 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Bounded wait.  err_smem: a shared word that any thread sets once a wait ran out; later waits return at once.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* err_smem, uint32_t code) {
  if (mbar_test(bar, parity)) return;
  for (uint32_t i = 0; i < kWaitPolls; ++i) {
    if (*err_smem) return;
    if (mbar_test(bar, parity)) return;
    if (i > 64) __nanosleep(32);
  }
  *err_smem = code;
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 3-D tiled TMA load into this CTA's shared memory, completing on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// The same with an L2 eviction policy for the lines it brings in.  A KV stream is read once per call: marking its
// lines "evict first" leaves what is re-read from L2 (instructions, q, records, the next call's early tiles) in place.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const CUtensorMap* m, int x, int y, int z, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
      : "memory");
}
// 3-D tiled TMA store from this CTA's shared memory (rows and chunks outside the tensor are not written), as a bulk
// group of the issuing thread; tma_store_wait_read returns once the group's shared-memory reads are done.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, int x, int y, int z, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(src) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, int x, int y, int z, int w, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
      : "memory");
}

// the same box, requested into L2 only (no shared-memory destination, nothing to wait for)
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* m, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
// D (16x8, f32) += A (16x16 f16, row) * B (16x8 f16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// cos / sin of one rotary angle: the float64 values and each split into an f32 pair (hi = fl32(v), lo = fl32(v - hi))
struct Angle { double c, s; float c_hi, c_lo, s_hi, s_lo; };
__host__ __device__ inline Angle make_angle(double c, double s) {
  Angle g; g.c = c; g.s = s;
  g.c_hi = (float)c; g.c_lo = (float)(c - (double)g.c_hi);
  g.s_hi = (float)s; g.s_lo = (float)(s - (double)g.s_hi);
  // a nonzero value so small that its low half would underflow in f32: poison the pair, which sends every use of
  // this angle to the float64 instructions
  const double tiny = 8.0e-28;   // ~2^-90
  if ((c != 0.0 && fabs(c) < tiny) || (s != 0.0 && fabs(s) < tiny)) g.c_hi = __builtin_nanf("");
  return g;
}

// One output of a float64 rotation, rounded to f32:  fl32( fl64( fl64(x * cos) -/+ fl64(y * sin) ) ), bit for bit,
// at f32 cost.  (Plain FP64 instructions run at a small fraction of the FP32 rate on this GPU, and a prefill chunk
// rotates millions of elements.)  x*cos_hi and y*sin_hi are split exactly into product + error by FMA, the low
// halves of cos / sin are folded in, and the sum is kept as an unevaluated f32 pair hi + lo that is within
// 2^-44 (|x cos| + |y sin|) of the exact value; the float64 expression is within 2^-51 of it.  fl32 of both is the
// same number unless the value lies within that distance of a rounding boundary of f32 (hi +- ulp/2, or hi - ulp/4
// below a power of two): only then (about one output in 2^17, and for zero, tiny, huge or non-finite operands) the
// float64 instructions run.
__device__ __forceinline__ float rot_exact(float x, float y, const Angle& g, bool minus) {
  const float ys = minus ? -y : y;
  const float p1 = __fmul_rn(x, g.c_hi), e1 = __fmaf_rn(x, g.c_hi, -p1), t1 = __fmaf_rn(x, g.c_lo, e1);
  const float p2 = __fmul_rn(ys, g.s_hi), e2 = __fmaf_rn(ys, g.s_hi, -p2), t2 = __fmaf_rn(ys, g.s_lo, e2);
  const float sh = __fadd_rn(p1, p2), z = __fsub_rn(sh, p1);
  const float se = __fadd_rn(__fsub_rn(p1, __fsub_rn(sh, z)), __fsub_rn(p2, z));   // p1 + p2 = sh + se exactly
  const float l0 = __fadd_rn(se, __fadd_rn(t1, t2));
  const float hi = __fadd_rn(sh, l0), lo = __fsub_rn(l0, __fsub_rn(hi, sh));
  const float M = __fadd_rn(fabsf(p1), fabsf(p2));
  const float delta = __fmul_rn(M, 2.2737368e-13f);   // 2^-42 M: well above both error bounds
  const float ah = fabsf(hi), al = fabsf(lo);
  const float u = __fmul_rn(__uint_as_float(__float_as_uint(ah) & 0x7f800000u), 1.1920929e-7f);   // ulp(hi) = 2^(e-23)
  const bool safe = M > 7.8886091e-31f && M < 1.2676506e30f && ah > 7.8886091e-31f &&      // 2^-100 .. 2^100
                    fabsf(__fsub_rn(al, 0.5f * u)) > delta && fabsf(__fsub_rn(al, 0.25f * u)) > delta && al <= 0.5f * u;
  if (safe) return hi;
  const double a = __dmul_rn((double)x, g.c), b = __dmul_rn((double)y, g.s);
  return (float)(minus ? __dsub_rn(a, b) : __dadd_rn(a, b));
}

// hi + lo f16 pair of an f32: x ~= hi + lo with about 22 significant bits
__device__ __forceinline__ void split_h(float x, __half& hi, __half& lo) {
  hi = __float2half_rn(x);
  lo = __float2half_rn(x - __half2float(hi));
}

// Programmatic dependent launch.  A kernel launched with launch_pdl() may begin before its predecessor in the
// stream has finished, once every CTA of the predecessor has called pdl_trigger() or exited; pdl_wait() returns
// when the predecessor has completed and its writes are visible.  Rule used by this library: every kernel calls
// pdl_wait() before its first global write and before reading anything an earlier kernel of the stream wrote, and
// only the RoPE/append kernel triggers before its own wait, so whatever runs ahead of its predecessor's end
// overlaps nothing but that one kernel.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void named_bar_arrive(uint32_t id, uint32_t threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- host side -----------------------------------------------------------------------------------

// Consumer groups of the decode kernel for a call of nt 8-row groups of query rows.  The kernel can run two groups of
// four warps on alternate tiles (slots carry tile numbers, the second group's (o, m, l) is folded into the first's
// before the record is written); measured on config 2 that is slower than one group: a group's tile goes from 1.2 to
// 1.7 us when another group shares the SM's shared-memory bandwidth (each tile re-reads the hi and lo query fragments
// besides K and V), and the fold adds a microsecond at the end.  One group is what runs.
__host__ __device__ constexpr int decode_groups(int nt) { return nt >= 0 ? 1 : 2; }

constexpr int kMaxItems = 32;     // items of one batched decode call
constexpr int kMaxRows = 64;      // query rows (columns x heads of one kv head) one decode CTA carries

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

struct ItemList {
  uint32_t seq[kMaxItems];
  int32_t lim0[kMaxItems];     // cache rows column 0 sees, before clamping: pos + 1 - layer origin (may be <= 0)
  uint32_t n_rows[kMaxItems];  // cache rows the last column sees: clamp(pos + n_cols - origin, 0, max_seq)
  uint32_t n_cols[kMaxItems];
  uint32_t col0[kMaxItems];    // first column of the item in q / gate / out
  uint32_t pos[kMaxItems];     // position of the item's first column
};

// Peer exchange of merged (o, m, l) records between the GPUs of one box.  Every rank owns one buffer that all ranks
// (itself included) write into with plain 8-byte stores over NVLink; peer[r] is rank r's buffer as seen from this
// GPU.  Layout of a buffer, in 8-byte entries {f32 value, u32 tag}, for parity p in {0,1} and source rank s: block
// (p * world + s) of max_rows * (hd + 2 * hd/64) entries (o rows first, then (m, l) per (row, 64-dim slice)).  The
// tag is the call counter + 1: a receiver spins on an entry until it carries the current call's tag.
struct ExchangeView {
  float* peer[8];
  uint32_t world, rank, max_rows, hd;
  unsigned int* ctr;   // local: [0] call counter (epoch); every exchanging call advances it once, ahead of its combine kernel
};

}  // namespace pa

struct pa_ctx {
  int device = 0;
  int sm_count = 148;
  int smem_optin = 0;
  pa_config cfg{};
  uint32_t G = 1, q_dim = 0, kv_dim = 0;
  double* inv_freq = nullptr;  // device: theta^(-2i/n_rot), i < n_rot/2, evaluated on the host in float64
  double inv_freq_host[128] = {};   // the same table on the host
  // The one call whose cache writes may still be in flight when the kernels of the next call start ahead of their
  // own wait: a fused one-token decode (its kernel appends the row) or a stand-alone append.  The next call on the
  // same layer fetches early only below inflight_row0 (row within the layer's shard).
  // cos / sin table of the current step's columns (PA_ROPE_F64), filled by pa_angles_kernel.  Valid for calls with
  // the same position and width in the same capture (or, outside captures, until a graph that rewrites it may have
  // been replayed: once a capture has been seen, stand-alone calls refill it, except inside one multi-layer call).
  pa::Angle host_ang[64];            // the last small call's angles (host libm), reused while the position repeats
  uint32_t host_ang_pos = 0, host_ang_n = 0;
  pa::Angle* angles = nullptr;
  uint32_t angles_pos0 = 0, angles_n = 0;
  unsigned long long angles_capture = 0;
  bool angles_valid = false, ever_captured = false, scope_active = false, scope_fresh = false;
  const pa_layer* inflight_layer = nullptr;
  uint32_t inflight_row0 = 0;
  float* q_rot = nullptr;      // device: rotated q of the current call, f32 [max_cols][q_dim]
  float* k_rot = nullptr;      // device: rotated k of the current call, f32 [max_cols][kv_dim] (int8 / f32 caches; made with the first such layer)
  float* part_o = nullptr;     // device: split partials, f32 [rows][splits][head_dim] of the current call
  float* part_ml = nullptr;    // device: f32 [rows][splits][2]
  uint32_t max_splits = 0;
  size_t part_slots = 0;       // (query row, split) records the partial buffers hold
  unsigned int* merge_ctr = nullptr;   // device: per (item, kv head) of a decode call, records left and CTAs done merging (zero between calls)
  uint32_t merge_slots = 0;
  uint32_t* dev_err = nullptr;   // device error word (bounded waits)
  uint32_t* host_err = nullptr;  // pinned mirror
  void* norm_q = nullptr;        // normed q / k of the current layer call (act_dtype, [max_cols][q_dim] / [max_cols][kv_dim])
  void* norm_k = nullptr;
  void* stage_dev = nullptr;     // device staging of the host-buffer entry point
  void* stage_host = nullptr;    // pinned staging
  size_t stage_bytes = 0;
  pa::ExchangeView xc{};         // peer exchange (pa_exchange_init); world == 0: not set up
  std::vector<cudaEvent_t> ev;   // timing: event pairs around core-kernel launches
  size_t ev_used = 0;
  bool timing = false;
  bool core_only = false;        // profiling aid: calls launch their core kernel only
  // measurement switches, read from the environment once when the context is created
  struct Tuning {
    int pre_stages = 2;          // POOLED_ATTN_PRE_STAGES: K/V tiles a decode CTA fetches ahead of its predecessor's end
    int next_tiles = 0;          // POOLED_ATTN_NEXT_TILES: tiles of the next layer each decode CTA asks L2 to fetch at its end
    bool no_fuse = false;        // POOLED_ATTN_NO_FUSE: RoPE/append -> decode -> combine chain instead of the fused front
    bool verify_mma_sync = false;// POOLED_ATTN_VERIFY_MMA_SYNC: k-token blocks on the mma.sync kernel
    int own_prefetch = 0;        // POOLED_ATTN_OWN_PREFETCH=n: L2 requests for n of a decode CTA's own later tiles at entry
    int xch_prefetch = 0;        // POOLED_ATTN_XCH_PREFETCH=n: the same for calls that end in a cross-GPU exchange
    bool no_q_tma = false;       // POOLED_ATTN_NO_Q_TMA=1: the prefill kernel's query rows through the softmax threads' registers
    bool old_tail = false;       // POOLED_ATTN_OLD_TAIL=1: in-kernel merge with every CTA waiting for the records (unit-less ones too)
    bool no_out_tma = false;     // POOLED_ATTN_NO_OUT_TMA=1: ... and its output rows by per-thread stores
    bool kv_evict_first = true;  // POOLED_ATTN_KV_EVICT_FIRST=0: decode / verify K and V tiles enter L2 with the default policy instead of evict-first
    bool no_merge = false;       // POOLED_ATTN_NO_MERGE: always merge the split records in the combine kernel
    uint32_t wait_polls = 0;     // pa_set_wait_limit: limit of the cross-GPU exchange wait (0: the built-in limit)
  } tune;
  bool failed = false;
  std::string err;
  pa_stats stats{};
};

struct pa_layer {
  pa_ctx* ctx = nullptr;
  uint32_t n_seqs = 0, max_seq = 0;
  uint32_t origin = 0;           // global position of cache row 0 (a shard of a longer sequence)
  __half* k = nullptr;           // f16 caches (PA_KV_F16) ...
  __half* v = nullptr;
  int kv_format = PA_KV_F16;
  void* k_alt = nullptr;         // ... or int8 / f32 caches (PA_KV_Q8 / PA_KV_F32) ...
  void* v_alt = nullptr;
  float* k_scale = nullptr;      // ... with one f32 scale per 32 values (PA_KV_Q8)
  float* v_scale = nullptr;
  CUtensorMap tm_k64, tm_v64;    // 64-row boxes over all sequences' rows, for the decode kernel
  const pa_layer* next = nullptr; // the layer the engine runs after this one (pa_layer_set_next): its first tiles are
                                  // requested into L2 while this layer's call drains
  const float* qnorm_w = nullptr;   // QK head-norm weights of this layer (device, f32 [head_dim]); nullptr: the layer
  const float* knorm_w = nullptr;   // call takes q and k as they come
  double norm_eps = 0.0;
};
