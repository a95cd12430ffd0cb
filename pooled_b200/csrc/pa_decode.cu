// Split-K flash-decode / k-token verify for an f16 KV cache, and the LSE combine that follows it.
//
// One CTA per (split of the KV sequence, kv head, item).  All query rows that share the kv head — the G
// heads of the GQA group times the item's columns, at most 64 — ride in the same CTA, so every K and V
// byte is fetched from HBM once.  A producer thread streams 64-position K and V tiles with TMA
// (cp.async.bulk.tensor, 128-byte swizzle, each CTA fetching its own tiles) into a ring of shared-memory slots guarded by
// mbarriers; four consumer warps take the tiles apart with ldmatrix and multiply on the tensor cores
// (mma.sync m16n8k16, f32 accumulate):
//     S^T[pos, row] = K[pos, :] . Q[row, :]        warp w owns positions 16w .. 16w+15 of the tile
//     O^T[dim, row] += V^T[dim, pos] . P^T[pos, row]   warp w owns a quarter of the head dims
// with an online softmax in between (running maximum and sum per row, exchanged between the warps through
// shared memory).  q, and the softmax weights P, enter the tensor cores as hi + lo f16 pairs unless the
// context asks for PA_FLAG_FAST, so the result carries about 22 significant bits of both.
// The kernel is HBM-bound: 2 * rows * head_dim * 2 bytes per kv head; the math needs a fraction of the
// time a tile takes to arrive.
//
// With at most 16 query rows the consumers come as two groups of four warps that take alternate tiles of the CTA's
// range, each with its own running (m, l, o): one group's tile is latency-bound (fragment loads, two barriers, the
// exponentials: about 1.3 us), two in flight keep up with data that arrives faster than that (from L2, or while the
// ring is full).  Each group leaves its own partial record.
//
// Gather mode (pa_decode_gather): a column attends a list of cache rows instead of rows 0 .. n-1.  List position t
// stands where position t stands otherwise; the producer warp fetches the listed rows with 16-byte cp.async into the
// very slots and swizzle a TMA tile would fill, so everything after the load is the same arithmetic in the same order.
//
// Each group writes an unnormalised partial (o, m, l) per query row; pa_combine_kernel merges the records
// (out = sum o_s e^(m_s-M) / sum l_s e^(m_s-M)), applies the sigmoid gate and stores f32 or f16.
//
// Stands in for attn_dec / attn_dec_combine / attn_dec_combine_g of pooled (engine/wgsl/attn_dec.js:67-287).
#include "pa_params.cuh"

namespace pa {


constexpr int kT = 64;             // positions per tile
constexpr int kConsumers = 128;    // 4 consumer warps per group
constexpr int kMaxStages = 8;


// acc += x * w, each component one fused multiply-add: the merge inside the decode kernel (merge_slice_128) and the
// combine kernel round the same way, so either path gives the same bits
__device__ __forceinline__ void fma4(float4& acc, const float4& x, float w) {
  acc.x = __fmaf_rn(x.x, w, acc.x); acc.y = __fmaf_rn(x.y, w, acc.y); acc.z = __fmaf_rn(x.z, w, acc.z); acc.w = __fmaf_rn(x.w, w, acc.w);
}

// Cross-GPU step of a merge.  Every rank publishes its merged slice of a query row (64 dims of o, and m, l) into every
// rank's buffer, waits (bounded) for the other ranks' slices and merges them in rank order, so every rank ends with the
// same bits.  Every value travels as one 8-byte store {value, tag} (tag = call counter + 1): an 8-byte store lands
// whole, so the receiver spins on the words themselves and no flag, fence or second round trip is needed.  The buffers
// alternate with the call counter's parity.  The counter is advanced once per exchanging call, ahead of the combine
// kernel that reads it: by the first thread of the call's decode kernel after its wait (every kernel of the call
// before has finished then), or by a one-thread kernel where no decode kernel runs.  (Counting the slices through at
// the end of the combine kernel instead put 512 atomics on one word at the tail of a 128-row call.)
// A thread owns NV dims of the slice (dd[]: dims within the slice).  `epoch`: the call counter as the combine kernel
// finds it after its wait.
template <int HD>
struct XchSlot {
  size_t blk, o_idx, ml_idx;
  uint32_t parity, tag;
  // d0: first dim of the unit (a multiple of 32); (m, l) are kept per 64-dim slice
  __device__ __forceinline__ XchSlot(const ExchangeView& x, uint32_t epoch, uint32_t prow, uint32_t d0) {
    constexpr uint32_t n_slices = HD / 64;
    parity = epoch & 1u; tag = epoch + 1u;
    blk = (size_t)x.max_rows * (HD + 2 * n_slices);   // entries of 8 bytes: o rows, then (m, l) per (row, slice)
    o_idx = (size_t)prow * HD + d0;
    ml_idx = (size_t)x.max_rows * HD + ((size_t)prow * n_slices + d0 / 64) * 2;
  }
};
__device__ __forceinline__ void xch_store(uint2* dst, float v, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
// o values of this thread's dims (n_o of them: 0 for a thread that only carries m and l) and, from one thread, (m, l)
template <int HD, int NV>
__device__ __forceinline__ void xch_put(const ExchangeView& x, const XchSlot<HD>& a, const uint32_t (&dd)[NV], const float (&t)[NV], bool with_o, bool with_ml,
                                        float M, float Lsum) {
  for (uint32_t r = 0; r < x.world; ++r) {
    uint2* dst = reinterpret_cast<uint2*>(x.peer[r]) + (size_t)(a.parity * x.world + x.rank) * a.blk;
    if (with_o) {
#pragma unroll
      for (int k = 0; k < NV; ++k) xch_store(dst + a.o_idx + dd[k], t[k], a.tag);
    }
    if (with_ml) { xch_store(dst + a.ml_idx, M, a.tag); xch_store(dst + a.ml_idx + 1, Lsum, a.tag); }
  }
}
// every sweep requests all entries still missing at once (m, l and this thread's o of every source rank) and keeps
// those that carry the call's tag; bounded.  t and Lsum come back as the merged sums over all ranks.
template <int HD, int NV>
__device__ __forceinline__ void xch_get(const ExchangeView& x, const XchSlot<HD>& a, const uint32_t (&dd)[NV], float (&t)[NV], float& Lsum, uint32_t sweeps,
                                        uint32_t* err) {
  const uint2* mine = reinterpret_cast<const uint2*>(x.peer[x.rank]);
  float mr[8], lr[8], orr[8][NV];
  uint32_t pending = (1u << x.world) - 1u;
  for (uint32_t it = 0; it < sweeps && pending; ++it) {
    uint32_t v[8][2 + NV], tg[8][2 + NV];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (!((pending >> r) & 1u)) continue;
      const uint2* src = mine + (size_t)(a.parity * x.world + r) * a.blk;
      asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v[r][0]), "=r"(tg[r][0]) : "l"(src + a.ml_idx) : "memory");
      asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v[r][1]), "=r"(tg[r][1]) : "l"(src + a.ml_idx + 1) : "memory");
#pragma unroll
      for (int k = 0; k < NV; ++k)
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v[r][2 + k]), "=r"(tg[r][2 + k]) : "l"(src + a.o_idx + dd[k]) : "memory");
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (!((pending >> r) & 1u)) continue;
      bool all = tg[r][0] == a.tag && tg[r][1] == a.tag;
#pragma unroll
      for (int k = 0; k < NV; ++k) all = all && tg[r][2 + k] == a.tag;
      if (all) {
        mr[r] = __uint_as_float(v[r][0]); lr[r] = __uint_as_float(v[r][1]);
#pragma unroll
        for (int k = 0; k < NV; ++k) orr[r][k] = __uint_as_float(v[r][2 + k]);
        pending &= ~(1u << r);
      }
    }
    if (pending && it > 1024) __nanosleep(64);
  }
  if (pending) atomicMax(err, (uint32_t)WAIT_PEER);   // a peer never published: report and carry on
  float Mg = -3.0e38f;
#pragma unroll
  for (int r = 0; r < 8; ++r) if ((uint32_t)r < x.world && !((pending >> r) & 1u)) Mg = fmaxf(Mg, mr[r]);
  float Lg = 0.f, og[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) og[k] = 0.f;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    if ((uint32_t)r >= x.world || ((pending >> r) & 1u)) continue;
    const float w = __expf(mr[r] - Mg);
    Lg = __fmaf_rn(lr[r], w, Lg);
#pragma unroll
    for (int k = 0; k < NV; ++k) og[k] = __fmaf_rn(orr[r][k], w, og[k]);
  }
#pragma unroll
  for (int k = 0; k < NV; ++k) t[k] = og[k];
  Lsum = Lg;
}
// the three steps for a slice held by threads 0..63 (one dim each) with m and l in thread 64
template <int HD>
__device__ __forceinline__ void exchange_slice(const ExchangeView& x, uint32_t prow, uint32_t slice, int tid, float& t, float M, float& Lsum, uint32_t sweeps,
                                               uint32_t* err, uint32_t epoch) {
  const XchSlot<HD> a(x, epoch, prow, slice * 64);
  const uint32_t dd[1] = {(uint32_t)tid & 63u};
  float tv[1] = {t};
  xch_put<HD, 1>(x, a, dd, tv, tid < 64, tid == 64, M, Lsum);
  if (tid < 64) {
    xch_get<HD, 1>(x, a, dd, tv, Lsum, sweeps, err);
    t = tv[0];
  }
}

// LSE merge of the ns split records of one query row over one 64-dim slice, gate and store, by the 128 consumer threads
// of a decode CTA: the arithmetic of pa_combine_kernel, operation for operation and in the same order (that kernel has
// 256 threads; thread t here does the work of its threads t and t + 128), so a call gives the same bits whether its
// records are merged here or there.  o_rec / ml_rec: record 0 of the row; records follow one another.  Scratch: 6 KB of
// shared memory no one else uses any more.  bar: the group's named barrier.
struct MergeScratch { float w[512]; float red[8]; float red2[8]; float4 acc[16][16]; };
template <int HD>
__device__ __forceinline__ void merge_slice_128(const float* __restrict__ o_rec, const float* __restrict__ ml_rec, uint32_t ns, uint32_t slice, int t,
                                                MergeScratch& sc, uint32_t bar, bool gated, float gv, bool empty_is_zero, int act_f16, void* out, uint64_t oo) {
  const int wv = t >> 5, lane = t & 31, ln = t & 15, gA = t >> 4;
  // everything is requested before the first use: one memory round trip
  float mv[4], lv[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t s = t + 128 * k;
    mv[k] = -3.0e38f; lv[k] = 0.f;
    if (s < ns) { mv[k] = __ldcg(ml_rec + 2 * s); lv[k] = __ldcg(ml_rec + 2 * s + 1); }
  }
  const float* ob = o_rec + slice * 64 + ln * 4;
  float4 xa[8], xb[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const uint32_t sa = gA + 16 * u, sb = gA + 8 + 16 * u;
    xa[u] = sa < ns ? __ldcg(reinterpret_cast<const float4*>(ob + (size_t)sa * HD)) : make_float4(0.f, 0.f, 0.f, 0.f);
    xb[u] = sb < ns ? __ldcg(reinterpret_cast<const float4*>(ob + (size_t)sb * HD)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float M = fmaxf(fmaxf(mv[0], mv[1]), fmaxf(mv[2], mv[3]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  if (lane == 0) sc.red[wv] = M;
  named_bar_sync(bar, kConsumers);
  M = fmaxf(fmaxf(sc.red[0], sc.red[1]), fmaxf(sc.red[2], sc.red[3]));
  float wk[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t s = t + 128 * k;
    wk[k] = s < ns ? __expf(mv[k] - M) : 0.f;
    sc.w[s] = wk[k];
  }
  // the combine kernel's thread v sums records v and v + 256, then its warp reduces: v = t and v = t + 128 here
  float LpA = __fmaf_rn(lv[2], wk[2], __fmul_rn(lv[0], wk[0])), LpB = __fmaf_rn(lv[3], wk[3], __fmul_rn(lv[1], wk[1]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    LpA = __fadd_rn(LpA, __shfl_xor_sync(0xffffffffu, LpA, o));
    LpB = __fadd_rn(LpB, __shfl_xor_sync(0xffffffffu, LpB, o));
  }
  if (lane == 0) { sc.red2[wv] = LpA; sc.red2[wv + 4] = LpB; }
  named_bar_sync(bar, kConsumers);
  float Lsum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) Lsum = __fadd_rn(Lsum, sc.red2[i]);
  float4 accA = make_float4(0.f, 0.f, 0.f, 0.f), accB = accA;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const uint32_t sa = gA + 16 * u, sb = gA + 8 + 16 * u;
    fma4(accA, xa[u], sa < ns ? sc.w[sa] : 0.f);
    fma4(accB, xb[u], sb < ns ? sc.w[sb] : 0.f);
  }
  for (int h = 0; h < 2; ++h) {
    const uint32_t g = gA + 8 * h;
    float4& acc = h ? accB : accA;
    for (uint32_t s0 = g + 128; s0 < ns; s0 += 64) {
      float4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t s = s0 + 16 * u;
        x[u] = s < ns ? __ldcg(reinterpret_cast<const float4*>(ob + (size_t)s * HD)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t s = s0 + 16 * u;
        fma4(acc, x[u], s < ns ? sc.w[s] : 0.f);
      }
    }
  }
  sc.acc[gA][ln] = accA; sc.acc[gA + 8][ln] = accB;
  named_bar_sync(bar, kConsumers);
  float tt = 0.f;
  if (t < 64) {
    const float* sa = reinterpret_cast<const float*>(sc.acc);
    tt = sa[t];
#pragma unroll
    for (int i = 1; i < 16; ++i) tt = __fadd_rn(tt, sa[i * 64 + t]);
  }
  if (t < 64) {
    float rv = (empty_is_zero && Lsum == 0.f) ? 0.f : __fdiv_rn(tt, Lsum);
    if (gated) rv = __fmul_rn(rv, __fdiv_rn(1.0f, __fadd_rn(1.0f, __expf(-gv))));
    if (act_f16) reinterpret_cast<__half*>(out)[oo + t] = __float2half_rn(rv);
    else reinterpret_cast<float*>(out)[oo + t] = rv;
  }
  named_bar_sync(bar, kConsumers);   // the scratch is free again
}

template <int HD, int NT, bool PRECISE>
struct DecSmem {
  static constexpr int NG = decode_groups(NT);       // consumer groups
  static constexpr int THREADS = NG * kConsumers + 32;   // + 1 producer warp
  static constexpr int ROWS = NT * 8;
  static constexpr int SLOT = kT * HD * 2;           // bytes of one K or V tile
  static constexpr int QP = HD * 2 + 16;             // q row pitch (bytes): 16-byte skew against bank conflicts
  static constexpr int PP = ROWS * 2;                // P^T row pitch (bytes)
  static constexpr int Q_BYTES = ROWS * QP * (PRECISE ? 2 : 1);
  static constexpr int P_BYTES = kT * PP * (PRECISE ? 2 : 1);      // per group
  static constexpr int MISC = NG * 4 * ROWS * 4 * 2 + kMaxStages * 4 * 8 + 64 + 2048 + 1024 + 64;   // + the fused front's angles and new row, the slots' tile numbers
  static constexpr int fixed_bytes() { return Q_BYTES + NG * P_BYTES + MISC; }
  static int stages_for(int smem_limit) {
    int s = (smem_limit - 1024 - fixed_bytes()) / (2 * SLOT);
    return s > kMaxStages ? kMaxStages : s;
  }
  static int total_bytes(int stages) { return 1024 + stages * 2 * SLOT + fixed_bytes(); }
};

static_assert(sizeof(DecodeParams) + 4 * sizeof(CUtensorMap) <= 4096, "the decode kernel's launch parameters must fit 4 KB");

template <int HD, int NT, bool PRECISE>
__global__ void __launch_bounds__(DecSmem<HD, NT, PRECISE>::THREADS, 1)
pa_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kn,
                 const __grid_constant__ CUtensorMap tm_vn, const DecodeParams p) {
  using L = DecSmem<HD, NT, PRECISE>;
  constexpr int ROWS = L::ROWS, SLOT = L::SLOT, QP = L::QP, PP = L::PP;
  constexpr int NG = L::NG, CONS = NG * kConsumers, kDecThreads = L::THREADS, PW = 4 * NG;   // PW: the producer warp
  constexpr int MT = HD / 64;        // 16-dim output tiles per consumer warp
  constexpr int CH = HD / 64;        // 128-byte chunks per cache row of one kv head

  const uint32_t split = blockIdx.x, g = blockIdx.y, item = blockIdx.z;
  if (p.xch_ctr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    pdl_wait();                    // the exchanging call before this one has read the counter
    atomicAdd(p.xch_ctr, 1u);      // this call's number: its combine kernel starts after this kernel's end
  }
  const uint32_t n_cols = p.items.n_cols[item];
  if (p.gather) pdl_wait();   // the lists may come from the kernel before this one
  // gather: the item is one column whose list (length, then rows ascending) lives on the device; the split plan is
  // what the host would make for that many rows
  const uint32_t* g_list = p.gather ? p.gather + (size_t)p.items.col0[item] * p.gather_stride : nullptr;
  const uint32_t n_rows = g_list ? min(g_list[0], p.gather_stride - 1u) : p.items.n_rows[item];   // cache rows the last column sees
  const uint32_t tiles = (n_rows + kT - 1) / kT;
  // every item plans for its own length: at least two tiles per CTA, at most the launch's split count (the longest
  // item's plan, or in gather mode the most any list could need)
  const uint32_t ns_eff = min(p.n_splits, max(1u, tiles / 2));
  const uint32_t tps = (tiles + ns_eff - 1) / max(ns_eff, 1u);  // tiles per split
  const uint32_t tile0 = split * tps;
  if (tile0 >= tiles) {
    if constexpr (NT <= 2) {
      // a call that merges its own records has no combine kernel behind it to give an empty list its zeros
      if (p.merge && g_list && tiles == 0 && split == 0) {
        pdl_wait();
        const uint32_t G = p.G;
        for (uint32_t idx = threadIdx.x; idx < n_cols * G * HD; idx += blockDim.x) {
          const uint32_t row = idx / HD, d = idx % HD, c = row / G, hh = row % G;
          const uint64_t oo = (uint64_t)(p.items.col0[item] + c) * p.out_col_stride + (uint64_t)(g * G + hh) * HD + d;
          if (p.act_f16) reinterpret_cast<__half*>(p.out)[oo] = __float2half_rn(0.f);
          else reinterpret_cast<float*>(p.out)[oo] = 0.f;
        }
      }
    }
    return;
  }
  const uint32_t tile1 = min(tiles, tile0 + tps);
  const uint32_t n_tiles = tile1 - tile0;
  const uint32_t NS = p.n_stages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_slots = base;
  uint8_t* v_slots = base + NS * SLOT;
  uint8_t* q_hi = v_slots + NS * SLOT;
  uint8_t* q_lo = q_hi + ROWS * QP;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = warp < PW ? warp >> 2 : 0;                    // consumer group of this warp
  uint8_t* p_hi = q_hi + L::Q_BYTES + grp * L::P_BYTES;          // P^T of this group
  uint8_t* p_lo = p_hi + kT * PP;
  float* s_max0 = reinterpret_cast<float*>(q_hi + L::Q_BYTES + NG * L::P_BYTES);
  float* s_max = s_max0 + grp * 8 * ROWS;                       // [4][ROWS] of this group
  float* s_l = s_max + 4 * ROWS;                                // [4][ROWS]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_max0 + NG * 8 * ROWS); // kfull, kempty, vfull, vempty [kMaxStages] each
  volatile uint32_t* s_err = reinterpret_cast<volatile uint32_t*>(bars + 4 * kMaxStages);
  Angle* s_ang = reinterpret_cast<Angle*>(bars + 4 * kMaxStages + 8);   // [64], fused front only
  uint32_t* s_newk = reinterpret_cast<uint32_t*>(s_ang + 64);           // the token's own K / V row as f16 pairs (fused front)
  uint32_t* s_newv = s_newk + 128;
  // which tile each K slot [0..7] and V slot [8..15] holds or is being filled with.  With two consumer groups a slot
  // serves the groups in turn, and a group may come for its tile before the other group's earlier tile has even landed
  // there; a parity wait alone cannot tell "not yet" from "two phases on", the tile number can.
  volatile uint32_t* s_tile = reinterpret_cast<volatile uint32_t*>(s_newv + 128);

  const uint32_t kfull = smem_u32(bars), kempty = kfull + kMaxStages * 8, vfull = kempty + kMaxStages * 8,
                 vempty = vfull + kMaxStages * 8;

  // The consumers put their q loads in flight before the producer may start: a q load issued behind the
  // first 190 KB of K/V tiles of every SM would wait for all of them at the memory controllers.
  // With few query rows the values wait in registers across the barrier; with many they are staged into shared
  // memory first (the producer then starts about one memory round trip later).
  constexpr int QLD = ROWS * (HD / 2) / kConsumers;
  constexpr bool Q_IN_REGS = QLD <= 16;
  float2 qreg[Q_IN_REGS ? QLD : 1];
  const uint32_t G = p.G, live_rows = n_cols * G;
  auto q_load_rd = [&](int row, int d) {
    float2 x = make_float2(0.f, 0.f);
    if ((uint32_t)row < live_rows) {
      const uint32_t c = row / G, hh = row % G;
      const uint64_t off = (uint64_t)(p.items.col0[item] + c) * p.q_col_stride + (uint64_t)(g * G + hh) * p.q_head_stride + d;
      if (p.q_f16) x.x = __uint_as_float(*reinterpret_cast<const uint32_t*>(reinterpret_cast<const __half*>(p.q) + off));
      else x = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(p.q) + off);
    }
    return x;   // f16 input: the two halves, unconverted, in x.x -- nothing here waits for the load to land
  };
  auto q_load = [&](int idx) { return q_load_rd(idx / (HD / 2), (idx % (HD / 2)) * 2); };
  // a hint only (L2 is the point of coherence: a line the predecessor rewrites afterwards is simply updated there)
  auto q_pref_rd = [&](int row, int d) {
    if ((uint32_t)row >= live_rows) return;
    const uint32_t c = row / G, hh = row % G;
    const uint64_t off = (uint64_t)(p.items.col0[item] + c) * p.q_col_stride + (uint64_t)(g * G + hh) * p.q_head_stride + d;
    const void* a = p.q_f16 ? (const void*)(reinterpret_cast<const __half*>(p.q) + off) : (const void*)(reinterpret_cast<const float*>(p.q) + off);
    asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
  };
  auto act_cvt = [&](float2 raw) {
    if (!p.q_f16) return raw;
    const uint32_t u = __float_as_uint(raw.x);
    return __half22float2(*reinterpret_cast<const __half2*>(&u));
  };
  auto q_store_rd = [&](int row, int d, float2 x) {
    __half h0, l0, h1, l1;
    split_h(x.x, h0, l0); split_h(x.y, h1, l1);
    *reinterpret_cast<__half2*>(q_hi + row * QP + d * 2) = __halves2half2(h0, h1);
    if (PRECISE) *reinterpret_cast<__half2*>(q_lo + row * QP + d * 2) = __halves2half2(l0, l1);
  };
  auto q_store = [&](int idx, float2 x) { q_store_rd(idx / (HD / 2), (idx % (HD / 2)) * 2, x); };
  // Fused front (one token, 64 rotated dims, head_dim 256): q arrives unrotated; cos / sin of the float64 angle come
  // with the launch parameters.  The rotation is spread over all 128 consumer threads: thread t takes row t / 16 and
  // the dims (2b, 2b + 1) with their partners (2b + 32, 2b + 33), b = t % 16 (four outputs), and six of the 768
  // unrotated pairs.  In the CTA that walks the sequence's last tile thread t also carries dims (2t, 2t + 1) of the
  // token's own k / v row (rotary partners sit in lanes l and l ^ 16 of warp 0: one shuffle): rotated, rounded to f16,
  // stored to the cache, and kept in two registers to be placed into the tile the TMA fetched before (or while) it
  // was stored.
  // The two fused shapes: head_dim 256 with 64 rotary dims (the rest of a row is copied), and head_dim 128 rotated
  // in full.  An item is two adjacent dims with their rotary partners; thread t takes items t, t + 128, ...
  constexpr bool CAN_FUSE = NT == 1 && (HD == 256 || HD == 128);
  constexpr int NRD = HD == 256 ? 64 : HD;            // rotated dims
  constexpr int RHALF = NRD / 2, IPR = RHALF / 2;     // partner distance; items per row
  constexpr int RIT = CAN_FUSE ? ROWS * IPR / kConsumers : 1;   // rotated items per thread (1 or 2)
  constexpr int PPR = (HD - NRD) / 2;                 // unrotated pairs per row (96 or 0)
  const bool fused = CAN_FUSE && p.fused;
  const bool own_new = fused && ((p.append >> item) & 1u) && tile1 == tiles;
  float2 kx = make_float2(0.f, 0.f), vx = make_float2(0.f, 0.f), kxb = make_float2(0.f, 0.f);
  uint32_t k_new2 = 0, v_new2 = 0, k_new2b = 0;       // head_dim 128: lanes of warp 0 carry K words t and t + 32
  auto rotate = [&](float2 x) {   // warp 0 only, all lanes
    const float2 y = make_float2(__shfl_xor_sync(0xffffffffu, x.x, 16), __shfl_xor_sync(0xffffffffu, x.y, 16));
    const int i = 2 * (lane & 15);
    // first element of a pair (lanes 0-15): a cos - b sin; second: b cos + a sin -- own * cos -/+ partner * sin
    float2 o;
    o.x = rot_exact(x.x, y.x, s_ang[i], lane < 16);
    o.y = rot_exact(x.y, y.y, s_ang[i + 1], lane < 16);
    return o;
  };
  if (warp < 4) {
    // Threads that index launch parameters differently are served one address at a time, each a miss of the constant
    // cache: far too slow for the critical path.  The angles go to shared memory while the predecessor still runs.
    if (fused) {
      if (p.fused == 2) {
        // several items, each at its own position: the CTA evaluates its item's angles while the predecessor still runs
        if (tid < RHALF) {
          double sn, cs;
          sincos(__dmul_rn((double)p.items.pos[item], p.inv_freq[tid]), &sn, &cs);
          s_ang[tid] = make_angle(cs, sn);
        }
      } else {
#pragma unroll
        for (int u = 0; u < RHALF / 32; ++u) reinterpret_cast<uint2*>(s_ang)[tid + u * kConsumers] = reinterpret_cast<const uint2*>(p.rope_ang)[tid + u * kConsumers];
      }
    }
    if (p.merge && p.gate && p.prefetch_old_rows && tid < 4) {
      // the gate values of the (row, slice) unit this CTA will merge at the end: into L2 ahead of the K/V traffic
      const uint32_t u = split, n_units = live_rows * (HD / 64);
      if (u < n_units) {
        const uint32_t row = u / (HD / 64), slice = u % (HD / 64), c = row / G, hh = row % G;
        const uint64_t go = (uint64_t)(p.items.col0[item] + c) * p.gate_col_stride + (uint64_t)(g * G + hh) * p.gate_head_stride + slice * 64 + tid * 16;
        const void* a = p.act_f16 ? (const void*)(reinterpret_cast<const __half*>(p.gate) + go) : (const void*)(reinterpret_cast<const float*>(p.gate) + go);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
      }
    }
    if (Q_IN_REGS && p.prefetch_old_rows) {   // the CTA is ahead of its predecessor: bring the q lines to L2 meanwhile
      if (fused) {
#pragma unroll
        for (int u = 0; u < RIT; ++u) { const int i = tid + u * kConsumers; q_pref_rd(i / IPR, 2 * (i % IPR)); }
        if (PPR > 0) {
#pragma unroll
          for (int it = 2 * RIT; it < (Q_IN_REGS ? QLD : 1); it += 2) { const int idx = tid + (it - 2 * RIT) * kConsumers; q_pref_rd(idx / (PPR ? PPR : 1), NRD + 2 * (idx % (PPR ? PPR : 1))); }
        }
      } else {
#pragma unroll
        for (int it = 0; it < (Q_IN_REGS ? QLD : 1); it += 2) { const int idx = tid + it * kConsumers; q_pref_rd(idx / (HD / 2), (idx % (HD / 2)) * 2); }
      }
    }
    pdl_wait();      // q (and the partial buffers written at the end) belong to earlier kernels until here
    pdl_trigger();
    if (Q_IN_REGS) {
      if (fused) {
#pragma unroll
        for (int u = 0; u < RIT; ++u) {
          const int i = tid + u * kConsumers;
          qreg[(2 * u) % (Q_IN_REGS ? QLD : 1)] = q_load_rd(i / IPR, 2 * (i % IPR));
          qreg[(2 * u + 1) % (Q_IN_REGS ? QLD : 1)] = q_load_rd(i / IPR, 2 * (i % IPR) + RHALF);
        }
#pragma unroll
        for (int it = 2 * RIT; it < (Q_IN_REGS ? QLD : 1); ++it) {
          const int idx = tid + (it - 2 * RIT) * kConsumers;
          qreg[it] = q_load_rd(idx / (PPR ? PPR : 1), NRD + 2 * (idx % (PPR ? PPR : 1)));
        }
      } else {
#pragma unroll
        for (int it = 0; it < (Q_IN_REGS ? QLD : 1); ++it) qreg[it] = q_load(tid + it * kConsumers);
      }
      if (own_new) {
        auto ld2 = [&](const void* src, uint64_t off) {
          float2 x = make_float2(0.f, 0.f);
          if (p.q_f16) x.x = __uint_as_float(*reinterpret_cast<const uint32_t*>(reinterpret_cast<const __half*>(src) + off));
          else x = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(src) + off);
          return x;
        };
        const uint64_t so = (uint64_t)p.items.col0[item] * p.k_new_stride + (uint64_t)g * HD + 2 * tid;
        const uint64_t sv = (uint64_t)p.items.col0[item] * p.v_new_stride + (uint64_t)g * HD + 2 * tid;
        if (HD == 256) { kx = ld2(p.k_new, so); vx = ld2(p.v_new, sv); }
        else {
          if (tid < 32) { kx = ld2(p.k_new, so); kxb = ld2(p.k_new, so + RHALF); }
          if (tid < HD / 2) vx = ld2(p.v_new, sv);
        }
      }
    } else {
#pragma unroll 8
      for (int it = 0; it < QLD; ++it) q_store(tid + it * kConsumers, act_cvt(q_load(tid + it * kConsumers)));
    }
  }
  // The producer warp sets up the barriers and goes; the consumers meet it at named barrier 2.  Named barrier 3
  // tells the producer that the q loads are in flight: a q load issued behind 190 KB of K/V tiles per SM queues
  // behind all of them at the memory controllers.  A call that may not fetch ahead of its predecessor waits there
  // before its first tile; one that may fetches `pre_stages` tiles first and the rest after it, so that the early
  // burst has drained by the time the small loads of the critical path (q here, the predecessor's last stores) go.
  if (warp == PW) {
    if (lane == 0) {
      *s_err = 0;
      const uint32_t full_count = g_list ? 32u : 1u;   // a TMA tile completes by bytes; a gathered one by its 32 lanes' copies
      for (uint32_t s = 0; s < 16; ++s) s_tile[s] = 0xffffffffu;
      for (uint32_t s = 0; s < NS; ++s) {
        mbar_init(kfull + 8 * s, full_count);
        mbar_init(vfull + 8 * s, full_count);
        mbar_init(kempty + 8 * s, 4);
        mbar_init(vempty + 8 * s, 4);
      }
      fence_barrier_init();
    }
    __syncwarp();
    named_bar_arrive(2, kDecThreads);
  } else {
    if (warp >= 4) pdl_wait();   // the second group reads shared memory only, but writes its records at the end
    named_bar_arrive(3, kDecThreads);
    named_bar_sync(2, kDecThreads);
  }

  if (warp == PW) {
    // ---------------------------------------------------------------- producer ----
    // the whole warp walks the loop (named barrier 3 wants all of it); lane 0 issues
    const uint32_t pre = p.prefetch_old_rows ? p.pre_stages : 0u;
    const int y0 = (int)(p.items.seq[item] * p.max_seq + tile0 * kT);
    const int z = (int)(g * CH);
    // rows below the ones this call's columns added, and below whatever the call before may still be writing
    const uint32_t old_rows = min(n_rows - min(n_rows, n_cols), p.early_limit);
    bool waited = !p.prefetch_old_rows;
    const uint64_t kv_policy = l2_policy_evict_first();
    if (lane == 0) {
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
    }
    if (g_list) {
      // ---- gathered rows: lane l copies the 16-byte chunks l, l + 32, ... of each listed row into the slot and swizzle
      //      a TMA tile would fill; rows past the list's end repeat its last row (their scores are masked, their V
      //      rows cleared, as for a tile that reaches past the sequence) ----
      __syncwarp();
      named_bar_sync(3, kDecThreads);
      pdl_wait();
      constexpr int CPR = HD / 8;                      // 16-byte chunks per row of one kv head
      const uint64_t seq_row0 = (uint64_t)p.items.seq[item] * p.max_seq;
      const uint32_t kvd = gridDim.y * HD;
      for (uint32_t i = 0; i < n_tiles; ++i) {
        const uint32_t s = i % NS, ph = (i / NS) & 1, tpos = (tile0 + i) * kT;
        const uint32_t ra = min(g_list[1 + min(tpos + lane, n_rows - 1)], p.max_seq - 1);
        const uint32_t rb = min(g_list[1 + min(tpos + 32 + lane, n_rows - 1)], p.max_seq - 1);
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          const uint32_t full = (which ? vfull : kfull) + 8 * s, empty = (which ? vempty : kempty) + 8 * s;
          if (lane == 0) { mbar_wait(empty, ph ^ 1, s_err, WAIT_EMPTY); s_tile[which * 8 + s] = i; }
          __syncwarp();
          const __half* cache = which ? p.v_cache : p.k_cache;
          const uint32_t dst0 = smem_u32((which ? v_slots : k_slots) + s * SLOT);
#pragma unroll 4
          for (uint32_t idx = lane; idx < kT * CPR; idx += 32) {
            const uint32_t r = idx / CPR, c16g = idx % CPR;
            const uint32_t row = __shfl_sync(0xffffffffu, r < 32 ? ra : rb, r & 31);
            const __half* src = cache + (seq_row0 + row) * kvd + (uint64_t)g * HD + c16g * 8;
            const uint32_t dst = dst0 + (c16g >> 3) * (kT * 128) + r * 128 + (((c16g & 7) ^ (r & 7)) << 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
          }
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(full) : "memory");
        }
      }
      asm volatile("cp.async.wait_all;" ::: "memory");   // nothing of this warp is in flight when it leaves
    } else
    for (uint32_t i = 0; i < n_tiles; ++i) {
      if (i == pre) {
        if (lane == 0 && p.prefetch_old_rows && p.own_prefetch) {
          // The first tiles are on their way into the ring; the CTA's other tiles of rows nobody can be writing are
          // asked into L2 now, while the predecessor kernel drains and this one waits for it: HBM works through the
          // kernel boundary, and the loads that refill the ring later find their tiles in L2.
          for (uint32_t k = pre; k < n_tiles && k < pre + p.own_prefetch && (tile0 + k + 1) * kT <= old_rows; ++k) {
            tma_prefetch_3d(&tm_k, 0, y0 + (int)(k * kT), z);
            tma_prefetch_3d(&tm_v, 0, y0 + (int)(k * kT), z);
          }
        }
        __syncwarp();
        named_bar_sync(3, kDecThreads);
        if (!p.prefetch_old_rows && lane == 0) pdl_wait();
      }
      if (lane == 0) {
        const uint32_t s = i % NS, ph = (i / NS) & 1;
        if (!waited && (tile0 + i + 1) * kT > old_rows) { pdl_wait(); waited = true; }
        mbar_wait(kempty + 8 * s, ph ^ 1, s_err, WAIT_EMPTY);
        s_tile[s] = i;
        mbar_expect_tx(kfull + 8 * s, SLOT);
        if (p.kv_evict_first) tma_load_3d_hint(smem_u32(k_slots + s * SLOT), &tm_k, 0, y0 + (int)(i * kT), z, kfull + 8 * s, kv_policy);
        else tma_load_3d(smem_u32(k_slots + s * SLOT), &tm_k, 0, y0 + (int)(i * kT), z, kfull + 8 * s);
        mbar_wait(vempty + 8 * s, ph ^ 1, s_err, WAIT_EMPTY);
        s_tile[8 + s] = i;
        mbar_expect_tx(vfull + 8 * s, SLOT);
        if (p.kv_evict_first) tma_load_3d_hint(smem_u32(v_slots + s * SLOT), &tm_v, 0, y0 + (int)(i * kT), z, vfull + 8 * s, kv_policy);
        else tma_load_3d(smem_u32(v_slots + s * SLOT), &tm_v, 0, y0 + (int)(i * kT), z, vfull + 8 * s);
      }
    }
    if (!g_list && n_tiles <= pre) { __syncwarp(); named_bar_sync(3, kDecThreads); }   // keeps the barrier balanced
    if (lane == 0 && p.next_tiles) {
      // Everything this CTA will read has been requested.  The engine's next layer call walks the same split of
      // another cache: ask L2 for its first tiles now, so that HBM keeps delivering while this kernel drains, the
      // combine runs and the next kernel starts up (a hint: nothing waits for it, and a line that is written later is
      // simply updated in L2).
      const int yn = (int)(p.items.seq[item] * p.next_max_seq + tile0 * kT);
      const uint32_t n_pf = min(p.next_tiles, n_tiles);
      for (uint32_t i = 0; i < n_pf; ++i) {
        tma_prefetch_3d(&tm_kn, 0, yn + (int)(i * kT), z);
        tma_prefetch_3d(&tm_vn, 0, yn + (int)(i * kT), z);
      }
    }
    if (lane == 0) {
      if (*s_err) {
        // a wait ran out somewhere: let the copies still in flight land (bounded) before the CTA exits
        const uint32_t first = n_tiles > NS ? n_tiles - NS : 0;
        for (uint32_t i = first; i < n_tiles; ++i) {
          const uint32_t s = i % NS, ph = (i / NS) & 1;
          for (uint32_t k = 0; k < (1u << 16) && !mbar_test(kfull + 8 * s, ph); ++k) __nanosleep(64);
          for (uint32_t k = 0; k < (1u << 16) && !mbar_test(vfull + 8 * s, ph); ++k) __nanosleep(64);
        }
        atomicMax(p.err, *s_err);
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers ----
  const int w = warp & 3, r = lane >> 2, j = lane & 3;
  const int ltid = tid - grp * kConsumers;       // thread within its consumer group
  const uint32_t gbar = grp ? 4u : 1u;           // the group's own named barrier

  if (Q_IN_REGS && grp == 0) {
    if (own_new) { kx = act_cvt(kx); vx = act_cvt(vx); kxb = act_cvt(kxb); }
    if (fused) {
#pragma unroll
      for (int u = 0; u < RIT; ++u) {
        const int i = tid + u * kConsumers, row = i / IPR, b2 = 2 * (i % IPR);
        if ((uint32_t)row >= live_rows) {   // padding rows of the tile: zeros, no arithmetic
          q_store_rd(row, b2, make_float2(0.f, 0.f)); q_store_rd(row, b2 + RHALF, make_float2(0.f, 0.f));
          continue;
        }
        const float2 a = act_cvt(qreg[(2 * u) % (Q_IN_REGS ? QLD : 1)]), b = act_cvt(qreg[(2 * u + 1) % (Q_IN_REGS ? QLD : 1)]);
        float2 ra, rb;   // the bits of the float64 expression the stand-alone RoPE kernel evaluates
        ra.x = rot_exact(a.x, b.x, s_ang[b2], true);
        ra.y = rot_exact(a.y, b.y, s_ang[b2 + 1], true);
        rb.x = rot_exact(b.x, a.x, s_ang[b2], false);
        rb.y = rot_exact(b.y, a.y, s_ang[b2 + 1], false);
        q_store_rd(row, b2, ra);
        q_store_rd(row, b2 + RHALF, rb);
      }
#pragma unroll
      for (int it = 2 * RIT; it < (Q_IN_REGS ? QLD : 1); ++it) {
        const int idx = tid + (it - 2 * RIT) * kConsumers, rr = idx / (PPR ? PPR : 1), d = NRD + 2 * (idx % (PPR ? PPR : 1));
        if (p.q_f16) {   // unrotated f16 values are their own high parts: the loaded bits go in as they are
          *reinterpret_cast<uint32_t*>(q_hi + rr * QP + d * 2) = __float_as_uint(qreg[it].x);
          if (PRECISE) *reinterpret_cast<uint32_t*>(q_lo + rr * QP + d * 2) = 0u;
        } else {
          q_store_rd(rr, d, qreg[it]);
        }
      }
      if (own_new && w == 0) {
        if (HD == 256) kx = rotate(kx);
        else {
          const int b2 = 2 * lane;
          const float2 a = kx, b = kxb;
          kx.x = rot_exact(a.x, b.x, s_ang[b2], true);   kx.y = rot_exact(a.y, b.y, s_ang[b2 + 1], true);
          kxb.x = rot_exact(b.x, a.x, s_ang[b2], false); kxb.y = rot_exact(b.y, a.y, s_ang[b2 + 1], false);
        }
      }
    } else {
#pragma unroll
      for (int it = 0; it < (Q_IN_REGS ? QLD : 1); ++it) q_store(tid + it * kConsumers, act_cvt(qreg[it]));
    }
    if (own_new) {
      auto h16 = [](float x) -> uint32_t {   // round to nearest even; NaN -> sign | 0x7e00, as the append kernel
        return x != x ? (((__float_as_uint(x) >> 16) & 0x8000u) | 0x7e00u) : (uint32_t)__half_as_ushort(__float2half_rn(x));
      };
      k_new2 = h16(kx.x) | (h16(kx.y) << 16);
      k_new2b = h16(kxb.x) | (h16(kxb.y) << 16);
      v_new2 = h16(vx.x) | (h16(vx.y) << 16);
      // the row also goes to shared memory: the group that takes the sequence's last tile places it there
      if (HD == 256) { s_newk[tid] = k_new2; s_newv[tid] = v_new2; }
      else { if (tid < 32) { s_newk[tid] = k_new2; s_newk[tid + 32] = k_new2b; } if (tid < HD / 2) s_newv[tid] = v_new2; }
      const uint64_t ro = ((uint64_t)p.items.seq[item] * p.max_seq + (n_rows - 1)) * ((uint64_t)gridDim.y * HD) + (uint64_t)g * HD + 2 * tid;
      if (HD == 256) {
        *reinterpret_cast<uint32_t*>(p.k_cache + ro) = k_new2;
        *reinterpret_cast<uint32_t*>(p.v_cache + ro) = v_new2;
      } else {
        if (tid < 32) { *reinterpret_cast<uint32_t*>(p.k_cache + ro) = k_new2; *reinterpret_cast<uint32_t*>(p.k_cache + ro + RHALF) = k_new2b; }
        if (tid < HD / 2) *reinterpret_cast<uint32_t*>(p.v_cache + ro) = v_new2;
      }
    }
  }

  // causal limit of the two rows this thread owns in every 8-row group
  uint32_t lim[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      uint32_t row = nt * 8 + 2 * j + e;
      const int32_t c = (int32_t)min(row / G, n_cols - 1);
      lim[nt][e] = (uint32_t)min(max(p.items.lim0[item] + c, 0), (int32_t)n_rows);
    }

  float m_run[NT][2], l_run[NT][2];
  float oacc[MT][NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    m_run[nt][0] = m_run[nt][1] = -3.0e38f;
    l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) oacc[mt][nt][e] = 0.f;
  }
  named_bar_sync(5, CONS);   // q (and the token's own row) visible to both groups

  const uint32_t q_hi_s = smem_u32(q_hi), q_lo_s = smem_u32(q_lo), p_hi_s = smem_u32(p_hi), p_lo_s = smem_u32(p_lo);
  // the slot is this group's turn once the producer has put the tile's number on it (bounded like every wait)
  auto wait_tile = [&](uint32_t word, uint32_t i) {
    if (NG == 1) return;
    for (uint32_t k = 0; s_tile[word] != i && !*s_err; ++k) {
      if (k > kWaitPolls) { *s_err = WAIT_KFULL; break; }
      if (k > 16) __nanosleep(32);
    }
  };

  // With one 8-row group the query fragments of all k-steps (hi and lo: HD/4 registers) stay in registers for the
  // CTA's life: re-reading them from shared memory for every tile was half of the score product's fragment loads.
  constexpr bool Q_FRAGS = NT == 1;
  uint32_t qfh[Q_FRAGS ? HD / 32 : 1][4], qfl[Q_FRAGS ? HD / 32 : 1][4];
  if constexpr (Q_FRAGS) {
#pragma unroll
    for (int k2 = 0; k2 < HD / 32; ++k2) {
      const uint32_t qoff = (lane & 7) * QP + (4 * k2 + (lane >> 3)) * 16;
      ldsm_x4(q_hi_s + qoff, qfh[k2][0], qfh[k2][1], qfh[k2][2], qfh[k2][3]);
      if (PRECISE) ldsm_x4(q_lo_s + qoff, qfl[k2][0], qfl[k2][1], qfl[k2][2], qfl[k2][3]);
    }
  }
  for (uint32_t i = grp; i < n_tiles; i += NG) {
    const uint32_t s = i % NS, ph = (i / NS) & 1;
    const uint32_t tile_pos = (tile0 + i) * kT;
    const uint32_t ks_base = smem_u32(k_slots + s * SLOT), vs_base = smem_u32(v_slots + s * SLOT);

    // ---- S^T = K . Q^T for positions 16w .. 16w+15 ----
    // NA independent accumulator sets per row group: with one, the 2 * HD/16 MMAs of a group form a single
    // dependency chain and the tensor pipe idles between them
    constexpr int NA = NT >= 4 ? 1 : 4 / NT;
    float sacc[NT][4], sacc_x[NT][NA > 1 ? NA - 1 : 1][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
      for (int a = 0; a < NA - 1; ++a) sacc_x[nt][a][0] = sacc_x[nt][a][1] = sacc_x[nt][a][2] = sacc_x[nt][a][3] = 0.f;
    }
    wait_tile(s, i);
    mbar_wait(kfull + 8 * s, ph, s_err, WAIT_KFULL);
    if (own_new && i == n_tiles - 1) {
      const uint32_t rr = n_rows - 1 - tile_pos;
      auto word_at = [&](uint8_t* slots, uint32_t wi) {   // 32-bit word wi of row rr in the swizzled tile
        const uint32_t c16g = wi >> 2;
        return reinterpret_cast<uint32_t*>(slots + s * SLOT + (c16g >> 3) * (kT * 128) + rr * 128 + (((c16g & 7) ^ (rr & 7)) << 4) + (wi & 3) * 4);
      };
      if (ltid < HD / 2) *word_at(k_slots, ltid) = s_newk[ltid];
      named_bar_sync(gbar, kConsumers);
    }
    if constexpr (NT <= 2) {
      // Software-pipelined: the fragments of step k2 + 1 are requested before the MMAs of step k2 are issued, so
      // the shared-memory latency of one step hides behind the tensor work of the other (one warp per scheduler:
      // nothing else would hide it).
      const uint32_t krow = 16 * w + (lane & 7) + ((lane >> 3) & 1) * 8;
      uint32_t a[2][2][4], bh[2][NT][4], bl[2][NT][4];
      auto load_step = [&](int k2, int buf) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t c16g = (2 * k2 + e) * 2 + (lane >> 4);
          const uint32_t addr = ks_base + (c16g >> 3) * (kT * 128) + krow * 128 + (((c16g & 7) ^ (krow & 7)) << 4);
          ldsm_x4(addr, a[buf][e][0], a[buf][e][1], a[buf][e][2], a[buf][e][3]);
        }
        if constexpr (!Q_FRAGS) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint32_t qoff = (nt * 8 + (lane & 7)) * QP + (4 * k2 + (lane >> 3)) * 16;
            ldsm_x4(q_hi_s + qoff, bh[buf][nt][0], bh[buf][nt][1], bh[buf][nt][2], bh[buf][nt][3]);
            if (PRECISE) ldsm_x4(q_lo_s + qoff, bl[buf][nt][0], bl[buf][nt][1], bl[buf][nt][2], bl[buf][nt][3]);
          }
        }
      };
      load_step(0, 0);
#pragma unroll
      for (int k2 = 0; k2 < HD / 32; ++k2) {
        const int cur = k2 & 1;
        if (k2 + 1 < HD / 32) load_step(k2 + 1, cur ^ 1);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t* qh = Q_FRAGS ? qfh[k2] : bh[cur][nt];
          const uint32_t* ql = Q_FRAGS ? qfl[k2] : bl[cur][nt];
          mma_16816(sacc[nt], a[cur][0][0], a[cur][0][1], a[cur][0][2], a[cur][0][3], qh[0], qh[1]);
          mma_16816(NA >= 2 ? sacc_x[nt][0] : sacc[nt], a[cur][1][0], a[cur][1][1], a[cur][1][2], a[cur][1][3], qh[2], qh[3]);
          if (PRECISE) {
            mma_16816(NA >= 4 ? sacc_x[nt][1] : sacc[nt], a[cur][0][0], a[cur][0][1], a[cur][0][2], a[cur][0][3], ql[0], ql[1]);
            mma_16816(NA >= 4 ? sacc_x[nt][2] : (NA >= 2 ? sacc_x[nt][0] : sacc[nt]), a[cur][1][0], a[cur][1][1], a[cur][1][2], a[cur][1][3],
                      ql[2], ql[3]);
          }
        }
      }
    } else
    {
      const uint32_t krow = 16 * w + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll 4
      for (int k2 = 0; k2 < HD / 32; ++k2) {
        uint32_t a[2][4];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t c16g = (2 * k2 + e) * 2 + (lane >> 4);
          const uint32_t addr = ks_base + (c16g >> 3) * (kT * 128) + krow * 128 + (((c16g & 7) ^ (krow & 7)) << 4);
          ldsm_x4(addr, a[e][0], a[e][1], a[e][2], a[e][3]);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t qoff = (nt * 8 + (lane & 7)) * QP + (4 * k2 + (lane >> 3)) * 16;
          uint32_t b0, b1, b2, b3;
          ldsm_x4(q_hi_s + qoff, b0, b1, b2, b3);
          mma_16816(sacc[nt], a[0][0], a[0][1], a[0][2], a[0][3], b0, b1);
          mma_16816(NA >= 2 ? sacc_x[nt][0] : sacc[nt], a[1][0], a[1][1], a[1][2], a[1][3], b2, b3);
          if (PRECISE) {
            ldsm_x4(q_lo_s + qoff, b0, b1, b2, b3);
            mma_16816(NA >= 4 ? sacc_x[nt][1] : sacc[nt], a[0][0], a[0][1], a[0][2], a[0][3], b0, b1);
            mma_16816(NA >= 4 ? sacc_x[nt][2] : (NA >= 2 ? sacc_x[nt][0] : sacc[nt]), a[1][0], a[1][1], a[1][2], a[1][3], b2, b3);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(kempty + 8 * s);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int a = 0; a < NA - 1; ++a)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[nt][e] += sacc_x[nt][a][e];

    // ---- scale, causal mask, tile maximum per row ----
    const uint32_t pos_a = tile_pos + 16 * w + r, pos_b = pos_a + 8;
    float tmax[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float sa = sacc[nt][e] * p.scale_log2, sb = sacc[nt][2 + e] * p.scale_log2;
        sa = pos_a < lim[nt][e] ? sa : -INFINITY;
        sb = pos_b < lim[nt][e] ? sb : -INFINITY;
        sacc[nt][e] = sa; sacc[nt][2 + e] = sb;
        float mx = fmaxf(sa, sb);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        tmax[nt][e] = mx;
      }
      if (r == 0) { s_max[w * ROWS + nt * 8 + 2 * j] = tmax[nt][0]; s_max[w * ROWS + nt * 8 + 2 * j + 1] = tmax[nt][1]; }
    }
    named_bar_sync(gbar, kConsumers);

    // ---- new running maximum, weights P = 2^(s - m), rescale factor ----
    float alpha[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int row = nt * 8 + 2 * j + e;
        float mn = m_run[nt][e];
        mn = fmaxf(mn, fmaxf(fmaxf(s_max[row], s_max[ROWS + row]), fmaxf(s_max[2 * ROWS + row], s_max[3 * ROWS + row])));
        alpha[nt][e] = exp2f(m_run[nt][e] - mn);
        m_run[nt][e] = mn;
        const float pa = exp2f(sacc[nt][e] - mn), pb = exp2f(sacc[nt][2 + e] - mn);
        sacc[nt][e] = pa; sacc[nt][2 + e] = pb;
        l_run[nt][e] = l_run[nt][e] * alpha[nt][e] + (pa + pb);
      }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      // P^T[pos][row]: this thread holds rows 2j, 2j+1 of group nt at positions 16w+r and 16w+r+8
      const uint32_t o_a = (16 * w + r) * PP + (nt * 8 + 2 * j) * 2, o_b = o_a + 8 * PP;
      __half ha0, la0, ha1, la1, hb0, lb0, hb1, lb1;
      split_h(sacc[nt][0], ha0, la0); split_h(sacc[nt][1], ha1, la1);
      split_h(sacc[nt][2], hb0, lb0); split_h(sacc[nt][3], hb1, lb1);
      *reinterpret_cast<__half2*>(p_hi + o_a) = __halves2half2(ha0, ha1);
      *reinterpret_cast<__half2*>(p_hi + o_b) = __halves2half2(hb0, hb1);
      if (PRECISE) {
        *reinterpret_cast<__half2*>(p_lo + o_a) = __halves2half2(la0, la1);
        *reinterpret_cast<__half2*>(p_lo + o_b) = __halves2half2(lb0, lb1);
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        oacc[mt][nt][0] *= alpha[nt][0]; oacc[mt][nt][1] *= alpha[nt][1];
        oacc[mt][nt][2] *= alpha[nt][0]; oacc[mt][nt][3] *= alpha[nt][1];
      }

    wait_tile(8 + s, i);
    mbar_wait(vfull + 8 * s, ph, s_err, WAIT_VFULL);
    if (own_new && i == n_tiles - 1 && ltid < HD / 2) {   // made visible by the barrier below
      const uint32_t rr = n_rows - 1 - tile_pos, c16g = ltid >> 2;
      *reinterpret_cast<uint32_t*>(v_slots + s * SLOT + (c16g >> 3) * (kT * 128) + rr * 128 + (((c16g & 7) ^ (rr & 7)) << 4) + (ltid & 3) * 4) = s_newv[ltid];
    }
    if (tile_pos + kT > n_rows) {
      // rows of the tile past the sequence end hold whatever the cache holds there (possibly NaN):
      // their weights are zero, but 0 * NaN is NaN, so clear them
      const uint32_t nv = n_rows - tile_pos;
      for (uint32_t idx = ltid; idx < (kT - nv) * (HD / 8); idx += kConsumers) {
        const uint32_t row = nv + idx / (HD / 8), c16g = idx % (HD / 8);
        *reinterpret_cast<uint4*>(v_slots + s * SLOT + (c16g >> 3) * (kT * 128) + row * 128 + (((c16g & 7) ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
      }
    }
    named_bar_sync(gbar, kConsumers);   // P (and the cleared rows) visible to every warp of the group

    // ---- O^T += V^T . P^T, dims (w*MT + mt)*16 .. +15 ----
    if constexpr (NT <= 2) {
      // pipelined like the score product: step t = (ks, mt); V fragments of step t + 1 and the P fragments of the
      // next ks are requested before the MMAs of step t
      constexpr int STEPS = (kT / 16) * MT;
      uint32_t av[2][4], pbh[2][NT][2], pbl[2][NT][2];
      auto load_p = [&](int ks, int buf) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t poff = (ks * 16 + (lane & 15)) * PP + nt * 16;
          ldsm_x2_t(p_hi_s + poff, pbh[buf][nt][0], pbh[buf][nt][1]);
          if (PRECISE) ldsm_x2_t(p_lo_s + poff, pbl[buf][nt][0], pbl[buf][nt][1]);
        }
      };
      auto load_v = [&](int t, int buf) {
        const int ks = t / MT, mt = t % MT;
        const uint32_t qd = lane >> 3;
        const uint32_t vrow = ks * 16 + (lane & 7) + (qd >> 1) * 8;
        const uint32_t c16g = (w * MT + mt) * 2 + (qd & 1);
        const uint32_t addr = vs_base + (c16g >> 3) * (kT * 128) + vrow * 128 + (((c16g & 7) ^ (vrow & 7)) << 4);
        ldsm_x4_t(addr, av[buf][0], av[buf][1], av[buf][2], av[buf][3]);
      };
      load_p(0, 0);
      load_v(0, 0);
#pragma unroll
      for (int t = 0; t < STEPS; ++t) {
        const int ks = t / MT, mt = t % MT, cur = t & 1, pc = ks & 1;
        if (t + 1 < STEPS) {
          if ((t + 1) % MT == 0) load_p(ks + 1, pc ^ 1);
          load_v(t + 1, cur ^ 1);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_16816(oacc[mt][nt], av[cur][0], av[cur][1], av[cur][2], av[cur][3], pbh[pc][nt][0], pbh[pc][nt][1]);
          if (PRECISE) mma_16816(oacc[mt][nt], av[cur][0], av[cur][1], av[cur][2], av[cur][3], pbl[pc][nt][0], pbl[pc][nt][1]);
        }
      }
    } else
#pragma unroll
    for (int ks = 0; ks < kT / 16; ++ks) {
      uint32_t bh[NT][2], bl[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint32_t poff = (ks * 16 + (lane & 15)) * PP + nt * 16;
        ldsm_x2_t(p_hi_s + poff, bh[nt][0], bh[nt][1]);
        if (PRECISE) ldsm_x2_t(p_lo_s + poff, bl[nt][0], bl[nt][1]);
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint32_t qd = lane >> 3;
        const uint32_t vrow = ks * 16 + (lane & 7) + (qd >> 1) * 8;
        const uint32_t c16g = (w * MT + mt) * 2 + (qd & 1);
        const uint32_t addr = vs_base + (c16g >> 3) * (kT * 128) + vrow * 128 + (((c16g & 7) ^ (vrow & 7)) << 4);
        uint32_t a0, a1, a2, a3;
        ldsm_x4_t(addr, a0, a1, a2, a3);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_16816(oacc[mt][nt], a0, a1, a2, a3, bh[nt][0], bh[nt][1]);
          if (PRECISE) mma_16816(oacc[mt][nt], a0, a1, a2, a3, bl[nt][0], bl[nt][1]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(vempty + 8 * s);
  }

  // ---- partial (o, m, l) per row ----
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float l = l_run[nt][e];
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      if (r == 0) s_l[w * ROWS + nt * 8 + 2 * j + e] = l;
    }
  named_bar_sync(gbar, kConsumers);
  // ---- one record per (row, split).  The rows' o go through shared memory (the ring is idle now) so that the record
  //      stores are whole 16-byte vectors of consecutive addresses; with two groups, the second leaves its (o, m, l)
  //      there and the first folds it into its own: o = o0 2^(m0 - M) + o1 2^(m1 - M), likewise l ----
  float* xo = reinterpret_cast<float*>(k_slots);       // [ROWS][HD]
  float* xml = xo + ROWS * HD;                         // [ROWS][2]: m (log2 units), l as the second group leaves them
  float* xml_out = xml + 2 * ROWS;                     // [ROWS][2]: the record's m and l
  float l_row[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const uint32_t row = nt * 8 + 2 * j + e;
      l_row[nt][e] = (s_l[row] + s_l[ROWS + row]) + (s_l[2 * ROWS + row] + s_l[3 * ROWS + row]);
    }
  auto put_rows = [&](bool fold, float* ml_dst) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const uint32_t row = nt * 8 + 2 * j + e;
        float w0 = 1.f, w1 = 0.f, M = m_run[nt][e];
        if (fold) {
          const float m1 = xml[row * 2];
          M = fmaxf(M, m1);
          w0 = exp2f(m_run[nt][e] - M); w1 = exp2f(m1 - M);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int d = (w * MT + mt) * 16 + r;
          float a = oacc[mt][nt][e], b = oacc[mt][nt][2 + e];
          if (fold) { a = a * w0 + xo[row * HD + d] * w1; b = b * w0 + xo[row * HD + d + 8] * w1; }
          xo[row * HD + d] = a; xo[row * HD + d + 8] = b;
        }
        if (w == 0 && r == 0) {
          const float l = fold ? l_row[nt][e] * w0 + xml[row * 2 + 1] * w1 : l_row[nt][e];
          ml_dst[row * 2] = M; ml_dst[row * 2 + 1] = l;
        }
      }
  };
  if constexpr (NG == 2) {
    named_bar_sync(5, CONS);                 // both groups are past their last tile: nobody reads the ring any more
    if (grp == 1) put_rows(false, xml);
    named_bar_sync(5, CONS);
    if (grp == 1) return;                    // the first group carries on alone
    put_rows(true, xml_out);
  } else {
    put_rows(false, xml_out);
  }
  named_bar_sync(gbar, kConsumers);
  for (uint32_t idx = ltid; idx < live_rows * (HD / 4); idx += kConsumers) {
    const uint32_t row = idx / (HD / 4), c4 = idx % (HD / 4);
    const uint32_t c = row / G, hh = row % G;
    const uint64_t prow = (uint64_t)(p.items.col0[item] + c) * p.n_heads + g * G + hh;
    const uint64_t slot = prow * p.n_splits + split;
    reinterpret_cast<float4*>(p.part_o + slot * HD)[c4] = reinterpret_cast<const float4*>(xo + row * HD)[c4];
    if (c4 == 0) {
      p.part_ml[slot * 2] = xml_out[row * 2] * 0.6931471805599453f;
      p.part_ml[slot * 2 + 1] = xml_out[row * 2 + 1];
    }
  }
  if constexpr (NT <= 2) if (p.merge) {
    // ---- one kernel per call: when every CTA of this (item, kv head) has left its record, the CTAs share out the
    //      merge: (query row, 64-dim slice) units, dealt round-robin; LSE merge, gate and store as pa_combine_kernel does.
    //      All CTAs of the launch are resident together (the host checks that the grid fits the GPU in one wave), so
    //      the wait below is for CTAs that are running; it is bounded all the same. ----
    const uint32_t ns_live = (tiles + tps - 1) / tps;             // CTAs of this (item, kv head) that hold tiles
    const uint32_t n_units = live_rows * (HD / 64);
    unsigned int* ctr = p.merge_ctr + 2 * ((size_t)item * gridDim.y + g);   // [0] records left, [1] CTAs done merging
    // the gate value of this CTA's first unit is requested now and has landed by the time the records may be read
    float gv0 = 0.f;
    const bool gated = p.gate != nullptr;
    auto unit_addr = [&](uint32_t u, uint64_t& prow, uint32_t& slice, uint64_t& go, uint64_t& oo) {
      const uint32_t row = u / (HD / 64); slice = u % (HD / 64);
      const uint32_t c = row / G, hh = row % G, col = p.items.col0[item] + c, h = g * G + hh;
      prow = (uint64_t)col * p.n_heads + h;
      go = (uint64_t)col * p.gate_col_stride + (uint64_t)h * p.gate_head_stride + slice * 64;
      oo = (uint64_t)col * p.out_col_stride + (uint64_t)h * HD + slice * 64;
    };
    auto gate_ld = [&](uint64_t go) {
      return p.act_f16 ? __half2float(reinterpret_cast<const __half*>(p.gate)[go + ltid]) : reinterpret_cast<const float*>(p.gate)[go + ltid];
    };
    if (split < n_units && gated && ltid < 64) {
      uint64_t prow, go, oo; uint32_t slice;
      unit_addr(split, prow, slice, go, oo);
      gv0 = gate_ld(go);
    }
    // A CTA that holds no merge unit counts itself in and leaves at once: its SM is free for the next kernel's CTA
    // (p.merge == 1: every CTA waits for the records, for comparison).  The fence stays in every thread: a single one
    // in the counting thread behind the barrier measured slower.
    const bool has_units = split < n_units || p.merge == 1;
    __threadfence();                       // this thread's record stores, device-wide
    named_bar_sync(gbar, kConsumers);
    if (ltid == 0) {
      atomicAdd(ctr, 1u);
      if (has_units) {
        uint32_t polls = 0;
        while (*reinterpret_cast<volatile unsigned int*>(ctr) < ns_live && !*s_err) {
          if (++polls > (1u << 20)) { *s_err = WAIT_MERGE; break; }
          if (polls > 8) __nanosleep(64);
        }
        __threadfence();
      }
    }
    if (has_units) named_bar_sync(gbar, kConsumers);
    MergeScratch& sc = *reinterpret_cast<MergeScratch*>(k_slots);   // the ring is idle: every tile has been consumed
    if (!*s_err) {
      for (uint32_t u = split; u < n_units; u += ns_live) {
        uint64_t prow, go, oo; uint32_t slice;
        unit_addr(u, prow, slice, go, oo);
        const float gv = (u == split) ? gv0 : ((gated && ltid < 64) ? gate_ld(go) : 0.f);
        const uint64_t rec0 = prow * p.n_splits;
        merge_slice_128<HD>(p.part_o + rec0 * HD, p.part_ml + rec0 * 2, ns_live, slice, ltid, sc, gbar, gated, gv, p.gather != nullptr, p.act_f16, p.out, oo);
      }
    }
    // the last CTA to finish clears the counters for the next call (every other CTA is past its wait by then)
    if (ltid == 0 && atomicAdd(ctr + 1, 1u) == ns_live - 1) { ctr[0] = 0; ctr[1] = 0; }
  }
  if (*s_err && tid == 0) atomicMax(p.err, *s_err);
}

// the exchange's call counter for a call whose decode kernel does not run (a shard that holds no row of the call) or
// is the tensor-core verify kernel
__global__ void pa_epoch_bump_kernel(unsigned int* ctr) {
  pdl_wait();
  pdl_trigger();
  atomicAdd(ctr, 1u);
}
cudaError_t launch_epoch_bump(unsigned int* ctr, cudaStream_t st) { return launch_pdl(pa_epoch_bump_kernel, dim3(1), dim3(1), 0, st, ctr); }

// ------------------------------------------------------------------------------ combine --


// grid (query rows, HD / 64): one CTA per (column, head, 64-dim slice).  Every thread fetches the (m, l) of up to two
// splits while 16 groups of 16 lanes (a float4 each) fetch the o records, splits 16 apart, eight loads in flight per
// lane; the weights are applied when both have arrived.  Every sum has a fixed order.
template <int HD, bool XCH>
__global__ void __launch_bounds__(256) pa_combine_kernel(const CombineParams p) {
  __shared__ float s_w[512];
  __shared__ float s_red[8], s_red2[8];
  __shared__ float4 s_acc[16][16];
  const uint32_t prow = blockIdx.x, slice = blockIdx.y, col = prow / p.n_heads, h = prow % p.n_heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();      // the partial records belong to the kernel before this one
  pdl_trigger();
  uint32_t xepoch = 0;   // the exchange's call counter: requested with everything else
  if constexpr (XCH) xepoch = *reinterpret_cast<volatile unsigned int*>(p.xc.ctr);
  uint32_t ns = p.fixed_parts;
  if (ns == 0) {
    uint32_t it = 0;
    for (uint32_t i = 0; i < p.n_items; ++i) if (col >= p.items.col0[i]) it = i;
    // gather: one column per item, its length on the device; the plan is the one the decode kernel derived from it
    const uint32_t n_rows = p.gather ? min(p.gather[(size_t)col * p.gather_stride], p.gather_stride - 1u) : p.items.n_rows[it];
    const uint32_t tiles = (n_rows + kT - 1) / kT;
    const uint32_t n_sp = min(p.n_splits, max(1u, tiles / 2));
    const uint32_t tps = (tiles + n_sp - 1) / max(n_sp, 1u);
    ns = tiles ? ((tiles + tps - 1) / tps) * p.groups : 0;   // a shard that holds no row of the item: an empty record
  }
  // Everything the CTA reads is requested before the first use: the (m, l) pairs, the o records of the first 128
  // splits (eight float4 per lane, splits 16 apart) and the gate value.  One memory round trip instead of three.
  const float* ml = p.ml + prow * p.ml_row_stride;
  const int grp = tid >> 4, ln = tid & 15;
  const float* ob = p.o + prow * p.o_row_stride + slice * 64 + ln * 4;
  const uint32_t d = slice * 64 + tid;
  float gv = 0.f;
  const bool gated = p.gate && tid < 64 && !p.partial_out;
  if (gated) {
    const uint64_t go = (uint64_t)col * p.gate_col_stride + (uint64_t)h * p.gate_head_stride + d;
    gv = p.act_f16 ? __half2float(reinterpret_cast<const __half*>(p.gate)[go]) : reinterpret_cast<const float*>(p.gate)[go];
  }
  float m0 = -3.0e38f, l0 = 0.f, m1 = -3.0e38f, l1 = 0.f;
  if ((uint32_t)tid < ns) { m0 = ml[tid * p.ml_part_stride]; l0 = ml[tid * p.ml_part_stride + 1]; }
  if ((uint32_t)tid + 256 < ns) { m1 = ml[(tid + 256) * p.ml_part_stride]; l1 = ml[(tid + 256) * p.ml_part_stride + 1]; }
  float4 x8[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const uint32_t s = grp + 16 * u;
    x8[u] = s < ns ? *reinterpret_cast<const float4*>(ob + s * p.o_part_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float M = fmaxf(m0, m1);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  if (lane == 0) s_red[warp] = M;
  __syncthreads();
  M = s_red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) M = fmaxf(M, s_red[i]);
  const float w0 = (uint32_t)tid < ns ? __expf(m0 - M) : 0.f, w1 = (uint32_t)tid + 256 < ns ? __expf(m1 - M) : 0.f;
  s_w[tid] = w0; s_w[tid + 256] = w1;
  float Lp = __fmaf_rn(l1, w1, __fmul_rn(l0, w0));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) Lp = __fadd_rn(Lp, __shfl_xor_sync(0xffffffffu, Lp, o));
  if (lane == 0) s_red2[warp] = Lp;
  __syncthreads();
  float Lsum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) Lsum = __fadd_rn(Lsum, s_red2[i]);

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const uint32_t s = grp + 16 * u;
    const float wgt = s < ns ? s_w[s] : 0.f;
    fma4(acc, x8[u], wgt);
  }
  for (uint32_t s0 = grp + 128; s0 < ns; s0 += 64) {
    float4 x[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t s = s0 + 16 * u;
      x[u] = s < ns ? *reinterpret_cast<const float4*>(ob + s * p.o_part_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t s = s0 + 16 * u;
      const float wgt = s < ns ? s_w[s] : 0.f;
      fma4(acc, x[u], wgt);
    }
  }
  s_acc[grp][ln] = acc;
  __syncthreads();
  float t = 0.f;
  if (tid < 64) {
    const float* sa = reinterpret_cast<const float*>(s_acc);
    t = sa[tid];
#pragma unroll
    for (int i = 1; i < 16; ++i) t = __fadd_rn(t, sa[i * 64 + tid]);
  }
  if constexpr (XCH) {
    exchange_slice<HD>(p.xc, prow, slice, tid, t, M, Lsum, p.xch_sweeps, p.err, xepoch);
  }
  if (tid < 64) {
    if (p.partial_out) {
      p.partial_out[(uint64_t)prow * HD + d] = t;
      if (d == 0) {
        float* mlo = p.partial_out + p.partial_rows * HD + (uint64_t)prow * 2;
        mlo[0] = M; mlo[1] = Lsum;
      }
      return;
    }
    float rv = (p.gather && Lsum == 0.f) ? 0.f : __fdiv_rn(t, Lsum);   // an empty list attends nothing
    if (gated) rv = __fmul_rn(rv, __fdiv_rn(1.0f, __fadd_rn(1.0f, __expf(-gv))));
    const uint64_t oo = (uint64_t)col * p.out_col_stride + (uint64_t)h * HD + d;
    if (p.act_f16) reinterpret_cast<__half*>(p.out)[oo] = __float2half_rn(rv);
    else reinterpret_cast<float*>(p.out)[oo] = rv;
  }
}

// ------------------------------------------------------------------------------ launchers --

template <int HD, int NT, bool PRECISE>
static cudaError_t launch_decode_t(const pa_layer* L, const DecodeParams& p, dim3 grid, cudaStream_t st) {
  using S = DecSmem<HD, NT, PRECISE>;
  DecodeParams pp = p;
  int stages = S::stages_for(L->ctx->smem_optin);
  if (stages < 2) return cudaErrorInvalidConfiguration;
  pp.n_stages = (uint32_t)stages;
  const int bytes = S::total_bytes(stages);
  static bool attr_set[64] = {};
  if (pp.gather && (!pp.k_cache || !pp.v_cache)) return cudaErrorInvalidValue;
  auto kern = pa_decode_kernel<HD, NT, PRECISE>;
  const int dev = L->ctx->device & 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const pa_layer* N = L->next;
  if (!N || !pp.next_tiles || N->n_seqs != L->n_seqs) { N = L; pp.next_tiles = 0; }
  pp.next_max_seq = N->max_seq;
  return launch_pdl(kern, grid, dim3(S::THREADS), (size_t)bytes, st, L->tm_k64, L->tm_v64, N->tm_k64, N->tm_v64, pp);
}

template <int HD, bool PRECISE>
static cudaError_t launch_decode_nt(const pa_layer* L, const DecodeParams& p, dim3 grid, int nt, cudaStream_t st) {
  switch (nt) {
    case 1: return launch_decode_t<HD, 1, PRECISE>(L, p, grid, st);
    case 2: return launch_decode_t<HD, 2, PRECISE>(L, p, grid, st);
    case 3: case 4: return launch_decode_t<HD, 4, PRECISE>(L, p, grid, st);
    default: return launch_decode_t<HD, 8, PRECISE>(L, p, grid, st);
  }
}

cudaError_t launch_decode(const pa_layer* L, const DecodeParams& p, dim3 grid, int nt, cudaStream_t st) {
  const bool precise = !(L->ctx->cfg.flags & PA_FLAG_FAST);
  if (L->ctx->cfg.head_dim == 256) return precise ? launch_decode_nt<256, true>(L, p, grid, nt, st) : launch_decode_nt<256, false>(L, p, grid, nt, st);
  if (L->ctx->cfg.head_dim == 128) return precise ? launch_decode_nt<128, true>(L, p, grid, nt, st) : launch_decode_nt<128, false>(L, p, grid, nt, st);
  if (L->ctx->cfg.head_dim == 64) return precise ? launch_decode_nt<64, true>(L, p, grid, nt, st) : launch_decode_nt<64, false>(L, p, grid, nt, st);
  return cudaErrorInvalidValue;
}

cudaError_t launch_combine(int head_dim, const CombineParams& p, uint32_t rows, cudaStream_t st) {
  // the cross-GPU exchange is its own instantiation: its registers would halve the occupancy of the plain merge
  if (head_dim == 256) return p.exchange ? launch_pdl(pa_combine_kernel<256, true>, dim3(rows, 4), dim3(256), 0, st, p)
                                         : launch_pdl(pa_combine_kernel<256, false>, dim3(rows, 4), dim3(256), 0, st, p);
  if (head_dim == 128) return p.exchange ? launch_pdl(pa_combine_kernel<128, true>, dim3(rows, 2), dim3(256), 0, st, p)
                                         : launch_pdl(pa_combine_kernel<128, false>, dim3(rows, 2), dim3(256), 0, st, p);
  if (head_dim == 64) return p.exchange ? launch_pdl(pa_combine_kernel<64, true>, dim3(rows, 1), dim3(256), 0, st, p)
                                        : launch_pdl(pa_combine_kernel<64, false>, dim3(rows, 1), dim3(256), 0, st, p);
  return cudaErrorInvalidValue;
}

}  // namespace pa
