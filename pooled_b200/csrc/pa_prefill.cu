// Tiled causal prefill attention on the 5th-generation tensor cores: tcgen05.mma with the accumulators in tensor
// memory (TMEM), K/V tiles brought in by TMA.
//
// One CTA takes 128 consecutive query columns of one q head and walks the KV cache in tiles of 64 positions up to
// the causal diagonal.  K/V tiles of the G heads of a GQA group are the same bytes, read by G CTAs that run at about
// the same time; the caches of a prefill fit the 126 MB L2, so HBM sees them once.
//
//   warps 0, 3  TMA producers: K tiles and V tiles (64 x head_dim f16, 128-byte swizzle), a three-slot ring each
//   warp 1      MMA issuer (one thread) of the scores: S = Q K^T into one of three TMEM tiles (128 x 64 f32)
//   warp 2      allocates / frees tensor memory, and in between is the MMA issuer of O += P V into the TMEM
//               accumulator (128 x head_dim f32).  Both A operands come from tensor memory (Q sits there for the
//               CTA's life, P is written over its own S tile), so shared-memory bandwidth carries the K / V slices
//               only; completion is signalled to mbarriers with tcgen05.commit.  Two issuers: issuing blocks while
//               the tensor cores' queue is full, and a single thread alternating between the two products left it
//               empty during every wait
//   warps 4-7   softmax: thread r owns query row r (TMEM lane r): stores its Q row into TMEM as f16 pairs, then per
//   (and 8-11)  tile tcgen05.ld of its S row, causal mask, running max / sum, P = 2^(s - m) as f16 pairs back into
//               TMEM (tcgen05.st), and the epilogue (O / l, sigmoid gate, store).  The causal prefill runs two such
//               groups on alternate KV tiles (warp w and warp w + 4 reach the same 32 TMEM lanes): the exponentials
//               of a 128 x 64 tile take one group about as long as the tile's two products take the tensor cores,
//               so with one group the tensor pipe idles half of the time.  A row's reference maximum travels with
//               the tiles from group to group through shared memory; each group keeps its own share of the row sum
// S(j+1) is issued before the softmax of tile j has finished, so the tensor cores work on the next scores while
// the weights of the current tile are being formed.  O is rescaled only when a row's running maximum has grown by
// more than 2^8 since its last rescale (weights stay below 2^8, exact in f32 sums and safe in f16); the rescale
// waits for the previous P V to retire and rewrites the row's TMEM accumulator.
//
// Stands in for attn_flash_tile + attn_combine_tile + sigmoid_mul_mc of pooled (engine/wgsl/attn_tile.js:108-193,
// engine/wgsl/qwen35.js:877-887); there the pass is 16 columns wide and split over the sequence, here a pass takes
// the whole chunk and needs no split/combine because one CTA walks all of its keys.
#include "pa_params.cuh"

namespace pa {


constexpr int kBM = 128;   // query rows per CTA
constexpr int kBN = 64;    // keys per tile

// ---- tcgen05 wrappers ------------------------------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D (TMEM) (+)= A (smem descriptor) * B (smem descriptor), f16 inputs, f32 accumulate, issued by one thread
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has retired
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 consecutive f32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Shared-memory matrix descriptor, 128-byte swizzle.  K-major operand (rows of 64 f16 = 128 bytes, 8-row groups of
// 1024 bytes): sbo = 1024, lbo unused.  MN-major operand (64 contiguous MN elements per row of 128 bytes, 8 rows
// along K per 1024-byte group): lbo = distance between 64-element chunks along MN, sbo = 1024.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version of this architecture
  d |= (uint64_t)2 << 61;   // 128-byte swizzle
  return d;
}
// Instruction descriptor: f16 x f16 -> f32, A K-major, B K-major or MN-major, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t M, uint32_t N, uint32_t b_mn_major) {
  return (1u << 4) | (b_mn_major << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// TMEM loads / stores of 32 raw 32-bit columns (packed f16 pairs)
__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
        "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D (TMEM) (+)= A (TMEM, packed f16 pairs: lane = row, column c = elements 2c, 2c+1) * B (smem descriptor)
// The whole MMA warp runs the issue loop with identical values and only the elected lane executes the instruction:
// the operands of tcgen05.mma live in uniform registers, which the compiler can only use where control flow is
// warp-uniform (inside an `if (lane == 0)` every operand would be copied over one by one before each MMA).
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t leader;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(leader));
  return leader;
}
__device__ __forceinline__ void umma_f16_ts(uint32_t leader, uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 e, %5, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader));
}
__device__ __forceinline__ void umma_f16_ss(uint32_t leader, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 e, %5, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader));
}
__device__ __forceinline__ void umma_commit_elected(uint32_t leader, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "setp.ne.b32 e, %1, 0;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar), "r"(leader) : "memory");
}


// MODE 0: causal prefill, one CTA per (128 query columns, q head).
// MODE 1 / 2: split-K form for a k-token verify block: one CTA per (split of the KV sequence, kv head); the rows of the
//   tile are (column, head of the GQA group) pairs, at most 64 of them, and the CTA writes an unnormalised (o, m, l)
//   partial per row for the LSE combine.  MODE 2 keeps about 22 bits of q and of the softmax weights at no extra
//   tensor work: even rows carry the f16 high parts (q_hi, P_hi), odd rows the low parts (q_lo, P_lo) of the same
//   query row, so the two sit in neighbouring lanes of one warp: S_hi + S_lo is one shuffle per score in the
//   softmax, O_hi + O_lo one per output in the epilogue, and the split writes a single record per query row.

template <int HD, int MODE>
struct PfSmem {
  // S / P tiles in tensor memory.  The loop S(j) -> softmax(j) -> P V(j) -> S(j + SBUF) is a cycle of fixed length
  // (about 2.9 us at head_dim 256): the tile rate is SBUF tiles per cycle.  The causal prefill at head_dim 256 takes
  // four (Q then comes from shared memory only: as an A operand in tensor memory it was no faster, and its 64 columns
  // are the fourth tile); the other forms keep three and the lower half of Q in tensor memory.
  static constexpr int SBUF = (MODE == 0 && HD == 256) ? 4 : 3;
  // K ring and V ring depth.  Split-K: three K slots (the scores run two tiles ahead) and two V slots, which leaves
  // 32 KB free so that its CTAs can join SMs that still run a small kernel.  Prefill: one K slot per scores issuer,
  // tile j in slot j % 2, so that the fills of a slot are consumed by ONE thread, in order.  (With three slots shared by
  // two issuers a parity wait can be passed two fills early: the issuer of the odd tiles comes for tile 3 in slot 0
  // before tile 0 has landed there -- TMA copies finish out of order under the burst of a kernel's start -- the barrier
  // is still in its first phase, and a wait for "parity 1" takes that for fill 1 done.  The second arrival on the
  // slot's empty barrier that follows ends in a trap, once in some hundred launches.)
  static constexpr int NK = MODE == 0 ? 2 : 3, NV = MODE == 0 ? 3 : 2;
  static constexpr int KV_BYTES = HD * 128;         // [HD/64][64 rows][128 B]
  // tensor memory columns: the first TQC 64-dim chunks of Q (32 columns of f16 pairs each) | S tiles (64 each; P
  // overwrites the first 32 of its S) | O (HD).  HD 256: 64 + 192 + 256, or 0 + 256 + 256 = 512.
  static constexpr int TQC = SBUF == 4 ? 0 : (HD == 64 ? 1 : HD / 128);
  static constexpr int QS_BYTES = (HD / 64 - TQC > 0 ? HD / 64 - TQC : 1) * 128 * 128;   // the chunks of Q not in tensor memory: [chunk][128 rows][128 B]
  static constexpr int X_BYTES = 0;
  // softmax warpgroups: the causal prefill runs two, which take alternate KV tiles of the CTA's 128 query rows (the
  // exponentials of one tile take about as long as its two products on the tensor cores, so one group leaves the
  // tensor pipe idle half of the time); the split-K form does the same: with one group the softmax of a tile, not the
  // arrival of the tile from HBM, set the pace of its seven-tile loop
  static constexpr int NGRP = 2;
  // 4 service warps (K producer, scores issuer, TMEM allocator + P V issuer, V producer) + the softmax warps + a second
  // scores issuer (the last warp).  A score product is HD/16 instructions of 128 x 64 x 16 each: 32 cycles of tensor
  // work apiece against about twice that to issue one, so a single issuing thread, not the tensor cores, set the
  // loop's pace; two threads take alternate tiles (a tile's instructions stay in one thread: the order of its sums is
  // fixed).
  static constexpr int QK_ISSUERS = MODE == 0 ? 2 : 1;   // (the split-K form's 168 registers leave no room for a 13th warp)
  static_assert(QK_ISSUERS == 1 || (NK % QK_ISSUERS == 0 && SBUF >= 3), "a K slot belongs to one scores issuer");
  static constexpr int THREADS = 128 + 128 * NGRP + 32 * (QK_ISSUERS - 1);
  static constexpr int QK2_WARP = 4 + 4 * NGRP;      // the second scores issuer
  static constexpr int OFF_K = 0, OFF_V = NK * KV_BYTES, OFF_Q = (NK + NV) * KV_BYTES, OFF_X = OFF_Q + QS_BYTES, OFF_BAR = OFF_X + X_BYTES;
  static constexpr int OFF_ROW = OFF_BAR + 256;      // per-row hand-over between the softmax groups: the reference maximum, m[128]
  static constexpr int TOTAL = 1024 + OFF_ROW + 128 * 4;
  static_assert(TOTAL <= 227 * 1024, "shared memory of one CTA");
  static constexpr int T_Q = 0, T_S = TQC * 32, T_O = TQC * 32 + SBUF * kBN;
  static_assert(T_O + HD <= 512, "tensor memory columns");
  static constexpr int TMEM_COLS = 512;
};

template <int HD, int MODE>
__global__ void __launch_bounds__(PfSmem<HD, MODE>::THREADS, 1)
pa_prefill_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_q,
                  const __grid_constant__ CUtensorMap tm_o, const __grid_constant__ CUtensorMap tm_q2, const PrefillParams p) {
  using L = PfSmem<HD, MODE>;
  constexpr int CH = HD / 64;
  constexpr bool SK = MODE != 0, PREC = MODE == 2;
  constexpr int NK = L::NK, NV = L::NV, NGRP = L::NGRP, kSBuf = L::SBUF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + L::OFF_BAR);
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(bars + 31);
  volatile uint32_t* s_err = s_tmem + 1;
  float* s_rm = reinterpret_cast<float*>(base + L::OFF_ROW);   // [128] reference maximum of each query row (scaled, log2 units)
  // [2][128] each group's row sum and [2][128] the reference maximum it is expressed in: exchanged once, after the
  // last tile's scores exist, in the first K slot (every K tile has been multiplied by then)
  float* s_rl = reinterpret_cast<float*>(base + L::OFF_K);
  float* s_rr = s_rl + 256;
  const uint32_t bar0 = smem_u32(bars);
  enum { K_FULL = 0, K_EMPTY = 3, V_FULL = 6, V_EMPTY = 9, S_FULL = 12, P_FULL = 12 + kSBuf, PV_DONE = 12 + 2 * kSBuf, O_DONE = 12 + 3 * kSBuf,
         Q_FULL = O_DONE + 1, Q_ISSUED = O_DONE + 2, Q_SENT = O_DONE + 3,
         M_READY = O_DONE + 4 /* [2]: group g has published the row maxima after its tile */ };
  static_assert(M_READY + 2 <= 31, "barrier slots");
  uint8_t* q_s = base + L::OFF_Q;
  auto BAR = [&](int which, int idx) { return bar0 + 8u * (uint32_t)(which + idx); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // prefill: q tile (longest rows first) x q head.  split-K: split x kv head.
  const uint32_t q_tile = gridDim.x - 1 - blockIdx.x;
  const uint32_t h = blockIdx.y, g = SK ? blockIdx.y : h / p.G;
  const uint32_t c0 = q_tile * kBM;
  const uint32_t rows_valid = SK ? 0u : min((uint32_t)kBM, p.n_cols - c0);
  const uint32_t p0 = p.pos + c0;                       // cache row of column c0's own token
  uint32_t tile0 = 0, n_tiles = (p0 + rows_valid + kBN - 1) / kBN;
  if (SK) {
    const uint32_t tiles = (p.n_rows + kBN - 1) / kBN, tps = (tiles + p.n_splits - 1) / p.n_splits;
    tile0 = blockIdx.x * tps;
    if (tile0 >= tiles) return;                         // this split holds no row (uniform for the CTA)
    n_tiles = min(tiles, tile0 + tps) - tile0;
  }

  // prefill at head_dim 256 with f16 q: the 128 query rows (64 KB) land in shared memory, in the layout the score
  // products read, by one TMA copy issued at once, instead of through the softmax threads' registers
  const bool q_by_tma = MODE == 0 && L::TQC == 0 && p.q_tma;
  if (warp == 1 && lane == 0) {
    *s_err = 0;
    for (int i = 0; i < NK; ++i) { mbar_init(BAR(K_FULL, i), 1); mbar_init(BAR(K_EMPTY, i), 1); }
    for (int i = 0; i < NV; ++i) { mbar_init(BAR(V_FULL, i), 1); mbar_init(BAR(V_EMPTY, i), 1); }
    for (int i = 0; i < kSBuf; ++i) { mbar_init(BAR(S_FULL, i), 1); mbar_init(BAR(P_FULL, i), 128); mbar_init(BAR(PV_DONE, i), 1); }
    mbar_init(BAR(O_DONE, 0), 1);
    mbar_init(BAR(Q_FULL, 0), q_by_tma ? 1 : 128 * NGRP);
    mbar_init(BAR(Q_ISSUED, 0), HD >= 256 ? 128 * NGRP : 128);   // every thread that reads the staging area, after its last read
    mbar_init(BAR(Q_SENT, 0), 128 * NGRP);
    mbar_init(BAR(M_READY, 0), 128); mbar_init(BAR(M_READY, 1), 128);
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32((const void*)s_tmem), L::TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  // q, and the rows the RoPE/append kernel before this one writes, may only be touched after pdl_wait(); in the
  // split-K form the producers may fetch older K/V tiles ahead of it when the caller allows
  const bool early = SK && p.prefetch_old_rows;
  const uint32_t old_rows = SK ? min(p.n_rows - min(p.n_rows, p.n_cols), p.early_limit) : 0u;
  if (!early) pdl_wait();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t t_q = tmem + L::T_Q, t_s0 = tmem + L::T_S, t_o = tmem + L::T_O;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer, K ----
    if (lane == 0) {
      prefetch_tmap(&tm_k);
      if (q_by_tma) {
        mbar_expect_tx(BAR(Q_FULL, 0), (HD / 64) * kBM * 128);
        tma_load_3d(smem_u32(q_s), &tm_q, 0, (int)c0, (int)(h * (p.q_head_stride / 64)), BAR(Q_FULL, 0));
        if (p.q_tma == 2)   // the chunks no rotation touches come straight from the caller's q
          tma_load_3d(smem_u32(q_s + p.q_rot_chunks * (kBM * 128)), &tm_q2, 0, (int)c0, (int)(h * (p.q2_head_stride / 64) + p.q_rot_chunks), BAR(Q_FULL, 0));
      }
      bool waited = !early;
      for (uint32_t j = 0; j < n_tiles; ++j) {
        const uint32_t st = j % NK, u = j / NK;
        if (!waited && (tile0 + j + 1) * kBN > old_rows) { pdl_wait(); waited = true; }
        // split-K: tile 0 may go out at once (ahead of the wait if the caller allows); the next one only when the
        // requests for the query rows are on their way (a burst of tiles would queue in front of them), and the
        // third, whose slot stages the query rows, when those have been consumed
        if (SK && j == ((early && p.pre_stages == 0) ? 0u : 1u)) mbar_wait(BAR(Q_SENT, 0), 0, s_err, WAIT_QFULL);
        if (SK && j == 2) mbar_wait(BAR(Q_ISSUED, 0), 0, s_err, WAIT_QFULL);
        mbar_wait(BAR(K_EMPTY, st), (u & 1) ^ 1, s_err, WAIT_EMPTY);
        mbar_expect_tx(BAR(K_FULL, st), L::KV_BYTES);
        if (SK && p.kv_evict_first) tma_load_3d_hint(smem_u32(base + L::OFF_K + st * L::KV_BYTES), &tm_k, 0, (int)((tile0 + j) * kBN), (int)(g * CH), BAR(K_FULL, st), l2_policy_evict_first());
        else tma_load_3d(smem_u32(base + L::OFF_K + st * L::KV_BYTES), &tm_k, 0, (int)((tile0 + j) * kBN), (int)(g * CH), BAR(K_FULL, st));
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ TMA producer, V ----
    // (its own thread: behind the K loads in one loop, K(j+1) would wait for the V slot that P V (j-1) still reads)
    if (lane == 0) {
      prefetch_tmap(&tm_v);
      bool waited = !early;
      for (uint32_t j = 0; j < n_tiles; ++j) {
        const uint32_t st = j % NV, u = j / NV;
        if (!waited && (tile0 + j + 1) * kBN > old_rows) { pdl_wait(); waited = true; }
        if (SK && j == 1) mbar_wait(BAR(Q_ISSUED, 0), 0, s_err, WAIT_QFULL);   // slot 1 stages query rows until then
        mbar_wait(BAR(V_EMPTY, st), (u & 1) ^ 1, s_err, WAIT_EMPTY);
        mbar_expect_tx(BAR(V_FULL, st), L::KV_BYTES);
        if (SK && p.kv_evict_first) tma_load_3d_hint(smem_u32(base + L::OFF_V + st * L::KV_BYTES), &tm_v, 0, (int)((tile0 + j) * kBN), (int)(g * CH), BAR(V_FULL, st), l2_policy_evict_first());
        else tma_load_3d(smem_u32(base + L::OFF_V + st * L::KV_BYTES), &tm_v, 0, (int)((tile0 + j) * kBN), (int)(g * CH), BAR(V_FULL, st));
      }
    }
  } else if (warp == 1 || (L::QK_ISSUERS == 2 && warp == L::QK2_WARP)) {
    // ------------------------------------------------------------------ MMA issuers, scores ----
    // S(j) = Q K(j)^T.  The whole warp runs the loop and the elected lane issues.  Issuing blocks while the tensor
    // cores' queue is full, so one thread issuing both products of every tile spends its time in turns on each and
    // the waits in between leave the queue empty; with the scores here and P V in warp 2 there are two queues' worth
    // of work in front of the tensor cores.  S(j) goes into the TMEM tile of S(j - 3) / P(j - 3): once that P V has
    // retired (PV_DONE).
    {
      const uint32_t leader = elect_one();
      constexpr uint32_t idesc_qk = umma_idesc(kBM, kBN, 0);
      // Both A operands live in tensor memory (Q for the whole CTA, P per tile), so a k-step costs shared-memory
      // bandwidth for the K or V slice only.  B descriptors are built once; a k-step adds a byte offset (>> 4).
      uint64_t k_desc[NK];
#pragma unroll
      for (int i = 0; i < NK; ++i) k_desc[i] = smem_desc(smem_u32(base + L::OFF_K + i * L::KV_BYTES), 16, 1024);
      const uint64_t q_desc = smem_desc(smem_u32(q_s), 16, 1024);
      mbar_wait(BAR(Q_FULL, 0), 0, s_err, WAIT_QFULL);
      tc_fence_after();
      for (uint32_t j = (warp == 1 ? 0u : 1u); j < n_tiles; j += L::QK_ISSUERS) {
        const uint32_t sb = j % kSBuf, st = j % NK;
        if (j >= (uint32_t)kSBuf) mbar_wait(BAR(PV_DONE, sb), ((j - kSBuf) / kSBuf) & 1, s_err, WAIT_MMA);
        mbar_wait(BAR(K_FULL, st), (j / NK) & 1, s_err, WAIT_KFULL);
        tc_fence_after();
        const uint64_t kd = st == 0 ? k_desc[0] : (st == 1 ? k_desc[1] : k_desc[NK - 1]);
        const uint32_t ts = t_s0 + sb * kBN;
        // the head dims whose Q chunks sit in tensor memory first, then those whose Q comes from shared memory
        constexpr int TS_STEPS = L::TQC * 4;
#pragma unroll
        for (int ks = 0; ks < TS_STEPS; ++ks)
          umma_f16_ts(leader, ts, t_q + ks * 8, kd + (uint64_t)(((ks >> 2) * (kBN * 128) + (ks & 3) * 32) >> 4), idesc_qk, ks > 0);
#pragma unroll
        for (int ks = TS_STEPS; ks < HD / 16; ++ks)
          umma_f16_ss(leader, ts, q_desc + (uint64_t)(((((ks - TS_STEPS) >> 2)) * (kBM * 128) + (ks & 3) * 32) >> 4),
                      kd + (uint64_t)(((ks >> 2) * (kBN * 128) + (ks & 3) * 32) >> 4), idesc_qk, ks > 0 ? 1u : 0u);
        umma_commit_elected(leader, BAR(K_EMPTY, st));
        umma_commit_elected(leader, BAR(S_FULL, sb));
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ MMA issuer, P V ----
    // O += P(j) V(j), in tile order (this thread's products retire in order, so O is always complete up to a tile)
    {
      const uint32_t leader = elect_one();
      constexpr uint32_t idesc_pv = umma_idesc(kBM, HD, 1);
      uint64_t v_desc[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) v_desc[i] = smem_desc(smem_u32(base + L::OFF_V + i * L::KV_BYTES), kBN * 128, 1024);
      for (uint32_t j = 0; j < n_tiles; ++j) {
        const uint32_t sb = j % kSBuf, st = j % NV;
        mbar_wait(BAR(P_FULL, sb), (j / kSBuf) & 1, s_err, WAIT_QFULL);
        mbar_wait(BAR(V_FULL, st), (j / NV) & 1, s_err, WAIT_VFULL);
        tc_fence_after();
        const uint64_t vd = st == 0 ? v_desc[0] : (st == 1 ? v_desc[1] : v_desc[NV - 1]);
        const uint32_t tp = t_s0 + sb * kBN;     // P(j): packed f16 pairs in the first 32 columns of S(j)'s tile
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks)
          umma_f16_ts(leader, t_o, tp + ks * 8, vd + (uint64_t)((ks * 2048) >> 4), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit_elected(leader, BAR(V_EMPTY, st));
        umma_commit_elected(leader, BAR(PV_DONE, sb));
      }
      umma_commit_elected(leader, BAR(O_DONE, 0));
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax + epilogue ----
    const uint32_t wg = (warp - 4) >> 2;                 // softmax group: takes KV tiles wg, wg + NGRP, ...
    const uint32_t qd = (warp - 4) & 3, row = qd * 32 + lane;   // a warp reaches the 32 TMEM lanes of its index mod 4
    const uint32_t lane_addr = (qd * 32) << 16;
    // split-K: a (column, head-of-group) pair per row; MODE 2: per two rows (even: high parts, odd: low parts)
    const bool is_lo = SK && (PREC ? (row & 1u) != 0 : row >= 64);
    const uint32_t lr = SK ? (PREC ? row >> 1 : (row & 63u)) : row;
    const uint32_t sk_c = lr / p.G, sk_hh = lr % p.G;
    const uint32_t head = SK ? g * p.G + sk_hh : h;
    const bool live = SK ? (lr < p.n_cols * p.G && (PREC || !is_lo)) : row < rows_valid;
    // keys [0, lim) are visible to this row
    const uint32_t lim = SK ? (uint32_t)min(max(p.lim0 + (int32_t)min(sk_c, p.n_cols - 1), 0), (int32_t)p.n_rows) : p0 + row + 1;
    // m_st: the row's reference maximum (the weights of a tile are 2^(s - m_st); it moves only when a tile's maximum
    // passes it by more than 2^8).  With two softmax groups it travels with the tiles: the group that took tile j - 1
    // publishes it in s_rm, the group that takes tile j picks it up there.  l_sum: this group's share of the row sum,
    // expressed in the reference m_l.  (split-K: a split may hold no visible key of a row, hence the finite start.)
    // ---- split-K: the few query rows are fetched by all 128 threads at once, 16 bytes per request, straight into
    //      shared memory (cp.async: no registers held, every request in flight together), into the K and the V slot
    //      the producers leave alone until Q_ISSUED (32 rows each); a row's chunks are XOR-swizzled so that the
    //      per-row reads below do not all hit one bank.  (One thread loading its own 1 KB row needs the loads in register-sized batches,
    //      a memory round trip each: 4.8 us between the wait and the first MMA.) ----
    auto stage_row = [&](uint32_t pr) {
      return (pr < 32 ? base + L::OFF_K + 2 * L::KV_BYTES : base + L::OFF_V + L::KV_BYTES - (size_t)32 * (HD * 4)) + (size_t)pr * (HD * 4);
    };
    // q as f32 (this kernel splits it), as f16 (no low part), or as two f16 planes, high and low parts, which the
    // RoPE kernel of a layer call writes: then a staged row is [high HD halves][low HD halves] and nothing is left
    // to convert here (the f32 -> f16 conversions of 128 x HD elements took 3 us on four warps)
    const bool planes = SK && p.q_f16 && p.q_lo != nullptr;
    const uint32_t q_es = p.q_f16 ? 2u : 4u, q_ch = planes ? HD * 4 / 16 : HD * q_es / 16;     // 16-byte chunks per staged row
    if (early) pdl_wait();
    pdl_trigger();
    if (SK) {
      const uint32_t pairs = p.n_cols * p.G, st_tid = tid - 128, total = pairs * q_ch;
      for (uint32_t idx = st_tid; idx < total; idx += 128 * NGRP) {
        const uint32_t pr = idx / q_ch, c = idx % q_ch;
        const uint32_t half_ch = HD * 2 / 16;
        const bool lo_plane = planes && c >= half_ch;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(lo_plane ? p.q_lo : p.q) +
                             ((uint64_t)(p.col0 + pr / p.G) * p.q_col_stride + (uint64_t)(g * p.G + pr % p.G) * p.q_head_stride) * q_es +
                             (uint64_t)(lo_plane ? c - half_ch : c) * 16;
        const uint32_t dst = smem_u32(stage_row(pr) + ((c ^ (pr & 7u)) << 4));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      mbar_arrive(BAR(Q_SENT, 0));
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      named_bar_sync(1, 128 * NGRP);
    }
    const uint8_t* my_stage = stage_row(lr & 63u);
    auto stage_ld = [&](uint32_t c) { return *reinterpret_cast<const uint4*>(my_stage + ((c ^ (lr & 7u)) << 4)); };
    // ---- this thread's Q row -> f16 pairs: lower half of the dims to tensor memory, upper half to shared memory ----
    if (!q_by_tma) {
      const uint64_t off = (uint64_t)(SK ? p.col0 + (live ? sk_c : 0) : c0 + (live ? row : 0)) * p.q_col_stride + (uint64_t)head * p.q_head_stride;
      // ER elements per round (the loads of a round are all in flight together), in 64-dim chunks: the first TQC chunks
      // of the row go to tensor memory (32 columns each), the others to shared memory (one 128-byte row chunk each)
      constexpr int ER = HD >= 128 ? 128 : 64, ROUNDS = HD / ER, HCN = ER / 64;
#pragma unroll 1
      for (int c2 = 0; c2 < ROUNDS; ++c2) {
        // with two softmax groups each stages one round of its rows (head_dim 256); a single round is the first group's
        if (NGRP == 2 && (uint32_t)(ROUNDS == 2 ? c2 : 0) != wg) continue;
        uint32_t w[ER / 2];
        if (p.q_f16) {
          const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.q) + off + c2 * ER);
#pragma unroll
          for (int i = 0; i < ER / 8; ++i) {
            const uint32_t cb = (planes && is_lo) ? HD * 2 / 16 : 0;
            const uint4 x = (live && (planes || !is_lo)) ? (SK ? stage_ld(cb + c2 * (ER / 8) + i) : src[i]) : make_uint4(0, 0, 0, 0);   // plain f16 q has no low part
            w[4 * i] = x.x; w[4 * i + 1] = x.y; w[4 * i + 2] = x.z; w[4 * i + 3] = x.w;
          }
        } else {
          const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.q) + off + c2 * ER);
          float4 xs[ER / 4];
#pragma unroll
          for (int i = 0; i < ER / 4; ++i) {
            if (SK) { const uint4 r4 = live ? stage_ld(c2 * (ER / 4) + i) : make_uint4(0, 0, 0, 0); xs[i] = *reinterpret_cast<const float4*>(&r4); }
            else xs[i] = live ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int i = 0; i < ER / 4; ++i) {
            float4 x = xs[i];
            if (is_lo) {   // what the f16 high part leaves over
              x.x -= __half2float(__float2half_rn(x.x)); x.y -= __half2float(__float2half_rn(x.y));
              x.z -= __half2float(__float2half_rn(x.z)); x.w -= __half2float(__float2half_rn(x.w));
            }
            w[2 * i] = pack_h2(x.x, x.y); w[2 * i + 1] = pack_h2(x.z, x.w);
          }
        }
        if (c2 == ROUNDS - 1 || (NGRP == 2 && ROUNDS == 2)) {
          // this thread is done with the staging area (with two groups and two rounds, each thread reads one round):
          // the producers may fetch into it (and may send the tiles they held back so that the early burst would not
          // queue in front of the q requests)
          fence_proxy_async();
          mbar_arrive(BAR(Q_ISSUED, 0));
        }
#pragma unroll
        for (int hc = 0; hc < HCN; ++hc) {
          const int c = HCN * c2 + hc;
          uint32_t wc[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) wc[i] = w[32 * hc + i];
          if (c < L::TQC) {
            tmem_st32u(t_q + c * 32 + lane_addr, wc);
          } else {
            uint8_t* dst = q_s + (c - L::TQC) * (kBM * 128) + row * 128;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<uint4*>(dst + ((i ^ (row & 7)) << 4)) = make_uint4(wc[4 * i], wc[4 * i + 1], wc[4 * i + 2], wc[4 * i + 3]);
          }
        }
      }
      fence_proxy_async();
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(BAR(Q_FULL, 0));
    }
    float m_st = SK ? -1.0e30f : -INFINITY, l_sum = 0.f, m_l = m_st;
    for (uint32_t j = wg; j < n_tiles; j += NGRP) {
      const uint32_t b = j % kSBuf, u = j / kSBuf, kv0 = (tile0 + j) * kBN;
      mbar_wait(BAR(S_FULL, b), u & 1, s_err, WAIT_MMA);
      tc_fence_after();
      float s[kBN];
      {
        float t0[32], t1[32];
        tmem_ld32(t_s0 + b * kBN + lane_addr, t0);
        tmem_ld32(t_s0 + b * kBN + 32 + lane_addr, t1);
#pragma unroll
        for (int i = 0; i < 32; ++i) { s[i] = t0[i]; s[32 + i] = t1[i]; }
      }
      if (PREC) {
        // S = S_hi + S_lo: the two rows of a query row are neighbouring lanes
#pragma unroll
        for (int i = 0; i < kBN; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], 1);
      }
      // maximum of the raw scores (the scale is positive), causal mask on tiles that reach this row's diagonal
      if (kv0 + kBN > lim) {
#pragma unroll
        for (int i = 0; i < kBN; ++i) if (kv0 + i >= lim) s[i] = -INFINITY;
      }
      float mt = s[0];
#pragma unroll
      for (int i = 1; i < kBN; ++i) mt = fmaxf(mt, s[i]);
      mt *= p.scale_log2;
      if (NGRP == 2 && j > 0) {
        mbar_wait(BAR(M_READY, (j - 1) & 1), ((j - 1) >> 1) & 1, s_err, WAIT_MMA);
        m_st = s_rm[row];
      }
      float alpha = 1.f;
      bool grow = false;
      if (!SK && j == 0) m_st = mt;                 // key 0 is visible to every row, so mt is finite
      else if (mt > m_st + 8.f) { alpha = ex2_approx(m_st - mt); m_st = mt; grow = true; }
      if (NGRP == 2) {
        // hand the reference on at once: the other group's next tile needs nothing else from this one
        s_rm[row] = m_st;
        mbar_arrive(BAR(M_READY, j & 1));
      }
      if (m_st != m_l) { l_sum *= ex2_approx(m_l - m_st); m_l = m_st; }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // O must not change under the previous P V: wait for it, then rescale this warp's 32 rows in TMEM
        const uint32_t jb = (j - 1) % kSBuf, ju = (j - 1) / kSBuf;
        mbar_wait(BAR(PV_DONE, jb), ju & 1, s_err, WAIT_MMA);
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          float o[32];
          tmem_ld32(t_o + c * 32 + lane_addr, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tmem_st32(t_o + c * 32 + lane_addr, o);
        }
      }
      // P = 2^(s - m) as packed f16 pairs over the first 32 columns of this S buffer (its scores are in registers now)
      uint32_t pw[32];
      float ls = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float e0 = ex2_approx(fmaf(s[2 * i], p.scale_log2, -m_st)), e1 = ex2_approx(fmaf(s[2 * i + 1], p.scale_log2, -m_st));
        ls += e0 + e1;
        if (is_lo) { e0 -= __half2float(__float2half_rn(e0)); e1 -= __half2float(__float2half_rn(e1)); }
        pw[i] = pack_h2(e0, e1);
      }
      l_sum += ls;
      tmem_st32u(t_s0 + b * kBN + lane_addr, pw);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(BAR(P_FULL, b));
    }
    // ---- epilogue: O / l, gate, store ----
    if (NGRP == 2) {
      // the row sum is the two groups' shares brought to the final reference; O already is in it
      const uint32_t last = n_tiles - 1;
      mbar_wait(BAR(M_READY, last & 1), (last >> 1) & 1, s_err, WAIT_MMA);   // published after S(last) was complete: the K ring is idle
      s_rl[wg * 128 + row] = l_sum; s_rr[wg * 128 + row] = m_l;
      named_bar_sync(2, 128 * NGRP);
      const float m_fin = s_rm[row];
      l_sum = s_rl[row] * ex2_approx(s_rr[row] - m_fin) + s_rl[128 + row] * ex2_approx(s_rr[128 + row] - m_fin);
    }
    mbar_wait(BAR(O_DONE, 0), 0, s_err, WAIT_MMA);
    tc_fence_after();
    const float inv_l = 1.f / l_sum;
    const uint32_t col = c0 + row;
    if (SK) {
      // unnormalised partial (o, m, l) of this split for the LSE combine.  MODE 2: O = O_hi + O_lo, the odd lane's
      // row added to the even lane's, which writes the record (m and l are the same in both)
      const uint64_t prow = (uint64_t)(p.col0 + sk_c) * p.n_heads + head;
      const uint64_t slot = prow * p.n_splits + blockIdx.x;
      const bool writer = live && !is_lo;
      // A lane holds a row: stored as they are, the 32 lanes of an instruction would write 16 bytes each into 32
      // records 1 KB apart.  The rows go to shared memory first (the K ring is idle: every product has retired; rows
      // 16 bytes apart in their bank phase), then all 128 threads write whole records, 16 consecutive bytes per
      // thread and 512 consecutive bytes per warp instruction.
      constexpr int RP = HD / 4 + 1;                                  // row pitch in float4
      float4* xs = reinterpret_cast<float4*>(base + L::OFF_K + 2048);   // [rows][RP], behind the groups' row sums (s_rl, s_rr)
      unsigned long long* xslot = reinterpret_cast<unsigned long long*>(xs + 64 * RP);   // [64] record of each row, ~0: none
      if (!is_lo && lr < 64 && wg == 0) xslot[lr] = writer ? (unsigned long long)slot : ~0ull;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        if (NGRP == 2 && (uint32_t)(c & 1) != wg) continue;   // the groups share the columns out
        float o[32];
        tmem_ld32(t_o + c * 32 + lane_addr, o);
        if (PREC) {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] += __shfl_xor_sync(0xffffffffu, o[i], 1);
        }
        if (writer) {
#pragma unroll
          for (int i = 0; i < 8; ++i) xs[lr * RP + c * 8 + i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
      }
      named_bar_sync(1, 128 * NGRP);
      for (uint32_t idx = tid - 128; idx < 64 * (HD / 4); idx += 128 * NGRP) {
        const uint32_t rr = idx / (HD / 4), c4 = idx % (HD / 4);
        const unsigned long long sl = xslot[rr];
        if (sl != ~0ull) reinterpret_cast<float4*>(p.part_o + sl * HD)[c4] = xs[rr * RP + c4];
      }
      if (writer && wg == 0) { p.part_ml[slot * 2] = (NGRP == 2 ? s_rm[row] : m_st) * 0.6931471805599453f; p.part_ml[slot * 2 + 1] = l_sum; }
    } else if (MODE == 0 && p.out_tma) {
      // The output tile leaves as the query tile came: through shared memory in the TMA layout ([64-dim chunk][row][128 B],
      // 16-byte pieces XOR-swizzled by the row), one bulk tensor store for the CTA.  The K ring is idle (every product
      // has retired, and so is the V ring that follows it: the tile may reach into it); the tile sits behind the row sums
      // the groups have just exchanged there.  Rows past the prompt's end are not written: the map ends at n_cols.
      // (A lane storing its own row issues 16-byte stores 12 KB apart.)
      static_assert(2048 + (HD / 64) * kBM * 128 <= (L::NK + L::NV) * L::KV_BYTES, "the output tile fits the idle rings");
      uint8_t* o_s = base + L::OFF_K + 2048;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        if (NGRP == 2 && (uint32_t)(c & 1) != wg) continue;   // the groups share the columns out
        float o[32];
        tmem_ld32(t_o + c * 32 + lane_addr, o);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= inv_l;
        if (p.gate && row < rows_valid) {
          const uint64_t go = (uint64_t)col * p.gate_col_stride + (uint64_t)h * p.gate_head_stride + c * 32;
          const uint4* gp = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.gate) + go);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 gq = gp[i];
            const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 gv = __half22float2(*reinterpret_cast<const __half2*>(&gw[k]));
              o[8 * i + 2 * k] *= 1.0f / (1.0f + __expf(-gv.x));
              o[8 * i + 2 * k + 1] *= 1.0f / (1.0f + __expf(-gv.y));
            }
          }
        }
        uint8_t* dst = o_s + (c >> 1) * (kBM * 128) + row * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(dst + ((((c & 1) * 4 + i) ^ (row & 7)) << 4)) =
              make_uint4(pack_h2(o[8 * i], o[8 * i + 1]), pack_h2(o[8 * i + 2], o[8 * i + 3]), pack_h2(o[8 * i + 4], o[8 * i + 5]), pack_h2(o[8 * i + 6], o[8 * i + 7]));
      }
      fence_proxy_async();
      named_bar_sync(1, 128 * NGRP);
      if (tid == 128) {
        tma_store_3d(&tm_o, 0, (int)c0, (int)(h * (HD / 64)), smem_u32(o_s));
        tma_store_wait_read();
      }
    } else {
#pragma unroll 1
    for (int c = 0; c < HD / 32; ++c) {
      if (NGRP == 2 && (uint32_t)(c & 1) != wg) continue;   // the groups share the columns out
      float o[32];
      tmem_ld32(t_o + c * 32 + lane_addr, o);
      if (row < rows_valid) {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= inv_l;
        if (p.gate) {
          const uint64_t go = (uint64_t)col * p.gate_col_stride + (uint64_t)h * p.gate_head_stride + c * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float gv = p.act_f16 ? __half2float(reinterpret_cast<const __half*>(p.gate)[go + i]) : reinterpret_cast<const float*>(p.gate)[go + i];
            o[i] *= 1.0f / (1.0f + __expf(-gv));
          }
        }
        const uint64_t oo = (uint64_t)col * p.out_col_stride + (uint64_t)h * HD + c * 32;
        if (p.act_f16) {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.out) + oo);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst[i] = make_uint4(pack_h2(o[8 * i], o[8 * i + 1]), pack_h2(o[8 * i + 2], o[8 * i + 3]), pack_h2(o[8 * i + 4], o[8 * i + 5]), pack_h2(o[8 * i + 6], o[8 * i + 7]));
        } else {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + oo);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
      }
    }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem, L::TMEM_COLS);
  }
  if (tid == 0 && *s_err) atomicMax(p.err, *s_err);
}

int prefill_supported(const pa_ctx* ctx) { return ctx->cfg.head_dim == 256 || ctx->cfg.head_dim == 128 || ctx->cfg.head_dim == 64; }

template <int HD, int MODE>
static cudaError_t launch_pf(const pa_layer* L, const PrefillParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_q,
                             const CUtensorMap& tm_o, const CUtensorMap& tm_q2, dim3 grid, cudaStream_t st) {
  static bool attr_set[64] = {};
  const int dev = L->ctx->device & 63;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(pa_prefill_kernel<HD, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfSmem<HD, MODE>::TOTAL);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  if (MODE == 0) {
    pa_prefill_kernel<HD, MODE><<<grid, PfSmem<HD, MODE>::THREADS, PfSmem<HD, MODE>::TOTAL, st>>>(tm_k, tm_v, tm_q, tm_o, tm_q2, p);
    return cudaGetLastError();
  }
  return launch_pdl(pa_prefill_kernel<HD, MODE>, grid, dim3(PfSmem<HD, MODE>::THREADS), (size_t)PfSmem<HD, MODE>::TOTAL, st, tm_k, tm_v, tm_q, tm_o, tm_q2, p);
}

cudaError_t launch_prefill(const pa_layer* L, const PrefillParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_q,
                           const CUtensorMap& tm_o, const CUtensorMap& tm_q2, cudaStream_t st) {
  const dim3 grid((p.n_cols + kBM - 1) / kBM, p.n_heads);
  switch (L->ctx->cfg.head_dim) {
    case 256: return launch_pf<256, 0>(L, p, tm_k, tm_v, tm_q, tm_o, tm_q2, grid, st);
    case 128: return launch_pf<128, 0>(L, p, tm_k, tm_v, tm_q, tm_o, tm_q2, grid, st);
    case 64: return launch_pf<64, 0>(L, p, tm_k, tm_v, tm_q, tm_o, tm_q2, grid, st);
    default: return cudaErrorInvalidValue;
  }
}

// k-token verify block (more than 8 query rows per kv head) on the tensor cores: split-K form of the same kernel
cudaError_t launch_verify(const pa_layer* L, const PrefillParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v, uint32_t n_kv, cudaStream_t st) {
  const dim3 grid(p.n_splits, n_kv);
  const bool precise = !(L->ctx->cfg.flags & PA_FLAG_FAST);
  if (L->ctx->cfg.head_dim == 256)
    return precise ? launch_pf<256, 2>(L, p, tm_k, tm_v, tm_k, tm_k, tm_k, grid, st) : launch_pf<256, 1>(L, p, tm_k, tm_v, tm_k, tm_k, tm_k, grid, st);   // (no maps of q and out in this form)
  return precise ? launch_pf<128, 2>(L, p, tm_k, tm_v, tm_k, tm_k, tm_k, grid, st) : launch_pf<128, 1>(L, p, tm_k, tm_v, tm_k, tm_k, tm_k, grid, st);
}

}  // namespace pa
