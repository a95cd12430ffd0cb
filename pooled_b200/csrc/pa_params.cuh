// Kernel parameter blocks shared by the kernels and the C-ABI front.
#pragma once
#include "pa_common.cuh"

namespace pa {

struct DecodeParams {
  const void* q;            // rotated queries
  int q_f16;                // dtype of q
  uint64_t q_col_stride, q_head_stride;
  float* part_o;            // [rows][n_splits][HD]
  float* part_ml;           // [rows][n_splits][2]   (m in natural-log units, l)
  uint32_t n_splits;
  uint32_t n_heads, G, max_seq, n_stages;
  // fused front (one token; head_dim 256 with 64 rotary dims, or head_dim 128 rotated in full): q arrives unrotated and the consumers rotate
  // it; the CTA that walks the sequence's last tile also rotates k, converts v and appends the token's row
  // fused: 1 = one item, cos / sin in rope_ang; 2 = one token of each of several items, each CTA evaluates its own
  // item's cos / sin (float64 sincos of pos * inv_freq, ahead of its wait).  append: bit i set = this cache holds item
  // i's new row (clear on another rank's shard)
  uint32_t fused, append;
  const void* k_new; const void* v_new;               // the tokens' k / v rows, [items][n_kv * hd], dtype as q
  uint64_t k_new_stride, v_new_stride;                // elements between the rows of consecutive items
  const double* inv_freq;                             // theta^(-2i/n_rot), i < n_rot/2 (fused == 2)
  __half* k_cache; __half* v_cache;                   // caches of the layer
  Angle rope_ang[64];       // cos / sin of pos * theta^(-2i/n_rot), i < n_rot/2, evaluated by the host in float64
  uint32_t prefetch_old_rows;  // 1: K/V tiles below the call's own new rows may be fetched before the predecessor kernel ends
  uint32_t pre_stages;         // ... but only this many per CTA before the q loads are in flight
  uint32_t kv_evict_first;     // 1: the K / V tiles enter L2 as evict-first lines (they are read once)
  uint32_t early_limit;        // ... and only rows below this one (the call before may still be writing its own row)
  float scale_log2;         // log2(e) / sqrt(head_dim)
  // the layer the engine runs next (pa_layer_set_next): once a CTA has requested its own last tile it asks L2 for the
  // first next_tiles tiles of the same split of that layer, so HBM keeps working across the kernel boundary
  uint32_t next_tiles, next_max_seq;
  uint32_t own_prefetch;       // n: with prefetch_old_rows, n of the CTA's tiles beyond the early ones are asked into L2 at entry
  // gather mode: item i is one column attending the rows listed at gather + col0[i] * gather_stride: [0] = n, then n
  // cache rows ascending (k_cache / v_cache above are the layer's caches)
  const uint32_t* gather; uint32_t gather_stride;
  // merge != 0: no combine kernel follows; the CTAs of each (item, kv head) merge their own records, gate and store
  // (2: CTAs without a merge unit leave as soon as their record is counted; 1: they wait like the others)
  uint32_t merge; unsigned int* merge_ctr;
  unsigned int* xch_ctr;   // != nullptr: the call ends in a cross-GPU exchange; the kernel's first thread advances its call counter
  const void* gate; uint64_t gate_col_stride, gate_head_stride;
  void* out; uint64_t out_col_stride; int act_f16;
  uint32_t* err;
  ItemList items;
};

struct CombineParams {
  const float* o;        // record s of row prow: o + prow * o_row_stride + s * o_part_stride, HD floats
  const float* ml;       // (m, l) of it:        ml + prow * ml_row_stride + s * ml_part_stride
  uint64_t o_row_stride, o_part_stride, ml_row_stride, ml_part_stride;
  uint32_t n_heads, fixed_parts;  // fixed_parts != 0: that many records per row; else from the item's split plan
  uint32_t n_splits;
  uint32_t groups;                // records per split (the decode kernel's consumer groups)
  const uint32_t* gather; uint32_t gather_stride;   // gather mode: the columns' row lists (their lengths set the plan)
  const void* gate; uint64_t gate_col_stride, gate_head_stride;
  void* out; uint64_t out_col_stride;
  int act_f16;
  float* partial_out;    // != nullptr: write the merged record (o unnormalised, m, l) instead of out
  uint64_t partial_rows; // rows in partial_out (o block first, then the (m, l) block)
  ItemList items; uint32_t n_items;
  int exchange;          // != 0: publish the merged record to every rank, wait for theirs, merge across ranks, then out
  ExchangeView xc;
  uint32_t xch_sweeps;   // polling limit of the exchange wait
  uint32_t* err;
};

struct RopeParams {
  uint32_t trigger_early;      // 1: the dependent kernel may start before this one's own wait (inside a layer call only)
  const void* q; uint64_t q_col_stride, q_head_stride; uint32_t q_heads;   // q == nullptr: skip
  void* q_out; uint64_t q_out_col_stride; int q_out_f16;                    // f32 (or f16), heads packed [q_heads][hd]
  uint64_t q_lo_offset;    // q_out_f16 == 2: f16 high parts at q_out, f16 low parts (x - fl16(x)) this many halves later
  uint32_t q_rot_only;     // 1 (vectorised kernel): only the rotated dims of q are written; the reader takes the rest from q itself
  const void* k; const void* v; uint64_t kv_col_stride, v_col_stride; uint32_t kv_heads;  // k == nullptr: skip; kv_col_stride is k's
  __half* k_cache; __half* v_cache; uint64_t cache_row0;                    // row of column 0
  uint32_t hd, n_rot, pos, mode;
  int in_f16;
  const double* inv_freq;
  const float* cs_table;   // [n_cols][n_rot] (cos, sin) per pair
  const Angle* angles;     // PA_ROPE_F64: [n_cols][n_rot/2] cos / sin of the call's columns (nullptr: evaluate here)
  uint32_t n_ang;          // > 0: a call of at most 64 angles carries them here, evaluated by the host's libm
  Angle ang[64];
  // one token of each of several sequences in one launch (single-token kernel only): column c is item c
  uint32_t n_items;
  uint32_t item_pos[32];   // global position of the item's token
  uint64_t item_row[32];   // its cache row (sequence * max_seq + position - origin), or ~0: not in this shard, no append
};

struct AnglesParams {
  Angle* out;              // [n_cols][half]
  const double* inv_freq;
  uint32_t pos0, n_cols, half;
};

struct HeadNormParams {
  const void* x; uint64_t x_col_stride, x_head_stride;
  void* y; uint64_t y_col_stride, y_head_stride;
  const float* w;          // [hd]
  // heads at or past n_first (blockIdx.y) belong to a second array with its own weight: q and k of a layer in one launch
  uint32_t n_first;
  const void* x2; uint64_t x2_col_stride, x2_head_stride;
  void* y2; uint64_t y2_col_stride, y2_head_stride;
  const float* w2;
  double eps;
  uint32_t hd; int f16;
};

struct SigmoidParams {
  void* a; uint64_t a_col_stride; const void* g; uint64_t g_col_stride, g_head_stride;
  uint32_t n_heads, hd; int f16;
};

// append into an int8 (+ scales) or f32 cache: k and v rows of n columns, already rotated
struct KvStoreParams {
  int format;                                   // PA_KV_Q8 or PA_KV_F32
  const void* k; const void* v; uint64_t k_col_stride, v_col_stride; int k_f16, v_f16;
  int8_t* k8; int8_t* v8; float* ks; float* vs;  // int8 caches and their scales (one per 32 values)
  float* k32; float* v32;                        // f32 caches
  uint32_t kv_dim; uint64_t cache_row0;          // cache row of column 0
};

// split-K decode / verify / prefill of the columns of one item over an int8 or f32 cache
struct AnyDecodeParams {
  const void* q; int q_f16; uint64_t q_col_stride, q_head_stride;
  const void* k; const void* v; const float* ks; const float* vs;
  uint32_t kv_dim, hd, G, n_heads, max_seq, n_splits;
  uint32_t seq; int32_t lim0; uint32_t n_rows;   // rows column 0 sees (before clamping), rows the last column sees
  uint64_t col0;                                 // first column of the item in q and in the record buffers
  float* part_o; float* part_ml;
};

struct PrefillParams {
  const void* q; int q_f16; uint64_t q_col_stride, q_head_stride;
  const void* q_lo;             // split-K, f16 q: the low parts as a second f16 array of the same shape (nullptr: none)
  const void* gate; uint64_t gate_col_stride, gate_head_stride;
  void* out; uint64_t out_col_stride; int act_f16;
  uint32_t seq, pos, n_cols, n_heads, G, max_seq;
  float scale_log2;
  uint32_t* err;
  // split-K form (k-token verify on the tensor cores): one CTA per (split, kv head), rows = columns x heads of the group
  float* part_o; float* part_ml; uint32_t n_splits; int32_t lim0; uint32_t n_rows, col0;
  uint32_t prefetch_old_rows;   // split-K form: K/V tiles wholly below the call's new rows may be fetched before the predecessor ends
  uint32_t early_limit;         // ... and below this row (the call before may still be writing its own row)
  uint32_t pre_stages;          // ... and only this many K tiles (one fewer V tiles) before the q loads are in flight
  uint32_t kv_evict_first;      // split-K: 1 = the K / V tiles enter L2 as evict-first lines
  uint32_t q_tma;               // prefill, head_dim 256, f16 q: the CTA's 128 query rows come by TMA (tm_q); 2: the first
                                // q_rot_chunks 64-dim chunks of a head from tm_q (the rotated q), the others from tm_q2
                                // (the caller's own q, head stride q2_head_stride: unrotated dims are not copied anywhere)
  uint32_t q_rot_chunks; uint64_t q2_head_stride;
  uint32_t out_tma;             // prefill, f16 out: the CTA's output tile leaves through shared memory by one TMA store (tm_o)
};

}  // namespace pa
