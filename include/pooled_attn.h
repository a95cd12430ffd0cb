/*
 * pooled_attn.h — C ABI of libpooled_attn.so: pooled's GQA attention hot path on B200 (sm_100a).
 *
 * The library replaces the WebGPU dispatches that pooled's engines encode for one attention layer:
 * RoPE, f16 KV-cache append, split-K flash-decode / k-token verify, tiled causal prefill, the LSE
 * combine and the sigmoid output gate.  Each entry point below names the reference interface it
 * stands in for (paths inside the pooled repository).
 *
 * Conventions
 *   - plain C: opaque handles, raw device pointers, sizes and strides in ELEMENTS of the tensor's dtype.
 *   - every call returns PA_OK (0) or a negative pa_status; pa_last_error() gives the message.  There is
 *     no CPU fallback: an unsupported shape is PA_EUNSUPPORTED (the reference's config functions return
 *     null there, engine/wgsl/attn_dec.js:41), a missing or faulting GPU is PA_ECUDA.
 *   - calls enqueue work on the CUDA stream given (0 = the legacy default stream) and return without
 *     waiting, like WebGPU command encoding followed by queue.submit (engine/qwen35.js:4223); work on one
 *     stream runs in order.  A context is not thread-safe (the reference host is single-threaded).
 *   - activations (q, k, v, gate, out) are [column][...] arrays with an explicit column stride, as the
 *     reference's batched buffers are (FD.s0 / FD.s1, engine/wgsl/attn_dec.js:60).  Column c of a call at
 *     position pos is the token at position pos + c and attends cache rows [0, pos + c + 1).
 *   - caches are f16 [n_seqs][max_seq][n_kv_heads * head_dim], K and V separate, pairs little-endian
 *     (engine/wgsl/qwen35.js:889-906, engine/qwen35.js:1102-1104).
 */
#ifndef POOLED_ATTN_H
#define POOLED_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PA_API __attribute__((visibility("default")))

typedef enum pa_status {
  PA_OK = 0,
  PA_EINVAL = -1,       /* bad argument (null pointer, position past max_seq, misaligned stride ...) */
  PA_EUNSUPPORTED = -2, /* shape outside what the kernels cover */
  PA_ENOMEM = -3,       /* device allocation failed */
  PA_ECUDA = -4,        /* CUDA runtime / driver error, or no usable device */
  PA_ETIMEOUT = -5,     /* a bounded device-side wait ran out (reported by pa_sync / pa_check) */
  PA_ESTATE = -6        /* context latched after an earlier failure; pa_reset() clears it
                           (engine/qwen35.js:111-119: every method rejects until reset()) */
} pa_status;

typedef enum pa_dtype { PA_F32 = 0, PA_F16 = 1 } pa_dtype;

/* Cache formats of a layer.  pooled's engines keep f16 (Qwen35Engine's "flash" caches, the default here), int8 with one
 * f32 scale per 32 values (kvQ8: kv_store_q8 / attn_flash_q8, engine/wgsl/qwen35.js:97-139, :908-946) or f32 (the dense
 * engine, engine/wgsl/dense.js:22-136). */
typedef enum pa_kv_format { PA_KV_F16 = 0, PA_KV_Q8 = 1, PA_KV_F32 = 2 } pa_kv_format;

typedef enum pa_rope_mode {
  PA_ROPE_NONE = 0,  /* q and k arrive already rotated */
  PA_ROPE_F64 = 1,   /* angle pos * theta^(-2i/n_rot), cos/sin and products in float64, f32 result
                        (the arithmetic of tests/reference/ref_q38.mjs:67-79; the WGSL rope_part,
                        engine/wgsl/qwen35.js:386-404, evaluates the same formula in f32) */
  PA_ROPE_TABLE = 2  /* host-supplied f32 cos/sin table, f32 products rounded one by one
                        (the Flash engine: engine/qwen4exp.js:549-553, engine/wgsl/qwen4exp.js:545-548) */
} pa_rope_mode;

enum {
  PA_FLAG_FAST = 1u /* single-f16 tensor-core operands for q and the softmax weights instead of the
                        default hi+lo f16 pairs (about 2^-11 relative error on them instead of 2^-22) */
};

/* Shape and arithmetic of one model's attention layers.  Stands in for the engine's Config / DN uniform
 * blocks (engine/wgsl/base.js:4-8, engine/qwen35.js:822-832) and the attention options of
 * Qwen35Engine.create (engine/qwen35.js:266: attnDecodeSplits ...). */
typedef struct pa_config {
  uint32_t n_heads;     /* query heads */
  uint32_t n_kv_heads;  /* K/V heads; n_heads % n_kv_heads == 0 */
  uint32_t head_dim;    /* 64, 128 or 256 */
  uint32_t n_rot;       /* rotated dims per head (== head_dim for full RoPE); even, multiple of 2 */
  double rope_theta;
  uint32_t rope_mode;   /* pa_rope_mode */
  uint32_t act_dtype;   /* pa_dtype of q, k, v, gate and out buffers */
  uint32_t max_cols;    /* most columns one call may carry (decode / verify / prefill chunk) */
  uint32_t splits;      /* split-K CTAs per (sequence, kv head); 0 = sized to the GPU's SM count */
  uint32_t flags;       /* PA_FLAG_* */
  uint32_t reserved[5];
} pa_config;

typedef struct pa_ctx pa_ctx;     /* one per (device, model shape) */
typedef struct pa_layer pa_layer; /* one attention layer's K and V caches */

/* One unit of a batched decode: n_cols consecutive tokens of sequence seq, the first at position pos. */
typedef struct pa_item {
  uint32_t seq, pos, n_cols, reserved;
} pa_item;

/* ---- lifetime ------------------------------------------------------------------------------------ */

/* Replaces pipeline creation in Qwen35Engine._initAttnDec / _initAttnTile (engine/qwen35.js:1959-2019). */
PA_API int pa_create(int device, const pa_config* cfg, pa_ctx** out);
PA_API int pa_destroy(pa_ctx* ctx);
/* Replaces the per-layer cache allocation and bind groups (engine/qwen35.js:1102-1145).  Fails with a
 * readable message when the caches do not fit (engine/qwen35.js:378-383 throws at create as well). */
PA_API int pa_layer_create(pa_ctx* ctx, uint32_t n_seqs, uint32_t max_seq, pa_layer** out);
/* The same with the cache format chosen.  PA_KV_F16 is pa_layer_create.  PA_KV_Q8: int8 [n_seqs][max_seq][kv_dim] plus f32
 * scales [n_seqs][max_seq][kv_dim / 32]; the append is kv_store_q8's arithmetic bit for bit (scale = max|x| / 127 per 32
 * values, round to nearest even, clamp to +-127), attention dequantises value * scale as attn_flash_q8 does.
 * PA_KV_F32: f32 caches.  On such layers pa_kv_append, pa_rope_append, pa_decode (any n_cols, each column attended on
 * its own as the reference's kernels do), pa_prefill, pa_attn_layer(_host), pa_cache_export / _import work; the sharded
 * and gathered calls, pa_decode_partial and the slots are for f16 caches (PA_EUNSUPPORTED).  At most 16 query heads
 * per kv head.  These formats run a plain vector-load kernel, not the TMA / tensor-core ones of the f16 cache. */
PA_API int pa_layer_create_fmt(pa_ctx* ctx, uint32_t n_seqs, uint32_t max_seq, int kv_format, pa_layer** out);
PA_API int pa_layer_destroy(pa_layer* layer);
/* Declares this layer's caches a shard of longer sequences: cache row 0 holds global position `origin`.  Every
 * position passed to later calls stays global; appends must fall inside [origin, origin + max_seq), decode
 * partials cover the rows of [0, pos + c + 1) the shard holds (possibly none).  No counterpart in the reference. */
PA_API int pa_layer_set_origin(pa_layer* layer, uint32_t origin);
/* Tells the library which layer the engine runs after this one (NULL: unknown).  pooled's engines walk their layers in
 * a fixed order (the loop over layers in forwardToken, engine/qwen35.js:4214-4222, and the last layer is followed by the
 * first one of the next token), so the order is known when the layers are created.  A decode call on `layer` then asks
 * L2, once it has requested its own last K/V tile, for the first tiles the same call on `next` will read: HBM keeps
 * delivering while this call drains and the next one starts.  A hint only: results do not depend on it. */
PA_API int pa_layer_set_next(pa_layer* layer, pa_layer* next);
/* Device pointer of the K (which = 0) or V (1) cache, or of the K (2) / V (3) scales of a PA_KV_Q8 layer: what
 * _stateParts exports (engine/qwen35.js:129-141). */
PA_API void* pa_cache_ptr(pa_layer* layer, int which);
/* KV state of one sequence to and from the host: cache rows of global positions [pos0, pos1) x kv_dim f16, K (which = 0)
 * or V (1), row p at host + (p - pos0) * kv_dim * 2 bytes.  These are the parts _stateParts lists per full-attention
 * layer ({buf: kCache, bytes: pos * kvRow}, engine/qwen35.js:129-141) and exportState / importState move
 * (engine/qwen35.js:153-196).  On a shard (pa_layer_set_origin) only the rows the shard holds are copied, each to its
 * place in the same host image, so the ranks of a sharded sequence export disjoint ranges; rows_copied (may be NULL)
 * receives how many.  Asynchronous on `stream` (use pinned host memory and pa_sync before reading).  Other formats: a row
 * is kv_dim bytes (PA_KV_Q8) or kv_dim * 4 bytes (PA_KV_F32), and which = 2 / 3 are the K / V scales of a PA_KV_Q8 layer
 * (kv_dim / 32 * 4 bytes a row: the kScale / vScale parts of _stateParts). */
PA_API int pa_cache_export(pa_layer* layer, uint32_t seq, uint32_t pos0, uint32_t pos1, int which, void* host_dst,
                           uint32_t* rows_copied, void* stream);
PA_API int pa_cache_import(pa_layer* layer, uint32_t seq, uint32_t pos0, uint32_t pos1, int which, const void* host_src,
                           uint32_t* rows_copied, void* stream);
/* GPU-side checkpoints of one sequence's rows [0, pos) of a layer: saveSlot / loadSlot / exportSlot / dropSlot
 * (engine/qwen35.js:197-228, :157-165), copies on the device with no readback.  A slot costs two device buffers of
 * pos * kv_dim * 2 bytes; pa_slot_load writes them back (into any sequence index of a layer of the same context and
 * shard) and reports the saved position; pa_slot_export reads a slot back to the host without switching to it. */
typedef struct pa_slot pa_slot;
PA_API int pa_slot_save(pa_layer* layer, uint32_t seq, uint32_t pos, pa_slot** out, void* stream);
PA_API int pa_slot_load(pa_layer* layer, uint32_t seq, const pa_slot* slot, uint32_t* pos_out, void* stream);
PA_API int pa_slot_export(const pa_slot* slot, int which, void* host_dst, void* stream);
PA_API int pa_slot_info(const pa_slot* slot, uint32_t* pos, uint32_t* first_row, uint32_t* rows);
PA_API int pa_slot_drop(pa_slot* slot);
PA_API const char* pa_last_error(pa_ctx* ctx);
PA_API const char* pa_version(void);
/* Waits for the stream and reports a device-side failure (onSubmittedWorkDone, engine/qwen35.js:3859). */
PA_API int pa_sync(pa_ctx* ctx, void* stream);
PA_API int pa_reset(pa_ctx* ctx); /* engine.reset() after a failed step (engine/qwen35.js:111-119) */

/* Plain device / pinned-host memory for callers without a CUDA binding of their own
 * (device.createBuffer / queue.writeBuffer / mapAsync in the reference). */
PA_API int pa_alloc(pa_ctx* ctx, size_t bytes, void** dev_ptr);
PA_API int pa_free(pa_ctx* ctx, void* dev_ptr);
PA_API int pa_alloc_host(pa_ctx* ctx, size_t bytes, void** host_ptr);
PA_API int pa_free_host(pa_ctx* ctx, void* host_ptr);
PA_API int pa_upload(pa_ctx* ctx, void* dev_dst, const void* host_src, size_t bytes, void* stream);
PA_API int pa_download(pa_ctx* ctx, void* host_dst, const void* dev_src, size_t bytes, void* stream);

/* ---- host mirrors of the reference's split arithmetic ---------------------------------------------- */

/* attnDecConfig / decSplitLen / decSplits (engine/wgsl/attn_dec.js:40-48): the reference's own split rule,
 * kept so engine code that sizes buffers from it still works.  pa_dec_config returns the target split
 * count S, or 0 where the reference returns null. */
PA_API uint32_t pa_dec_config(uint32_t head_dim, uint32_t G, uint32_t n_kv, uint32_t splits);
PA_API uint32_t pa_dec_split_len(uint32_t s, uint32_t S);
PA_API uint32_t pa_dec_splits(uint32_t s, uint32_t S);
/* tileSplitLen (engine/wgsl/attn_tile.js:53-56). */
PA_API uint32_t pa_tile_split_len(uint32_t seq_end, uint32_t fa_split, uint32_t fa_splits, uint32_t target);
/* The split count this library uses for a call whose longest column sees n_rows cache rows. */
PA_API uint32_t pa_plan_splits(pa_ctx* ctx, uint32_t n_rows, uint32_t n_items);

/* ---- the path, step by step ------------------------------------------------------------------------ */

/* QK head-norm, the step before RoPE in the reference's attention glue.  Replaces the head_norm part of attn_glue /
 * attn_glue_kv (engine/wgsl/qwen35.js:1112-1122, engine/wgsl/layer_fuse.js:112-125) with the arithmetic of its CPU
 * twin (tests/reference/ref_q38.mjs:50-57, :163-164): per head, y = f32((x * inv) * w[d]), inv = 1/sqrt(mean(x^2) + eps),
 * the mean accumulated in float64 in index order.  x, y: act_dtype [n_cols][col_stride], head h at h * head_stride
 * (x == y allowed); w: f32 [head_dim] on the device (the q-norm or the k-norm weight).  A separate pass today: call it
 * on q and on k before pa_attn_layer / pa_rope_append. */
PA_API int pa_head_norm(pa_ctx* ctx, const void* x, uint64_t col_stride, uint64_t head_stride, uint32_t n_heads_x,
                        uint32_t n_cols, const float* w, double eps, void* y, uint64_t y_col_stride,
                        uint64_t y_head_stride, void* stream);
/* Gives a layer its QK head-norm weights (device, f32 [head_dim] each; both or neither; they stay the caller's).  From
 * then on pa_attn_layer / pa_attn_layer_host / pa_attn_step_host / pa_attn_layer_sharded on this layer apply
 * pa_head_norm to q and k first (one extra kernel per call, into scratch of the context), which makes the call the
 * whole of attn_glue_kv + attn core + gate (engine/wgsl/layer_fuse.js:87-146): q_full, k and v go in as the GEMVs
 * leave them.  Passing null weights turns it off.  The first call on a context allocates that scratch: make it outside
 * a stream capture. */
PA_API int pa_layer_set_head_norm(pa_layer* layer, const float* q_w, const float* k_w, double eps);

/* RoPE.  Replaces rope_part / rope_part_mc (engine/wgsl/qwen35.js:386-404, :858-875), the full-head rope
 * (engine/wgsl/base.js:154-172) and the rotation inside attn_glue (engine/wgsl/qwen35.js:1124-1131).
 * x: act_dtype [n_cols][col_stride], head h at h * head_stride; y: f32 [n_cols][y_col_stride] with heads
 * packed [n_heads_x][head_dim].  x == y is allowed when act_dtype is f32 and the layouts coincide.
 * cs_table (PA_ROPE_TABLE only): f32 [n_cols][n_rot], (cos, sin) per rotated pair. */
PA_API int pa_rope(pa_ctx* ctx, const void* x, uint64_t col_stride, uint64_t head_stride, uint32_t n_heads_x,
                   uint32_t pos, uint32_t n_cols, const float* cs_table, float* y, uint64_t y_col_stride,
                   void* stream);

/* KV append, conversion only: rows pos .. pos+n_cols-1 of sequence seq get the f16 round-to-nearest-even
 * image of k and v (already rotated).  Replaces kv_store (engine/wgsl/qwen35.js:889-906) and kvStoreRow
 * (engine/wgsl/qwen4exp.js:494-506).  Bit-exact. */
PA_API int pa_kv_append(pa_layer* layer, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* k,
                        const void* v, uint64_t col_stride, int dtype, void* stream);

/* Fused front of the path: rotate q into q_rot (f32 [n_cols][n_heads*head_dim]), rotate k, append k and
 * v.  Replaces attn_glue_kv minus the head norm (engine/wgsl/layer_fuse.js:87-146).  q_rot may be NULL:
 * the rotated q then stays in the context's own buffer, which a following pa_decode reads when its q is NULL. */
PA_API int pa_rope_append(pa_layer* layer, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* q,
                          uint64_t q_col_stride, uint64_t q_head_stride, const void* k, const void* v,
                          uint64_t kv_col_stride, const float* cs_table, float* q_rot, void* stream);
/* The same for one token of each of several sequences in one launch (the batched engine's per-column positions,
 * engine/wgsl/qwen4exp_batch.js:535-579): item i = (seq, pos, 1) owns row i of q, k, v and of q_rot.  Items whose
 * position lies outside this layer's shard (pa_layer_set_origin) get their q rotated and nothing appended.
 * At most 32 items; PA_ROPE_F64 or PA_ROPE_NONE. */
PA_API int pa_rope_append_items(pa_layer* layer, const pa_item* items, uint32_t n_items, const void* q,
                                uint64_t q_col_stride, uint64_t q_head_stride, const void* k, const void* v,
                                uint64_t kv_col_stride, float* q_rot, void* stream);

/* Decode / verify core + combine + gate.  Replaces attn_dec + attn_dec_combine(_g) + sigmoid_mul
 * (engine/wgsl/attn_dec.js:67-287, engine/wgsl/qwen35.js:406-416) as dispatched by _encodeLayerR
 * (engine/qwen35.js:1619-1640) and the attn_dec branch of _encAttnCore (:2494-2499).
 * q: rotated queries, dtype q_dtype, [total columns][q_col_stride]; the items' columns follow one another
 * in q, gate and out.  gate may be NULL; with an interleaved q_full buffer pass gate = q + head_dim and
 * the same strides (engine/wgsl/attn_dec.js:282-283).  n_cols * (n_heads / n_kv_heads) <= 64 per item.  q = NULL: the
 * rotated q that the preceding pa_rope_append / pa_rope_append_items call left in the context (its q_rot = NULL). */
PA_API int pa_decode(pa_layer* layer, const pa_item* items, uint32_t n_items, const void* q, int q_dtype,
                     uint64_t q_col_stride, uint64_t q_head_stride, const void* gate, uint64_t gate_col_stride,
                     uint64_t gate_head_stride, void* out, uint64_t out_col_stride, void* stream);

/* Gather mode of the decode (the QSA kernels: attn_dec with gather = stride, engine/wgsl/attn_dec.js:33-38, :67-70, :105,
 * :170-181, and attnDecMcWGSL({gather}), engine/wgsl/qwen4exp_batch.js:590-641): column c attends the cache rows its
 * list names instead of rows 0 .. seqLen-1.  row_lists: u32 on the device, list_stride words per column: [0] = n, then n
 * row indices of sequence seq, ascending (n <= list_stride - 1; every listed row is visible to the column).  List
 * position t stands where position t stands in the dense kernel, so the list 0 .. seqLen-1 gives the very bits
 * pa_decode gives for the same columns passed as one-column items.  The lengths stay on the device (the reference's
 * selection kernels write them there); the library sizes its grid for list_stride - 1 rows.  At most 32 columns a
 * call, at most 8 query heads per kv head.  An empty list gives zeros. */
PA_API int pa_decode_gather(pa_layer* layer, uint32_t seq, uint32_t n_cols, const uint32_t* row_lists, uint32_t list_stride,
                            const void* q, int q_dtype, uint64_t q_col_stride, uint64_t q_head_stride, const void* gate,
                            uint64_t gate_col_stride, uint64_t gate_head_stride, void* out, uint64_t out_col_stride,
                            void* stream);

/* The same, stopping before normalisation: one (o[head_dim], m, l) f32 record per (column, head) over the
 * rows this cache holds, for a KV sequence sharded across GPUs.  partial: f32 [rows * head_dim] holding o
 * (unnormalised), followed by f32 [rows][2] holding (m in natural-log units, l); rows = total columns *
 * n_heads, so one rank's records are rows * (head_dim + 2) contiguous floats.  No counterpart in the
 * reference (attention never leaves one device there); the record is the one attn_dec writes per split
 * (engine/wgsl/attn_dec.js:186-199). */
PA_API int pa_decode_partial(pa_layer* layer, const pa_item* items, uint32_t n_items, const void* q, int q_dtype,
                             uint64_t q_col_stride, uint64_t q_head_stride, float* partial, void* stream);

/* LSE merge of n_parts partial records per (column, head) + gate: out = sum o_s e^(m_s-M) / sum l_s e^(m_s-M).
 * parts: n_parts blocks laid out as pa_decode_partial writes them, one after another (what an all-gather
 * of the ranks' blocks produces).  The arithmetic of attn_dec_combine(_g) (engine/wgsl/attn_dec.js:215-287)
 * applied to per-GPU records. */
PA_API int pa_merge(pa_ctx* ctx, const float* parts, uint32_t n_parts, uint32_t n_cols, const void* gate,
                    uint64_t gate_col_stride, uint64_t gate_head_stride, void* out, uint64_t out_col_stride,
                    void* stream);

/* ---- KV-sequence-sharded decode with the merge fused over peer memory ---------------------------------------- */

/* Peer exchange set-up (one process per GPU of one box; no counterpart in the reference).  Each rank allocates one
 * exchange buffer of pa_exchange_bytes() with pa_shared_alloc (zeroed, with a 64-byte IPC handle to hand to the
 * other ranks over any channel), opens the other ranks' handles with pa_shared_open, and passes all `world`
 * pointers (its own included, in rank order) to pa_exchange_init.  max_rows bounds columns * n_heads of one call. */
PA_API size_t pa_exchange_bytes(pa_ctx* ctx, uint32_t world, uint32_t max_rows);
PA_API int pa_shared_alloc(pa_ctx* ctx, size_t bytes, void** dev_ptr, void* ipc_handle_out);
PA_API int pa_shared_open(pa_ctx* ctx, const void* ipc_handle, void** dev_ptr);
PA_API int pa_shared_close(pa_ctx* ctx, void* dev_ptr);
/* pa_exchange_init starts a session: it waits for the device, zeroes this rank's own buffer and the call counter, so
 * buffers may be reused after an earlier session.  Every rank must call it, and all ranks must pass a barrier of their
 * own (any channel) between their pa_exchange_init and the first exchanging call of any rank: peers write into this
 * rank's buffer from that call on. */
PA_API int pa_exchange_init(pa_ctx* ctx, uint32_t rank, uint32_t world, void* const* bufs, uint32_t max_rows);
/* Limit of the polling loop in which an exchanging call waits for the other ranks' records (sweeps over the missing
 * entries; 0 restores the built-in 2^20, about a second).  When it runs out the kernel records status 7, finishes with
 * what it has, and pa_sync reports PA_ETIMEOUT: a peer that died between steps costs one bounded wait, not a hang. */
PA_API int pa_set_wait_limit(pa_ctx* ctx, uint32_t sweeps);
/* pa_decode over this rank's shard with the cross-GPU merge inside the combine kernel: each CTA stores its merged
 * (o, m, l) slice into every rank's exchange buffer over NVLink, each value as one 8-byte {value, call tag} store,
 * spins (bounded) on its own buffer until the other ranks' entries carry the call's tag, merges and writes the gated
 * output.  Every rank must make the same call in the same order; every rank ends with the full result.  The
 * arithmetic is attn_dec_combine(_g)'s (engine/wgsl/attn_dec.js:215-287) applied to per-GPU records. */
PA_API int pa_decode_exchange(pa_layer* layer, const pa_item* items, uint32_t n_items, const void* q, int q_dtype,
                              uint64_t q_col_stride, uint64_t q_head_stride, const void* gate, uint64_t gate_col_stride,
                              uint64_t gate_head_stride, void* out, uint64_t out_col_stride, void* stream);

/* pa_attn_layer for a KV-sequence shard (pa_layer_set_origin + pa_exchange_init): RoPE on q everywhere, append of
 * k / v on the rank whose shard holds the new positions, decode over the local rows, cross-GPU merge and gate inside
 * the combine kernel.  Same call, same order, on every rank. */
PA_API int pa_attn_layer_sharded(pa_layer* layer, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* q,
                                 uint64_t q_col_stride, uint64_t q_head_stride, const void* k, const void* v,
                                 uint64_t kv_col_stride, const void* gate, uint64_t gate_col_stride,
                                 uint64_t gate_head_stride, const float* cs_table, void* out, uint64_t out_col_stride,
                                 void* stream);

/* One decode token of each of several sequences through a whole attention layer in one call: what the batched engine
 * dispatches per layer as attnPrep followed by the multi-column decode (engine/qwen4exp_batch.js:282-296,
 * engine/wgsl/qwen4exp_batch.js:590-641), i.e. pa_rope_append_items + pa_decode (or pa_decode_exchange) as one call.
 * items: one column each (item i = column i of q / k / v / gate / out, at its own sequence and position).
 * exchange != 0: KV-sequence shards (pa_layer_set_origin + pa_exchange_init; positions global; the rank that holds an
 * item's position appends its row; every rank ends with the full result; same call, same order, on every rank).
 * For the shapes of the decode kernel's fused front (head_dim 256 with 64 rotary dims, or head_dim 128 rotated in full,
 * at most 8 heads per kv head, PA_ROPE_F64) no RoPE/append kernel runs: each CTA rotates its item's q, and the CTA on an
 * item's last tile rotates k, rounds k / v to f16 and appends the row.  Same results, bit for bit, as the two-call form.
 * f16 caches only. */
PA_API int pa_attn_items(pa_layer* layer, const pa_item* items, uint32_t n_items, const void* q, uint64_t q_col_stride,
                         uint64_t q_head_stride, const void* k, const void* v, uint64_t kv_col_stride, const void* gate,
                         uint64_t gate_col_stride, uint64_t gate_head_stride, void* out, uint64_t out_col_stride,
                         int exchange, void* stream);

/* Tiled causal prefill of n_cols columns of one sequence starting at pos (their K/V already appended).
 * Replaces attn_flash_tile + attn_combine_tile + sigmoid_mul_mc (engine/wgsl/attn_tile.js:108-193,
 * engine/wgsl/qwen35.js:877-887) as dispatched by _encAttnCore (engine/qwen35.js:2489-2493, :2516). */
PA_API int pa_prefill(pa_layer* layer, uint32_t seq, uint32_t pos, uint32_t n_cols, const void* q, int q_dtype,
                      uint64_t q_col_stride, uint64_t q_head_stride, const void* gate, uint64_t gate_col_stride,
                      uint64_t gate_head_stride, void* out, uint64_t out_col_stride, void* stream);

/* Standalone gate: a[i] *= 1/(1+exp(-g[i])).  Replaces sigmoid_mul(_mc) (engine/wgsl/qwen35.js:406-416). */
PA_API int pa_sigmoid_mul(pa_ctx* ctx, void* a, uint64_t a_col_stride, const void* g, uint64_t g_col_stride,
                          uint64_t g_head_stride, uint32_t n_cols, void* stream);

/* ---- the path in one call --------------------------------------------------------------------------- */

enum { PA_MODE_AUTO = 0, PA_MODE_DECODE = 1, PA_MODE_PREFILL = 2 };

/* One attention layer for n_cols new tokens of one sequence: RoPE on q and k, append k and v, attend
 * (decode / verify kernel, or the tiled prefill kernel, chosen as _encAttnCore chooses: engine/qwen35.js:
 * 2485-2503), gate.  This is the attention block of _encodeLayerR / _encodeLayerBatch between the q/k/v
 * projections and the o projection (engine/qwen35.js:1598-1640, :2473-2517).  Device pointers. */
PA_API int pa_attn_layer(pa_layer* layer, uint32_t seq, uint32_t pos, uint32_t n_cols, int mode, const void* q,
                         uint64_t q_col_stride, uint64_t q_head_stride, const void* k, const void* v,
                         uint64_t kv_col_stride, const void* gate, uint64_t gate_col_stride,
                         uint64_t gate_head_stride, const float* cs_table, void* out, uint64_t out_col_stride,
                         void* stream);

/* The same with HOST buffers (pinned or pageable): inputs are copied to the device, the layer runs, out is
 * copied back; returns after the stream has drained.  For hosts that hand the library ArrayBuffers. */
PA_API int pa_attn_layer_host(pa_layer* layer, uint32_t seq, uint32_t pos, uint32_t n_cols, int mode,
                              const void* q, uint64_t q_col_stride, uint64_t q_head_stride, const void* k,
                              const void* v, uint64_t kv_col_stride, const void* gate, uint64_t gate_col_stride,
                              uint64_t gate_head_stride, const float* cs_table, void* out,
                              uint64_t out_col_stride, void* stream);

/* One token step through several attention layers with HOST buffers: q, k, v, gate and out are [n_layers][n_cols][...]
 * arrays (layer strides in elements); each array is uploaded once, the layers run back to back, out comes back in
 * one copy and the call returns when the stream has drained.  This is the granularity at which pooled's engine
 * touches the host: forwardToken encodes every layer, submits once and maps the result once
 * (engine/qwen35.js:4214-4228).  PA_ROPE_TABLE contexts are not supported here (use pa_attn_layer_host). */
PA_API int pa_attn_step_host(pa_layer* const* layers, uint32_t n_layers, uint32_t seq, uint32_t pos, uint32_t n_cols, int mode,
                             const void* q, uint64_t q_layer_stride, uint64_t q_col_stride, uint64_t q_head_stride, const void* k,
                             const void* v, uint64_t kv_layer_stride, uint64_t kv_col_stride, const void* gate,
                             uint64_t gate_layer_stride, uint64_t gate_col_stride, uint64_t gate_head_stride, void* out,
                             uint64_t out_layer_stride, uint64_t out_col_stride, void* stream);

/* Decode / verify + combine + gate for callers that cannot allocate device memory (code running inside a stream
 * capture, on a thread that must not block on the allocator, or handed raw device pointers by a host that owns the
 * memory pool): such a caller cannot create a pa_ctx / pa_layer, so everything arrives as plain pointers and the
 * per-split partial records live in a fixed array inside the library image (2048 records, about 2.1 MB held by every
 * GPU that loads the library until the process exits).  It has no counterpart in the reference.
 *   k_cache, v_cache: f16 [cache_rows][n_kv_heads*head_dim]; q (already rotated), gate (may be NULL), out: f32
 *   [n_cols][n_heads*head_dim]; columns at positions pos .. pos+n_cols-1, their K/V rows already in the caches.
 *   Limits: head_dim 128 or 256; n_cols * (n_heads / n_kv_heads) <= 64; n_cols * n_heads <= 2048 (the split count is
 *   lowered so that rows * splits fits the array).  Anything beyond is refused with PA_EUNSUPPORTED and a message.
 *   The first call on a device looks up the array's address and sets kernel attributes: make it outside any stream
 *   capture.  All calls on a device share the array (it keeps the last call's records, which are rewritten before they
 *   are read; the status word is cleared on the stream by each call), so calls that overlap on the GPU race: keep
 *   them on one stream or order them with events.  Calls no cudaMalloc / cudaFree / allocating routine.
 *   msg (may be NULL): receives the error text. */
PA_API int pa_decode_static(int device, const void* k_cache, const void* v_cache, uint32_t cache_rows, uint32_t n_heads,
                            uint32_t n_kv_heads, uint32_t head_dim, uint32_t pos, uint32_t n_cols, const float* q,
                            const float* gate, float* out, void* stream, char* msg, size_t msg_len);
/* Waits for `stream` and hands back the status word of pa_decode_static's bounded device-side waits on `device`
 * (0: all satisfied; then PA_OK, else PA_ETIMEOUT and the outputs of the calls since the last clear are not to be
 * trusted).  pa_decode_static clears the word at the start of each call, so ask before the next call.  A 4-byte copy out
 * of the same built-in array: allocates nothing.  Further notes on pa_decode_static: it makes `device` the calling
 * thread's current device and leaves it so; its one-time set-up is serialised between host threads; kernel attributes
 * are set the first time each row-count class (1-8, 9-16, 17-32, 33-64 query rows per kv head) is used on a device, so
 * the "first call outside a capture" rule holds per class. */
PA_API int pa_decode_static_status(int device, void* stream, uint32_t* word);

/* Counters since creation: what tests/bench_attn_ctx.js collects with timestamp queries. */
typedef struct pa_stats {
  uint64_t kernel_launches; /* this library's kernels launched */
  uint64_t kv_bytes_streamed; /* algorithmic K+V bytes of decode / verify / prefill calls */
  uint64_t calls;
} pa_stats;
PA_API int pa_get_stats(pa_ctx* ctx, pa_stats* out);

/* Device time of the core kernel (the split-K decode kernel, or the tiled prefill kernel) measured with CUDA
 * events recorded on the call's stream right around that launch: what the per-dispatch timestamp queries of
 * tests/bench_attn_ctx.js:39-70 give in the reference.  pa_timing_begin arms up to max_events launches;
 * pa_timing_end waits for them and returns their summed duration and count. */
PA_API int pa_timing_begin(pa_ctx* ctx, uint32_t max_events);
/* Profiling aid: while on, pa_attn_layer / pa_decode launch their core kernel only (no RoPE/append, no merge of the
 * split records), so that successive calls put core launches back to back, as tests/bench/attn_tile_bench.js times
 * one kernel alone.  Outputs are not produced while it is on, and nothing else may write the caches meanwhile: a
 * pa_attn_layer launch starts fetching K/V ahead of the previous launch's end, as it does inside a token step. */
PA_API int pa_set_core_only(pa_ctx* ctx, int on);
PA_API int pa_timing_end(pa_ctx* ctx, double* core_ms, uint64_t* core_launches);

#ifdef __cplusplus
}
#endif
#endif /* POOLED_ATTN_H */
