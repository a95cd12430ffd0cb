// pooled_attn.js — Deno FFI binding of libpooled_attn.so (include/pooled_attn.h) and the attention call surface
// pooled's engines use, on top of it.
//
// Where it goes in pooled: engine/native/pooled_attn.js, imported by Qwen35Engine when attnDecode / attnPrefillTile
// are "native" (engine/qwen35.js:399-419 holds the switches this adds a value to).  Every export of the library is
// in the table below with the argument order of the header; device pointers are Deno pointer objects (or null),
// host buffers are TypedArrays.  Node: the same table works with koffi / ffi-napi, or a small N-API addon that
// dlopens the library and forwards BigInt pointers.
//
// This file has not been executed in the build image (no JavaScript runtime there); the same ABI is exercised through
// Python ctypes (pooled_b200/lib.py) by the GPU tests, and a test checks this table's names against the header.
const P = "pointer", BUF = "buffer", U32 = "u32", U64 = "u64", I32 = "i32";

export const SYMBOLS = {
  pa_create: { parameters: [I32, BUF, BUF], result: I32 },
  pa_destroy: { parameters: [P], result: I32 },
  pa_layer_create: { parameters: [P, U32, U32, BUF], result: I32 },
  pa_layer_create_fmt: { parameters: [P, U32, U32, I32, BUF], result: I32 },
  pa_layer_destroy: { parameters: [P], result: I32 },
  pa_layer_set_origin: { parameters: [P, U32], result: I32 },
  pa_layer_set_next: { parameters: [P, P], result: I32 },
  pa_cache_ptr: { parameters: [P, I32], result: P },
  pa_cache_export: { parameters: [P, U32, U32, U32, I32, BUF, BUF, P], result: I32 },
  pa_cache_import: { parameters: [P, U32, U32, U32, I32, BUF, BUF, P], result: I32 },
  pa_slot_save: { parameters: [P, U32, U32, BUF, P], result: I32 },
  pa_slot_load: { parameters: [P, U32, P, BUF, P], result: I32 },
  pa_slot_export: { parameters: [P, I32, BUF, P], result: I32 },
  pa_slot_info: { parameters: [P, BUF, BUF, BUF], result: I32 },
  pa_slot_drop: { parameters: [P], result: I32 },
  pa_last_error: { parameters: [P], result: P },
  pa_version: { parameters: [], result: P },
  pa_sync: { parameters: [P, P], result: I32, nonblocking: true },
  pa_reset: { parameters: [P], result: I32 },
  pa_alloc: { parameters: [P, U64, BUF], result: I32 },
  pa_free: { parameters: [P, P], result: I32 },
  pa_alloc_host: { parameters: [P, U64, BUF], result: I32 },
  pa_free_host: { parameters: [P, P], result: I32 },
  pa_upload: { parameters: [P, P, BUF, U64, P], result: I32 },
  pa_download: { parameters: [P, BUF, P, U64, P], result: I32 },
  pa_dec_config: { parameters: [U32, U32, U32, U32], result: U32 },
  pa_dec_split_len: { parameters: [U32, U32], result: U32 },
  pa_dec_splits: { parameters: [U32, U32], result: U32 },
  pa_tile_split_len: { parameters: [U32, U32, U32, U32], result: U32 },
  pa_plan_splits: { parameters: [P, U32, U32], result: U32 },
  pa_rope: { parameters: [P, P, U64, U64, U32, U32, U32, P, P, U64, P], result: I32 },
  pa_kv_append: { parameters: [P, U32, U32, U32, P, P, U64, I32, P], result: I32 },
  pa_rope_append: { parameters: [P, U32, U32, U32, P, U64, U64, P, P, U64, P, P, P], result: I32 },
  pa_rope_append_items: { parameters: [P, BUF, U32, P, U64, U64, P, P, U64, P, P], result: I32 },
  pa_decode: { parameters: [P, BUF, U32, P, I32, U64, U64, P, U64, U64, P, U64, P], result: I32 },
  pa_decode_gather: { parameters: [P, U32, U32, P, U32, P, I32, U64, U64, P, U64, U64, P, U64, P], result: I32 },
  pa_decode_partial: { parameters: [P, BUF, U32, P, I32, U64, U64, P, P], result: I32 },
  pa_merge: { parameters: [P, P, U32, U32, P, U64, U64, P, U64, P], result: I32 },
  pa_exchange_bytes: { parameters: [P, U32, U32], result: U64 },
  pa_shared_alloc: { parameters: [P, U64, BUF, BUF], result: I32 },
  pa_shared_open: { parameters: [P, BUF, BUF], result: I32 },
  pa_shared_close: { parameters: [P, P], result: I32 },
  pa_exchange_init: { parameters: [P, U32, U32, BUF, U32], result: I32 },
  pa_decode_exchange: { parameters: [P, BUF, U32, P, I32, U64, U64, P, U64, U64, P, U64, P], result: I32 },
  pa_attn_items: { parameters: [P, P, U32, P, U64, U64, P, P, U64, P, U64, U64, P, U64, I32, P], result: I32 },
  pa_attn_layer_sharded: { parameters: [P, U32, U32, U32, P, U64, U64, P, P, U64, P, U64, U64, P, P, U64, P], result: I32 },
  pa_prefill: { parameters: [P, U32, U32, U32, P, I32, U64, U64, P, U64, U64, P, U64, P], result: I32 },
  pa_sigmoid_mul: { parameters: [P, P, U64, P, U64, U64, U32, P], result: I32 },
  pa_layer_set_head_norm: { parameters: [P, P, P, "f64"], result: I32 },
  pa_head_norm: { parameters: [P, P, U64, U64, U32, U32, P, "f64", P, U64, U64, P], result: I32 },
  pa_attn_layer: { parameters: [P, U32, U32, U32, I32, P, U64, U64, P, P, U64, P, U64, U64, P, P, U64, P], result: I32 },
  pa_attn_layer_host: { parameters: [P, U32, U32, U32, I32, BUF, U64, U64, BUF, BUF, U64, BUF, U64, U64, BUF, BUF, U64, P], result: I32, nonblocking: true },
  pa_attn_step_host: { parameters: [BUF, U32, U32, U32, U32, I32, BUF, U64, U64, U64, BUF, BUF, U64, U64, BUF, U64, U64, U64, BUF, U64, U64, P], result: I32, nonblocking: true },
  pa_decode_static: { parameters: [I32, P, P, U32, U32, U32, U32, U32, U32, P, P, P, P, BUF, U64], result: I32 },
  pa_decode_static_status: { parameters: [I32, P, BUF], result: I32, nonblocking: true },
  pa_set_wait_limit: { parameters: [P, U32], result: I32 },
  pa_get_stats: { parameters: [P, BUF], result: I32 },
  pa_timing_begin: { parameters: [P, U32], result: I32 },
  pa_set_core_only: { parameters: [P, I32], result: I32 },
  pa_timing_end: { parameters: [P, BUF, BUF], result: I32 },
};

export const PA_F32 = 0, PA_F16 = 1;
export const PA_ROPE_NONE = 0, PA_ROPE_F64 = 1, PA_ROPE_TABLE = 2;
export const PA_MODE_AUTO = 0, PA_MODE_DECODE = 1, PA_MODE_PREFILL = 2;
export const PA_FLAG_FAST = 1;
const STATUS = { 0: "PA_OK", [-1]: "PA_EINVAL", [-2]: "PA_EUNSUPPORTED", [-3]: "PA_ENOMEM", [-4]: "PA_ECUDA", [-5]: "PA_ETIMEOUT", [-6]: "PA_ESTATE" };

let lib = null;
export function load(path = new URL("./libpooled_attn.so", import.meta.url)) {
  if (!lib) lib = Deno.dlopen(path, SYMBOLS);   // throws when the library is missing: there is no WGSL fallback behind "native"
  return lib.symbols;
}

// pa_config: u32 n_heads, n_kv_heads, head_dim, n_rot; f64 rope_theta; u32 rope_mode, act_dtype, max_cols, splits, flags, reserved[5]
export function paConfig({ nH, nKV, hd, nRot, theta, ropeMode = PA_ROPE_F64, f16 = false, maxCols = 16, splits = 0, flags = 0 }) {
  const b = new ArrayBuffer(64), u = new Uint32Array(b), f = new Float64Array(b);
  u.set([nH, nKV, hd, nRot]); f[2] = theta; u.set([ropeMode, f16 ? PA_F16 : PA_F32, maxCols, splits, flags], 6);
  return new Uint8Array(b);
}
// pa_item[]: u32 seq, pos, n_cols, reserved
export function paItems(items) {
  const u = new Uint32Array(4 * items.length);
  items.forEach(([seq, pos, nCols], i) => u.set([seq, pos, nCols, 0], 4 * i));
  return u;
}
// Failures read like the engine's own ("say what to do", engine/qwen35.js:381-382).
export function check(rc, ctx = null) {
  if (rc === 0) return;
  const msg = new Deno.UnsafePointerView(load().pa_last_error(ctx)).getCString();
  const e = new Error(`pooled_attn: ${msg} (${STATUS[rc] ?? rc})`);
  e.code = rc;
  throw e;
}
const outPtr = () => new BigUint64Array(1);
const asPtr = (a) => Deno.UnsafePointer.create(a[0]);

// The attention part of an engine: per-layer f16 K/V caches on the GPU and the per-layer attention step.
// Mirrors what _encodeLayerR's attention block and _encAttnGlue + _encAttnCore do (engine/qwen35.js:1598-1640,
// :2473-2517), with the same argument meaning: q_full [nCols][nH][2*hd] (q and gate interleaved), k, v [nCols][kvDim].
export class NativeAttention {
  constructor({ nH, nKV, hd, nRot, theta, maxSeq, nLayers, nSeqs = 1, f16 = false, maxCols = 16, device = 0 }) {
    const S = load();
    this.S = S; this.dims = { nH, nKV, hd, qDim: nH * hd, kvDim: nKV * hd }; this.es = f16 ? 2 : 4;
    const h = outPtr();
    check(S.pa_create(device, paConfig({ nH, nKV, hd, nRot, theta, f16, maxCols }), new Uint8Array(h.buffer)));
    this.ctx = asPtr(h);
    this.layers = [];
    for (let i = 0; i < nLayers; i++) {
      const lh = outPtr();
      check(S.pa_layer_create(this.ctx, nSeqs, maxSeq, new Uint8Array(lh.buffer)), this.ctx);   // throws with the MiB needed when it does not fit
      this.layers.push(asPtr(lh));
    }
    // the engine walks its layers in order, the last one followed by the first of the next token
    if (nLayers > 1) this.layers.forEach((L, i) => check(S.pa_layer_set_next(L, this.layers[(i + 1) % nLayers]), this.ctx));
    this.slots = new Map();
  }
  // device memory for the engine's q_full / k / v / attnOut when it has no CUDA binding of its own
  alloc(bytes) { const p = outPtr(); check(this.S.pa_alloc(this.ctx, BigInt(bytes), new Uint8Array(p.buffer)), this.ctx); return asPtr(p); }
  free(ptr) { this.S.pa_free(this.ctx, ptr); }
  upload(dst, src, stream = null) { check(this.S.pa_upload(this.ctx, dst, src, BigInt(src.byteLength), stream), this.ctx); }
  download(dst, src, stream = null) { check(this.S.pa_download(this.ctx, dst, src, BigInt(dst.byteLength), stream), this.ctx); }
  setHeadNorm(li, qNormW, kNormW, eps) { check(this.S.pa_layer_set_head_norm(this.layers[li], qNormW, kNormW, eps), this.ctx); }

  // One attention layer for nCols new tokens at pos: head-norm (if set), RoPE, append, attend, gate.  qFull is the q
  // projection's output with q and gate interleaved per head (engine/wgsl/attn_dec.js:282-283); verify passes say
  // mode = PA_MODE_DECODE, everything else PA_MODE_AUTO (engine/qwen35.js:2489-2499).
  encodeLayer(li, pos, nCols, qFull, k, v, out, { seq = 0, mode = PA_MODE_AUTO, gated = true, csTable = null, stream = null } = {}) {
    const { hd, qDim, kvDim } = this.dims, qs = gated ? 2n * BigInt(qDim) : BigInt(qDim), hs = gated ? 2n * BigInt(hd) : BigInt(hd);
    const gate = gated ? Deno.UnsafePointer.offset(qFull, hd * this.es) : null;
    check(this.S.pa_attn_layer(this.layers[li], seq, pos, nCols, mode, qFull, qs, hs, k, v, BigInt(kvDim), gate, qs, hs, csTable, out, BigInt(qDim), stream), this.ctx);
  }
  // The same with host TypedArrays; resolves when the result is in `out` (queue.onSubmittedWorkDone + mapAsync in one).
  async encodeLayerHost(li, pos, nCols, qFull, k, v, out, { seq = 0, mode = PA_MODE_AUTO, gated = true, csTable = null, stream = null } = {}) {
    const { hd, qDim, kvDim } = this.dims, qs = gated ? 2n * BigInt(qDim) : BigInt(qDim), hs = gated ? 2n * BigInt(hd) : BigInt(hd);
    const gate = gated ? qFull.subarray(hd) : null;
    check(await this.S.pa_attn_layer_host(this.layers[li], seq, pos, nCols, mode, qFull, qs, hs, k, v, BigInt(kvDim), gate, qs, hs, csTable, out, BigInt(qDim), stream), this.ctx);
  }
  // One token step through every layer with host arrays [nLayers][nCols][...]: forwardToken's submit-once / map-once
  // (engine/qwen35.js:4214-4228).
  async encodeStepHost(pos, nCols, qFull, k, v, out, { seq = 0, mode = PA_MODE_AUTO, gated = true, stream = null } = {}) {
    const { hd, qDim, kvDim } = this.dims, qc = gated ? 2 * qDim : qDim, hs = BigInt(gated ? 2 * hd : hd);
    const lp = new BigUint64Array(this.layers.map((L) => BigInt(Deno.UnsafePointer.value(L))));
    const gate = gated ? qFull.subarray(hd) : null;
    check(await this.S.pa_attn_step_host(new Uint8Array(lp.buffer), this.layers.length, seq, pos, nCols, mode, qFull, BigInt(nCols * qc), BigInt(qc), hs, k, v,
      BigInt(nCols * kvDim), BigInt(kvDim), gate, BigInt(nCols * qc), BigInt(qc), hs, out, BigInt(nCols * qDim), BigInt(qDim), stream), this.ctx);
  }
  // A batch of sequences decoding one token each (engine/qwen4exp_batch.js:268-296): items = [[seq, pos], ...];
  // one library call per layer (RoPE, append, decode, gate); sharded = KV-sequence shards with the peer exchange
  decodeBatch(li, items, q, k, v, gate, out, { sharded = false, stream = null } = {}) {
    const { hd, qDim, kvDim } = this.dims, it = paItems(items.map(([s, p]) => [s, p, 1]));
    check(this.S.pa_attn_items(this.layers[li], new Uint8Array(it.buffer), items.length, q, BigInt(qDim), BigInt(hd), k, v, BigInt(kvDim), gate, BigInt(qDim), BigInt(hd),
      out, BigInt(qDim), sharded ? 1 : 0, stream), this.ctx);
  }
  async sync(stream = null) { check(await this.S.pa_sync(this.ctx, stream), this.ctx); }
  reset() { check(this.S.pa_reset(this.ctx), this.ctx); }   // after a failed step every call rejects until here (engine/qwen35.js:111-119)

  // ---- session state: exportState / importState / saveSlot / loadSlot for the attention layers (engine/qwen35.js:129-228) ----
  stateSignature() { const d = this.dims; return { v: 1, layers: this.layers.length, kv: "f16", dims: [d.kvDim, d.nKV, d.hd] }; }
  async exportState(pos, seq = 0) {
    const parts = [];
    for (const L of this.layers) for (const which of [0, 1]) {
      const b = new Uint8Array(pos * this.dims.kvDim * 2);
      if (b.length) check(this.S.pa_cache_export(L, seq, 0, pos, which, b, null, null), this.ctx);
      parts.push(b);
    }
    await this.sync();
    return { sig: this.stateSignature(), pos, parts: parts.map((p) => p.buffer) };
  }
  async importState(st, seq = 0) {
    if (JSON.stringify(st.sig) !== JSON.stringify(this.stateSignature())) throw new Error("saved state is for a different model, layer range or KV format");
    if (st.parts.length !== 2 * this.layers.length || st.parts.some((p) => p.byteLength !== st.pos * this.dims.kvDim * 2)) throw new Error("saved state has the wrong shape");
    this.layers.forEach((L, i) => [0, 1].forEach((which) => {
      const b = new Uint8Array(st.parts[2 * i + which]);
      if (b.length) check(this.S.pa_cache_import(L, seq, 0, st.pos, which, b, null, null), this.ctx);
    }));
    await this.sync();
    return st.pos;
  }
  saveSlot(name, pos, seq = 0) {
    this.dropSlot(name);
    const hs = this.layers.map((L) => { const h = outPtr(); check(this.S.pa_slot_save(L, seq, pos, new Uint8Array(h.buffer), null), this.ctx); return asPtr(h); });
    this.slots.set(name, { pos, hs });
  }
  loadSlot(name, seq = 0) {
    const sl = this.slots.get(name);
    if (!sl) throw new Error("no saved slot " + name);
    this.layers.forEach((L, i) => check(this.S.pa_slot_load(L, seq, sl.hs[i], null, null), this.ctx));
    return sl.pos;
  }
  dropSlot(name) { const sl = this.slots.get(name); if (!sl) return; this.slots.delete(name); sl.hs.forEach((h) => this.S.pa_slot_drop(h)); }

  destroy() {
    for (const k of [...this.slots.keys()]) this.dropSlot(k);
    this.layers.forEach((L) => this.S.pa_layer_destroy(L));
    this.S.pa_destroy(this.ctx);
    this.layers = []; this.ctx = null;
  }
}
