"""Host side of the attention path: the call surface pooled's engines use, over libpooled_attn.so.

Mirrors, by name and argument meaning:
  attn_dec_config / dec_split_len / dec_splits / DEC_CQ   engine/wgsl/attn_dec.js:40-51
  attn_tile_config / tile_split_len                        engine/wgsl/attn_tile.js:43-56
  AttnEngine.encode_layer                                  the attention block of Qwen35Engine._encodeLayerR
                                                           (engine/qwen35.js:1598-1640) and _encAttnGlue + _encAttnCore
                                                           (engine/qwen35.js:2473-2517)
torch is used for device memory and streams only; every computation is a call into the CUDA library.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import torch

from . import lib as _l

DEC_CQ = 4  # engine/wgsl/attn_dec.js:51


def attn_dec_config(hd: int, G: int, nKV: int, splits: int = 0, kvQ8: bool = False, R: int = 1):
    """attnDecConfig (engine/wgsl/attn_dec.js:40-44): None where the reference's split-K decode refuses the shape."""
    if kvQ8 or hd != 256 or not (1 <= G <= 8) or not R >= 1:
        return None
    S = int(splits) if splits > 0 else max(16, 256 // nKV)
    return {"HD": hd, "G": G, "S": S, "R": R}


def dec_split_len(s: int, S: int) -> int:
    """decSplitLen (engine/wgsl/attn_dec.js:47)."""
    return max(64, math.ceil(math.ceil(s / S) / 64) * 64)


def dec_splits(s: int, S: int) -> int:
    """decSplits (engine/wgsl/attn_dec.js:48)."""
    return math.ceil(s / dec_split_len(s, S))


def attn_tile_config(hd: int, G: int, faSplit: int, faSplits: int, wgMem: int = 16384, target: int = 32, tk: int = 0,
                     kvh: bool = False, pf: bool = False, nr: bool = False):
    """attnTileConfig (engine/wgsl/attn_tile.js:43-50)."""
    if not (hd % 16 == 0 and 16 <= hd <= 256 and 1 <= G <= 64):
        return None
    if faSplit % 64 != 0 or faSplits < 1:
        return None
    nbytes = lambda TK: TK * hd * 4 + TK * 256 * 4
    TK = tk or next((t for t in (16, 8, 4) if nbytes(t) <= wgMem), 0)
    if not TK or nbytes(TK) > wgMem:
        return None
    return {"HD": hd, "G": G, "CW": 64 // G, "TK": TK, "FASPLIT": faSplit, "FASPLITS": faSplits, "TARGET": max(1, int(target)),
            "KVH": bool(kvh), "PF": bool(pf), "NR": bool(nr)}


def tile_split_len(seqEnd: int, c: dict) -> int:
    """tileSplitLen (engine/wgsl/attn_tile.js:53-56)."""
    up64 = lambda x: math.ceil(x / 64) * 64
    return min(c["FASPLIT"], max(64, up64(math.ceil(seqEnd / c["TARGET"])), up64(math.ceil(seqEnd / c["FASPLITS"]))))


@dataclass
class AttnConfig:
    """Shape of a model's attention layers (Config / DN of the reference, engine/qwen35.js:822-832)."""
    n_heads: int
    n_kv_heads: int
    head_dim: int
    n_rot: int
    rope_theta: float
    max_seq: int
    n_layers: int = 1
    n_seqs: int = 1
    rope_mode: str = "f64"            # "none" | "f64" | "table"
    act_dtype: torch.dtype = torch.float16
    max_cols: int = 8
    splits: int = 0
    fast: bool = False
    link_layers: bool = True          # layers run in index order, the last one followed by the first (pa_layer_set_next)
    kv_format: str = "f16"            # "f16" | "q8" (engine option kvQ8: int8 + a scale per 32 values) | "f32" (the dense engine's caches)

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim


_ROPE = {"none": _l.PA_ROPE_NONE, "f64": _l.PA_ROPE_F64, "table": _l.PA_ROPE_TABLE}
_KVFMT = {"f16": _l.PA_KV_F16, "q8": _l.PA_KV_Q8, "f32": _l.PA_KV_F32}
_MODE = {"auto": _l.PA_MODE_AUTO, "decode": _l.PA_MODE_DECODE, "prefill": _l.PA_MODE_PREFILL}


def _dt(t: torch.dtype) -> int:
    if t == torch.float16:
        return _l.PA_F16
    if t == torch.float32:
        return _l.PA_F32
    raise _l.PaError(-1, f"dtype {t} is not supported (float16 or float32)")


class _DevArray:
    """A raw device pointer as something torch can wrap (for cache views)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}


class AttnEngine:
    """The attention part of an engine: per-layer f16 K/V caches and the per-layer attention step."""

    def __init__(self, cfg: AttnConfig, device: int = 0):
        self.cfg, self.device = cfg, device
        self.L = _l.load()
        pc = _l.PaConfig(n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, n_rot=cfg.n_rot, rope_theta=cfg.rope_theta,
                         rope_mode=_ROPE[cfg.rope_mode], act_dtype=_dt(cfg.act_dtype), max_cols=cfg.max_cols, splits=cfg.splits,
                         flags=_l.PA_FLAG_FAST if cfg.fast else 0)
        h = C.c_void_p()
        self.ctx = None
        self.layers: list[C.c_void_p] = []
        self.slots: dict[str, dict] = {}
        self._xc_keep = None
        self.L.check(self.L.pa_create(device, C.byref(pc), C.byref(h)))
        self.ctx = h
        try:
            for _ in range(cfg.n_layers):
                lh = C.c_void_p()
                self.L.check(self.L.pa_layer_create_fmt(self.ctx, cfg.n_seqs, cfg.max_seq, _KVFMT[cfg.kv_format], C.byref(lh)), self.ctx)
                self.layers.append(lh)
            if cfg.link_layers and cfg.n_layers > 1 and cfg.kv_format == "f16":
                for li, lh in enumerate(self.layers):
                    self.L.check(self.L.pa_layer_set_next(lh, self.layers[(li + 1) % cfg.n_layers]), self.ctx)
        except Exception:
            self.destroy()
            raise

    @classmethod
    def create(cls, cfg: AttnConfig, device: int = 0) -> "AttnEngine":
        return cls(cfg, device)

    # ---- plumbing ----
    def _st(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _ck(self, rc: int):
        self.L.check(rc, self.ctx)

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr()) if t is not None else None

    def destroy(self):
        if self.ctx:
            self.drop_all_slots()
            self._exchange_release()
        for lh in self.layers:
            self.L.pa_layer_destroy(lh)
        self.layers = []
        if self.ctx:
            self.L.pa_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def sync(self):
        self._ck(self.L.pa_sync(self.ctx, self._st()))

    def reset(self):
        self._ck(self.L.pa_reset(self.ctx))

    def stats(self) -> dict:
        s = _l.PaStats()
        self._ck(self.L.pa_get_stats(self.ctx, C.byref(s)))
        return {"kernel_launches": s.kernel_launches, "kv_bytes_streamed": s.kv_bytes_streamed, "calls": s.calls}

    def set_core_only(self, on: bool):
        """Profiling aid: layer / decode calls launch their core kernel only (outputs are not produced)."""
        self._ck(self.L.pa_set_core_only(self.ctx, 1 if on else 0))

    def timing_begin(self, max_events: int = 4096):
        self._ck(self.L.pa_timing_begin(self.ctx, max_events))

    def timing_end(self):
        """(summed device ms of the core kernel, launches timed) since timing_begin."""
        ms, n = C.c_double(), C.c_uint64()
        self._ck(self.L.pa_timing_end(self.ctx, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def plan_splits(self, n_rows: int, n_items: int = 1) -> int:
        return int(self.L.pa_plan_splits(self.ctx, n_rows, n_items))

    def set_origin(self, li: int, origin: int):
        """Layer li's caches hold global positions origin .. origin + max_seq - 1 (a KV-sequence shard)."""
        self._ck(self.L.pa_layer_set_origin(self.layers[li], origin))

    def cache(self, li: int, which: str) -> torch.Tensor:
        """The K ("k") or V ("v") cache of layer li as a tensor [n_seqs, max_seq, kv_dim] (no copy): int16 words of the
        f16 values, int8 values of a "q8" layer, float32 of an "f32" one."""
        ptr = self.L.pa_cache_ptr(self.layers[li], 0 if which == "k" else 1)
        ts = {"f16": "<i2", "q8": "|i1", "f32": "<f4"}[self.cfg.kv_format]
        arr = _DevArray(ptr, (self.cfg.n_seqs, self.cfg.max_seq, self.cfg.kv_dim), ts)
        return torch.as_tensor(arr, device=f"cuda:{self.device}")

    def cache_scales(self, li: int, which: str) -> torch.Tensor:
        """The scales of a "q8" layer's K or V cache: float32 [n_seqs, max_seq, kv_dim / 32]."""
        ptr = self.L.pa_cache_ptr(self.layers[li], 2 if which == "k" else 3)
        arr = _DevArray(ptr, (self.cfg.n_seqs, self.cfg.max_seq, self.cfg.kv_dim // 32), "<f4")
        return torch.as_tensor(arr, device=f"cuda:{self.device}")

    # ---- the path, step by step ----
    def rope(self, x: torch.Tensor, n_heads: int, pos: int, head_stride: int | None = None, cs_table: torch.Tensor | None = None) -> torch.Tensor:
        """RoPE of x [n_cols, stride] -> float32 [n_cols, n_heads * head_dim]."""
        n_cols = x.shape[0]
        y = torch.empty((n_cols, n_heads * self.cfg.head_dim), dtype=torch.float32, device=x.device)
        self._ck(self.L.pa_rope(self.ctx, self._p(x), x.stride(0), head_stride or self.cfg.head_dim, n_heads, pos, n_cols, self._p(cs_table),
                                self._p(y), y.stride(0), self._st()))
        return y

    def kv_append(self, li: int, seq: int, pos: int, k: torch.Tensor, v: torch.Tensor):
        assert k.dtype == v.dtype and k.stride(0) == v.stride(0)
        self._ck(self.L.pa_kv_append(self.layers[li], seq, pos, k.shape[0], self._p(k), self._p(v), k.stride(0), _dt(k.dtype), self._st()))

    def rope_append(self, li: int, seq: int, pos: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_head_stride: int | None = None,
                    cs_table: torch.Tensor | None = None) -> torch.Tensor:
        n_cols = q.shape[0]
        q_rot = torch.empty((n_cols, self.cfg.q_dim), dtype=torch.float32, device=q.device)
        self._ck(self.L.pa_rope_append(self.layers[li], seq, pos, n_cols, self._p(q), q.stride(0), q_head_stride or self.cfg.head_dim, self._p(k),
                                       self._p(v), k.stride(0), self._p(cs_table), self._p(q_rot), self._st()))
        return q_rot

    def rope_append_items(self, li: int, seqs_pos, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_head_stride: int | None = None) -> torch.Tensor:
        """One token of each of several sequences in one launch: seqs_pos = [(seq, pos)], row i of q / k / v belongs to
        item i.  Returns the rotated q, float32 [n_items, q_dim]."""
        n = len(seqs_pos)
        q_rot = torch.empty((n, self.cfg.q_dim), dtype=torch.float32, device=q.device)
        self._ck(self.L.pa_rope_append_items(self.layers[li], self._items([(s, p, 1) for s, p in seqs_pos]), n, self._p(q), q.stride(0),
                                             q_head_stride or self.cfg.head_dim, self._p(k), self._p(v), k.stride(0), self._p(q_rot), self._st()))
        return q_rot

    def encode_items(self, li: int, seqs_pos, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor | None = None,
                     out: torch.Tensor | None = None, sharded: bool = False, q_head_stride: int | None = None,
                     gate_head_stride: int | None = None) -> torch.Tensor:
        """One decode token of each of several sequences through the layer in one C-ABI call: seqs_pos = [(seq, pos)],
        row i of q / k / v / gate / out belongs to item i.  sharded: KV-sequence shards with the peer exchange."""
        n = len(seqs_pos)
        if out is None:
            out = torch.empty((n, self.cfg.q_dim), dtype=self.cfg.act_dtype, device=q.device)
        gp, gcs, ghs = self._gate(gate, gate_head_stride)
        self._ck(self.L.pa_attn_items(self.layers[li], self._items([(s, p, 1) for s, p in seqs_pos]), n, self._p(q), q.stride(0),
                                      q_head_stride or self.cfg.head_dim, self._p(k), self._p(v), k.stride(0), gp, gcs, ghs, self._p(out),
                                      out.stride(0), 1 if sharded else 0, self._st()))
        return out

    def _items(self, items):
        arr = (_l.PaItem * len(items))()
        for i, (seq, pos, n_cols) in enumerate(items):
            arr[i].seq, arr[i].pos, arr[i].n_cols = seq, pos, n_cols
        return arr

    def _gate(self, gate, gate_head_stride):
        if gate is None:
            return None, 0, 0
        return self._p(gate), gate.stride(0), gate_head_stride or self.cfg.head_dim

    def decode(self, li: int, items, q: torch.Tensor, gate: torch.Tensor | None = None, out: torch.Tensor | None = None,
               q_head_stride: int | None = None, gate_head_stride: int | None = None) -> torch.Tensor:
        """Decode / verify: items = [(seq, pos, n_cols)], q rotated, [total columns, stride]."""
        total = sum(it[2] for it in items)
        if out is None:
            out = torch.empty((total, self.cfg.q_dim), dtype=self.cfg.act_dtype, device=q.device)
        gp, gcs, ghs = self._gate(gate, gate_head_stride)
        self._ck(self.L.pa_decode(self.layers[li], self._items(items), len(items), self._p(q), _dt(q.dtype), q.stride(0),
                                  q_head_stride or self.cfg.head_dim, gp, gcs, ghs, self._p(out), out.stride(0), self._st()))
        return out

    def decode_gather(self, li: int, row_lists: torch.Tensor, q: torch.Tensor, gate: torch.Tensor | None = None, out: torch.Tensor | None = None,
                      seq: int = 0, q_head_stride: int | None = None, gate_head_stride: int | None = None) -> torch.Tensor:
        """Decode over listed cache rows (the QSA gather mode of attn_dec, engine/wgsl/attn_dec.js:33-38): row_lists is an
        int32 device tensor [n_cols, stride] holding per column its length n, then n rows ascending."""
        n_cols = q.shape[0]
        assert row_lists.dtype == torch.int32 and row_lists.is_cuda and row_lists.shape[0] == n_cols and row_lists.is_contiguous()
        if out is None:
            out = torch.empty((n_cols, self.cfg.q_dim), dtype=self.cfg.act_dtype, device=q.device)
        gp, gcs, ghs = self._gate(gate, gate_head_stride)
        self._ck(self.L.pa_decode_gather(self.layers[li], seq, n_cols, self._p(row_lists), row_lists.shape[1], self._p(q), _dt(q.dtype), q.stride(0),
                                         q_head_stride or self.cfg.head_dim, gp, gcs, ghs, self._p(out), out.stride(0), self._st()))
        return out

    def decode_partial(self, li: int, items, q: torch.Tensor, q_head_stride: int | None = None) -> torch.Tensor:
        """Per-(column, head) records over this cache's rows: float32 [rows*head_dim (o) + rows*2 (m, l)]."""
        total = sum(it[2] for it in items)
        rows = total * self.cfg.n_heads
        part = torch.empty(rows * (self.cfg.head_dim + 2), dtype=torch.float32, device=q.device)
        self._ck(self.L.pa_decode_partial(self.layers[li], self._items(items), len(items), self._p(q), _dt(q.dtype), q.stride(0),
                                          q_head_stride or self.cfg.head_dim, self._p(part), self._st()))
        return part

    def merge(self, parts: torch.Tensor, n_cols: int, gate: torch.Tensor | None = None, out: torch.Tensor | None = None,
              gate_head_stride: int | None = None) -> torch.Tensor:
        """LSE merge of parts [n_parts, rows*(head_dim+2)] + gate."""
        if out is None:
            out = torch.empty((n_cols, self.cfg.q_dim), dtype=self.cfg.act_dtype, device=parts.device)
        gp, gcs, ghs = self._gate(gate, gate_head_stride)
        self._ck(self.L.pa_merge(self.ctx, self._p(parts), parts.shape[0], n_cols, gp, gcs, ghs, self._p(out), out.stride(0), self._st()))
        return out

    def prefill(self, li: int, seq: int, pos: int, q: torch.Tensor, gate: torch.Tensor | None = None, out: torch.Tensor | None = None,
                q_head_stride: int | None = None, gate_head_stride: int | None = None) -> torch.Tensor:
        n_cols = q.shape[0]
        if out is None:
            out = torch.empty((n_cols, self.cfg.q_dim), dtype=self.cfg.act_dtype, device=q.device)
        gp, gcs, ghs = self._gate(gate, gate_head_stride)
        self._ck(self.L.pa_prefill(self.layers[li], seq, pos, n_cols, self._p(q), _dt(q.dtype), q.stride(0), q_head_stride or self.cfg.head_dim,
                                   gp, gcs, ghs, self._p(out), out.stride(0), self._st()))
        return out

    def set_head_norm(self, li: int, q_w: torch.Tensor | None, k_w: torch.Tensor | None, eps: float = 1e-6):
        """Layer li applies the QK head-norm inside encode_layer* from now on (weights: float32 [head_dim] on the device,
        kept alive here); None turns it off."""
        if q_w is not None:
            assert q_w.dtype == torch.float32 and k_w.dtype == torch.float32 and q_w.is_cuda and k_w.is_cuda
            assert q_w.numel() == self.cfg.head_dim and k_w.numel() == self.cfg.head_dim
        self._norm_w = getattr(self, "_norm_w", {})
        self._norm_w[li] = (q_w, k_w)
        self._ck(self.L.pa_layer_set_head_norm(self.layers[li], self._p(q_w), self._p(k_w), float(eps)))

    def head_norm(self, x: torch.Tensor, n_heads_x: int, w: torch.Tensor, eps: float, head_stride: int | None = None,
                  out: torch.Tensor | None = None) -> torch.Tensor:
        """QK head-norm of q or k before RoPE (the head_norm step of attn_glue, engine/wgsl/qwen35.js:1112-1122):
        x [n_cols, stride] of act_dtype, w float32 [head_dim] on the device; in place unless `out` is given."""
        assert w.dtype == torch.float32 and w.is_cuda and w.numel() == self.cfg.head_dim
        y = x if out is None else out
        hs = head_stride or self.cfg.head_dim
        self._ck(self.L.pa_head_norm(self.ctx, self._p(x), x.stride(0), hs, n_heads_x, x.shape[0], self._p(w), float(eps), self._p(y), y.stride(0),
                                     hs, self._st()))
        return y

    def sigmoid_mul(self, a: torch.Tensor, g: torch.Tensor, g_head_stride: int | None = None):
        self._ck(self.L.pa_sigmoid_mul(self.ctx, self._p(a), a.stride(0), self._p(g), g.stride(0), g_head_stride or self.cfg.head_dim,
                                       a.shape[0], self._st()))

    # ---- the path in one call ----
    def encode_layer(self, li: int, pos: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor | None = None,
                     out: torch.Tensor | None = None, seq: int = 0, mode: str = "auto", q_head_stride: int | None = None,
                     gate_head_stride: int | None = None, cs_table: torch.Tensor | None = None) -> torch.Tensor:
        """RoPE + append + attend + gate for q.shape[0] new tokens at positions pos.. (device tensors).

        One token is the attention block of _encodeLayerR (engine/qwen35.js:1598-1640); several are _encAttnGlue +
        _encAttnCore (engine/qwen35.js:2473-2517): all columns' K/V are appended before any column attends."""
        n_cols = q.shape[0]
        if out is None:
            out = torch.empty((n_cols, self.cfg.q_dim), dtype=self.cfg.act_dtype, device=q.device)
        gp, gcs, ghs = self._gate(gate, gate_head_stride)
        self._ck(self.L.pa_attn_layer(self.layers[li], seq, pos, n_cols, _MODE[mode], self._p(q), q.stride(0), q_head_stride or self.cfg.head_dim,
                                      self._p(k), self._p(v), k.stride(0), gp, gcs, ghs, self._p(cs_table), self._p(out), out.stride(0), self._st()))
        return out

    def encode_layer_host(self, li: int, pos: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor,
                          seq: int = 0, mode: str = "auto", q_head_stride: int | None = None, gate_head_stride: int | None = None,
                          cs_table: torch.Tensor | None = None) -> torch.Tensor:
        """The same with HOST tensors (pinned or pageable): copies in, runs, copies out, returns when done."""
        assert not q.is_cuda and not out.is_cuda
        n_cols = q.shape[0]
        gp, gcs, ghs = self._gate(gate, gate_head_stride)
        self._ck(self.L.pa_attn_layer_host(self.layers[li], seq, pos, n_cols, _MODE[mode], self._p(q), q.stride(0), q_head_stride or self.cfg.head_dim,
                                           self._p(k), self._p(v), k.stride(0), gp, gcs, ghs, self._p(cs_table), self._p(out), out.stride(0), self._st()))
        return out

    def encode_step_host(self, pos: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor,
                         seq: int = 0, mode: str = "auto", q_head_stride: int | None = None, gate_head_stride: int | None = None) -> torch.Tensor:
        """One token step through every layer with HOST tensors [n_layers, n_cols, ...]: one upload per tensor, the layers
        back to back, one download (forwardToken's submit-once / map-once, engine/qwen35.js:4214-4228)."""
        assert not q.is_cuda and not out.is_cuda and q.shape[0] == len(self.layers)
        arr = (C.c_void_p * len(self.layers))(*[lh.value for lh in self.layers])
        self._ck(self.L.pa_attn_step_host(arr, len(self.layers), seq, pos, q.shape[1], _MODE[mode], self._p(q), q.stride(0), q.stride(1),
                                          q_head_stride or self.cfg.head_dim, self._p(k), self._p(v), k.stride(0), k.stride(1), self._p(gate),
                                          gate.stride(0) if gate is not None else 0, gate.stride(1) if gate is not None else 0,
                                          gate_head_stride or self.cfg.head_dim, self._p(out), out.stride(0), out.stride(1), self._st()))
        return out

    # ---- session state: what the engine's exportState / importState / saveSlot / loadSlot move for its attention layers ----
    def state_signature(self) -> dict:
        """What a saved state must match to be loaded here (stateSignature, engine/qwen35.js:143-151, attention part)."""
        c = self.cfg
        return {"v": 1, "layers": c.n_layers, "kv": c.kv_format, "dims": [c.kv_dim, c.n_kv_heads, c.head_dim]}

    def _state_parts(self, pos: int):
        """_stateParts (engine/qwen35.js:129-141): per layer the K rows [0, pos) then the V rows [0, pos), then (kvQ8) the K
        and the V scales."""
        row = self.cfg.kv_dim * {"f16": 2, "q8": 1, "f32": 4}[self.cfg.kv_format]
        parts = [(li, which, pos * row) for li in range(len(self.layers)) for which in (0, 1)]
        if self.cfg.kv_format == "q8":
            parts = [x for li in range(len(self.layers)) for x in ((li, 0, pos * row), (li, 1, pos * row), (li, 2, pos * self.cfg.kv_dim // 32 * 4),
                                                                    (li, 3, pos * self.cfg.kv_dim // 32 * 4))]
        return parts

    def export_state(self, pos: int, seq: int = 0) -> dict:
        """exportState (engine/qwen35.js:153): {sig, pos, parts: [bytes]}, rows [0, pos) of every layer.  On a shard the
        parts hold this rank's rows at their place and zeros elsewhere; `held` says which rows are this rank's."""
        parts, held = [], []
        for li, which, nbytes in self._state_parts(pos):
            host = torch.zeros(max(nbytes, 1), dtype=torch.uint8).pin_memory()
            n = C.c_uint32()
            self._ck(self.L.pa_cache_export(self.layers[li], seq, 0, pos, which, C.c_void_p(host.data_ptr()), C.byref(n), self._st()))
            parts.append(host); held.append(n.value)
        self.sync()
        return {"sig": self.state_signature(), "pos": pos, "parts": [bytes(h[:nb].numpy()) for h, (_, _, nb) in zip(parts, self._state_parts(pos))],
                "held": held}

    def import_state(self, st: dict, seq: int = 0) -> int:
        """importState (engine/qwen35.js:181-196): refuses a state of another shape; returns the restored position."""
        if st["sig"] != self.state_signature():
            raise _l.PaError(-1, "saved state is for a different model, layer range or KV format")
        parts = self._state_parts(st["pos"])
        if len(parts) != len(st["parts"]) or any(nb != len(b) for (_, _, nb), b in zip(parts, st["parts"])):
            raise _l.PaError(-1, "saved state has the wrong shape")
        keep = []
        for (li, which, nbytes), b in zip(parts, st["parts"]):
            if not nbytes:
                continue
            host = torch.frombuffer(bytearray(b), dtype=torch.uint8).pin_memory()
            keep.append(host)
            self._ck(self.L.pa_cache_import(self.layers[li], seq, 0, st["pos"], which, C.c_void_p(host.data_ptr()), None, self._st()))
        self.sync()
        return st["pos"]

    def save_slot(self, name: str, pos: int, seq: int = 0):
        """saveSlot (engine/qwen35.js:200-211): a copy of rows [0, pos) of every layer on the device."""
        self.drop_slot(name)
        hs = []
        for lh in self.layers:
            h = C.c_void_p()
            self._ck(self.L.pa_slot_save(lh, seq, pos, C.byref(h), self._st()))
            hs.append(h)
        self.slots[name] = {"pos": pos, "handles": hs}

    def load_slot(self, name: str, seq: int = 0) -> int:
        """loadSlot (engine/qwen35.js:212-222): returns the slot's position."""
        sl = self.slots.get(name)
        if sl is None:
            raise _l.PaError(-1, "no saved slot " + name)
        for lh, h in zip(self.layers, sl["handles"]):
            self._ck(self.L.pa_slot_load(lh, seq, h, None, self._st()))
        return sl["pos"]

    def export_slot(self, name: str) -> dict:
        """exportSlot (engine/qwen35.js:157-165): a slot read back without switching to it."""
        sl = self.slots.get(name)
        if sl is None:
            raise _l.PaError(-1, "no saved slot " + name)
        parts = []
        for h in sl["handles"]:
            rows = C.c_uint32()
            self._ck(self.L.pa_slot_info(h, None, None, C.byref(rows)))
            for which in (0, 1):
                host = torch.zeros(max(rows.value * self.cfg.kv_dim * 2, 1), dtype=torch.uint8).pin_memory()
                self._ck(self.L.pa_slot_export(h, which, C.c_void_p(host.data_ptr()), self._st()))
                parts.append((host, rows.value * self.cfg.kv_dim * 2))
        self.sync()
        return {"sig": self.state_signature(), "pos": sl["pos"], "parts": [bytes(h[:nb].numpy()) for h, nb in parts]}

    def drop_slot(self, name: str):
        sl = self.slots.pop(name, None)
        if sl:
            for h in sl["handles"]:
                self.L.pa_slot_drop(h)

    def drop_all_slots(self):
        for k in list(self.slots):
            self.drop_slot(k)

    # ---- sharded decode with the merge over peer memory ----
    def exchange_setup(self, rank: int, world: int, dist=None, max_rows: int = 512):
        """Allocate this rank's exchange buffer, swap IPC handles with the other ranks (torch.distributed object
        all-gather; any channel would do) and open theirs.  world == 1 needs no peers."""
        nbytes = self.L.pa_exchange_bytes(self.ctx, world, max_rows)
        own, handle = C.c_void_p(), C.create_string_buffer(64)
        self._ck(self.L.pa_shared_alloc(self.ctx, nbytes, C.byref(own), handle))
        handles = [handle.raw]
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, handle.raw)
        ptrs = (C.c_void_p * world)()
        for r in range(world):
            if r == rank:
                ptrs[r] = own.value
            else:
                pp = C.c_void_p()
                self._ck(self.L.pa_shared_open(self.ctx, C.create_string_buffer(handles[r], 64), C.byref(pp)))
                ptrs[r] = pp.value
        self._exchange_release()   # buffers of an earlier session
        self._xc_keep = (own, ptrs, rank, world)
        self._ck(self.L.pa_exchange_init(self.ctx, rank, world, ptrs, max_rows))
        if world > 1:
            dist.barrier()   # nobody writes into a buffer that is not mapped yet

    def _exchange_release(self):
        if not self._xc_keep:
            return
        own, ptrs, rank, world = self._xc_keep
        torch.cuda.synchronize(self.device)
        for r in range(world):
            if r != rank and ptrs[r]:
                self.L.pa_shared_close(self.ctx, C.c_void_p(ptrs[r]))
        self.L.pa_free(self.ctx, own)
        self._xc_keep = None

    def set_wait_limit(self, sweeps: int):
        """Polling limit of the cross-GPU exchange wait (0: the built-in limit, about a second)."""
        self._ck(self.L.pa_set_wait_limit(self.ctx, sweeps))

    def decode_exchange(self, li: int, items, q: torch.Tensor, gate: torch.Tensor | None = None, out: torch.Tensor | None = None,
                        q_head_stride: int | None = None, gate_head_stride: int | None = None) -> torch.Tensor:
        """decode() over this rank's shard, merged across the ranks inside the combine kernel (peer stores + flags)."""
        total = sum(it[2] for it in items)
        if out is None:
            out = torch.empty((total, self.cfg.q_dim), dtype=self.cfg.act_dtype, device=q.device)
        gp, gcs, ghs = self._gate(gate, gate_head_stride)
        self._ck(self.L.pa_decode_exchange(self.layers[li], self._items(items), len(items), self._p(q), _dt(q.dtype), q.stride(0),
                                           q_head_stride or self.cfg.head_dim, gp, gcs, ghs, self._p(out), out.stride(0), self._st()))
        return out

    def encode_layer_sharded(self, li: int, pos: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor | None = None,
                             out: torch.Tensor | None = None, seq: int = 0, q_head_stride: int | None = None, gate_head_stride: int | None = None,
                             cs_table: torch.Tensor | None = None) -> torch.Tensor:
        """encode_layer on a KV-sequence shard: one C-ABI call per layer; the owner of the new rows appends, every rank
        decodes its rows, the combine kernel merges across the ranks (needs set_origin and exchange_setup)."""
        n_cols = q.shape[0]
        if out is None:
            out = torch.empty((n_cols, self.cfg.q_dim), dtype=self.cfg.act_dtype, device=q.device)
        gp, gcs, ghs = self._gate(gate, gate_head_stride)
        self._ck(self.L.pa_attn_layer_sharded(self.layers[li], seq, pos, n_cols, self._p(q), q.stride(0), q_head_stride or self.cfg.head_dim,
                                              self._p(k), self._p(v), k.stride(0), gp, gcs, ghs, self._p(cs_table), self._p(out), out.stride(0), self._st()))
        return out
