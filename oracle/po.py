"""Python face of the CPU oracle: a ctypes loader for libattn_oracle.so and an
independent NumPy restatement of the same arithmetic.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark.  The product package never imports it.

Reference citations are paths inside the pooled repository.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libattn_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "attn_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s", "libattn_oracle.so"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        u16p, f32p, f64p, u32p = (C.POINTER(C.c_uint16), C.POINTER(C.c_float), C.POINTER(C.c_double), C.POINTER(C.c_uint32))
        L.po_f16_rne.restype = C.c_uint16; L.po_f16_rne.argtypes = [C.c_float]
        L.po_f16_ties_up.restype = C.c_uint16; L.po_f16_ties_up.argtypes = [C.c_float]
        L.po_f16_flush.restype = C.c_uint16; L.po_f16_flush.argtypes = [C.c_double]
        L.po_h2f.restype = C.c_float; L.po_h2f.argtypes = [C.c_uint16]
        L.po_f16_rne_array.argtypes = [f32p, u16p, C.c_size_t]
        L.po_h2f_array.argtypes = [u16p, f32p, C.c_size_t]
        L.po_rope_neox_f64.argtypes = [f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_double, C.c_double]
        L.po_head_norm_f64.argtypes = [f32p, C.c_uint32, C.c_uint32, f32p, C.c_double]
        L.po_rope_ggml_f32.argtypes = [f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_double, C.c_double]
        L.po_rope_table_f32.argtypes = [f32p, C.c_uint32, C.c_double, C.c_double]
        L.po_kv_append.argtypes = [f32p, f32p, C.c_uint32, C.c_uint64, u16p, u16p]
        attn = [f32p, C.c_uint64, u16p, u16p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint32, f32p, C.c_uint64]
        L.po_attn_f64.argtypes = attn + [f64p, C.c_uint64]
        L.po_attn_f32ref.argtypes = attn + [f32p, C.c_uint64]
        L.po_attn_f32_fast.argtypes = attn + [f32p, C.c_uint64]
        L.po_attn_f64_kv32.argtypes = [f32p, C.c_uint64, f32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint32, f32p, C.c_uint64, f64p, C.c_uint64]
        L.po_kv_store_q8.argtypes = [f32p, C.c_uint32, C.POINTER(C.c_int8), f32p]
        L.po_dequant_q8.argtypes = [C.POINTER(C.c_int8), f32p, C.c_uint32, f32p]
        L.po_threads.restype = C.c_int
        L.po_set_threads.argtypes = [C.c_int]
        L.po_lse_merge.argtypes = [f64p, f64p, f64p, C.c_uint32, C.c_uint32, f64p]
        L.po_lcg_dec_next.restype = C.c_uint32; L.po_lcg_dec_next.argtypes = [u32p]
        L.po_lcg_tile_next.restype = C.c_uint32; L.po_lcg_tile_next.argtypes = [u32p]
        L.po_gen_attn_dec.argtypes = [u32p, C.c_uint64, u16p, u16p, C.c_uint64, f32p]
        L.po_gen_attn_tile.argtypes = [u32p, C.c_uint32, C.c_uint32, C.c_uint32, u16p, u16p, C.c_uint64, f32p]
        _lib = L
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


# ---------------------------------------------------------------- C oracle --

def f16_rne(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    h = np.empty(x.shape, dtype=np.uint16)
    lib().po_f16_rne_array(_p(x, C.c_float), _p(h, C.c_uint16), x.size)
    return h


def h2f(h: np.ndarray) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    x = np.empty(h.shape, dtype=np.float32)
    lib().po_h2f_array(_p(h, C.c_uint16), _p(x, C.c_float), h.size)
    return x


def head_norm_f64(vec: np.ndarray, heads: int, hd: int, w: np.ndarray, eps: float) -> np.ndarray:
    """QK head-norm on a copy: float32 [heads*hd], weight float32 [hd]."""
    v = np.ascontiguousarray(vec, dtype=np.float32).copy()
    ww = np.ascontiguousarray(w, dtype=np.float32)
    lib().po_head_norm_f64(_p(v, C.c_float), heads, hd, _p(ww, C.c_float), float(eps))
    return v


def np_head_norm(vec: np.ndarray, heads: int, hd: int, w: np.ndarray, eps: float) -> np.ndarray:
    """NumPy twin of head_norm_f64 (cumsum adds in index order, as the serial loop does)."""
    x = np.asarray(vec, dtype=np.float32).reshape(heads, hd).astype(np.float64)
    ss = np.cumsum(x * x, axis=1)[:, -1]
    inv = 1.0 / np.sqrt(ss / hd + eps)
    return ((x * inv[:, None]) * np.asarray(w, dtype=np.float32).astype(np.float64)[None, :]).astype(np.float32).reshape(-1)


def rope_neox_f64(vec: np.ndarray, heads: int, hd: int, n_rot: int, pos: int, theta: float) -> np.ndarray:
    """In-place on a copy: float32 [heads*hd]."""
    v = np.ascontiguousarray(vec, dtype=np.float32).copy()
    lib().po_rope_neox_f64(_p(v, C.c_float), heads, hd, n_rot, float(pos), float(theta))
    return v


def rope_ggml_f32(vec, heads, hd, n_rot, pos, base):
    v = np.ascontiguousarray(vec, dtype=np.float32).copy()
    lib().po_rope_ggml_f32(_p(v, C.c_float), heads, hd, n_rot, float(pos), float(base))
    return v


def rope_table_f32(n_rot, pos, base):
    cs = np.empty(n_rot, dtype=np.float32)
    lib().po_rope_table_f32(_p(cs, C.c_float), n_rot, float(pos), float(base))
    return cs


def _attn(fn, out_dtype, q, k_cache, v_cache, n_heads, n_kv, hd, pos0, n_cols, gate=None):
    q = np.ascontiguousarray(q, dtype=np.float32)
    assert q.ndim == 2 and q.shape[0] >= n_cols
    k_cache = np.ascontiguousarray(k_cache, dtype=np.uint16)
    v_cache = np.ascontiguousarray(v_cache, dtype=np.uint16)
    out = np.zeros((n_cols, n_heads * hd), dtype=out_dtype)
    if gate is not None:
        gate = np.ascontiguousarray(gate, dtype=np.float32)
        gp, gs = _p(gate, C.c_float), gate.shape[1]
    else:
        gp, gs = None, 0
    fn(_p(q, C.c_float), q.shape[1], _p(k_cache, C.c_uint16), _p(v_cache, C.c_uint16), n_heads, n_kv, hd, pos0, n_cols,
       gp, gs, _p(out, C.c_double if out_dtype == np.float64 else C.c_float), out.shape[1])
    return out


def attn_f64(q, k_cache, v_cache, n_heads, n_kv, hd, pos0, n_cols, gate=None):
    """Exact causal GQA attention in float64; q float32 [n_cols][stride>=nH*hd], caches uint16 [rows][nKV*hd]."""
    return _attn(lib().po_attn_f64, np.float64, q, k_cache, v_cache, n_heads, n_kv, hd, pos0, n_cols, gate)


def attn_f32ref(q, k_cache, v_cache, n_heads, n_kv, hd, pos0, n_cols, gate=None):
    return _attn(lib().po_attn_f32ref, np.float32, q, k_cache, v_cache, n_heads, n_kv, hd, pos0, n_cols, gate)


def attn_f32_fast(q, k_cache, v_cache, n_heads, n_kv, hd, pos0, n_cols, gate=None):
    return _attn(lib().po_attn_f32_fast, np.float32, q, k_cache, v_cache, n_heads, n_kv, hd, pos0, n_cols, gate)


def kv_store_q8(x: np.ndarray):
    """kv_store_q8 of rows x [..., n] (n % 32 == 0): (int8 values, f32 scales [..., n / 32])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.zeros(x.shape, dtype=np.int8); sc = np.zeros(x.shape[:-1] + (x.shape[-1] // 32,), dtype=np.float32)
    lib().po_kv_store_q8(_p(x, C.c_float), x.size, _p(q, C.c_int8), _p(sc, C.c_float))
    return q, sc


def np_kv_store_q8(x: np.ndarray):
    """NumPy twin of kv_store_q8 (engine/wgsl/qwen35.js:908-946)."""
    x = np.asarray(x, dtype=np.float32)
    b = x.reshape(x.shape[:-1] + (x.shape[-1] // 32, 32))
    sc = (np.abs(b).max(axis=-1) / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(sc > 0, np.float32(1.0) / sc, np.float32(0.0)).astype(np.float32)
    q = np.clip(np.rint((b * inv[..., None]).astype(np.float32)), -127, 127).astype(np.int8)
    return q.reshape(x.shape), sc


def dequant_q8(q: np.ndarray, sc: np.ndarray) -> np.ndarray:
    """value * scale in f32, the order attn_flash_q8 reads them in (engine/wgsl/qwen35.js:117-120)."""
    return (q.astype(np.float32).reshape(sc.shape + (32,)) * sc[..., None]).astype(np.float32).reshape(q.shape)


def attn_f64_kv32(q, k_cache, v_cache, n_heads, n_kv, hd, pos0, n_cols, gate=None):
    """attn_f64 over float32 K/V values [rows][nKV*hd] (an f32 cache, or a dequantised int8 one)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k_cache = np.ascontiguousarray(k_cache, dtype=np.float32); v_cache = np.ascontiguousarray(v_cache, dtype=np.float32)
    out = np.zeros((n_cols, n_heads * hd), dtype=np.float64)
    if gate is not None:
        gate = np.ascontiguousarray(gate, dtype=np.float32)
        gp, gs = _p(gate, C.c_float), gate.shape[1]
    else:
        gp, gs = None, 0
    lib().po_attn_f64_kv32(_p(q, C.c_float), q.shape[1], _p(k_cache, C.c_float), _p(v_cache, C.c_float), n_heads, n_kv, hd, pos0, n_cols, gp, gs,
                           _p(out, C.c_double), out.shape[1])
    return out


def threads() -> int:
    return int(lib().po_threads())


def set_threads(n: int) -> int:
    """Host threads the threaded oracle functions use from now on; returns the count in effect."""
    lib().po_set_threads(int(n))
    return threads()


def gen_attn_dec(seed: int, max_seq: int, kv_dim: int, q_dim: int, n_cols: int = 4):
    """One run() of tests/test_attn_dec.js:38-45; returns (K, V, q, new_seed)."""
    s = C.c_uint32(seed)
    K = np.empty(max_seq * kv_dim, dtype=np.uint16); V = np.empty_like(K)
    q = np.empty(n_cols * q_dim, dtype=np.float32)
    lib().po_gen_attn_dec(C.byref(s), K.size, _p(K, C.c_uint16), _p(V, C.c_uint16), q.size, _p(q, C.c_float))
    return K.reshape(max_seq, kv_dim), V.reshape(max_seq, kv_dim), q.reshape(n_cols, q_dim), s.value


def gen_attn_tile(seed: int, max_seq: int, kv_dim: int, seq_end: int, n_cols: int, s0: int):
    """check() of tests/unit/attn_tile_test.js:43-52; returns (K, V, q[n_cols][s0], new_seed)."""
    s = C.c_uint32(seed)
    K = np.empty(max_seq * kv_dim, dtype=np.uint16); V = np.empty_like(K)
    q = np.empty(n_cols * s0, dtype=np.float32)
    lib().po_gen_attn_tile(C.byref(s), max_seq, kv_dim, seq_end, _p(K, C.c_uint16), _p(V, C.c_uint16), q.size, _p(q, C.c_float))
    return K.reshape(max_seq, kv_dim), V.reshape(max_seq, kv_dim), q.reshape(n_cols, s0), s.value


# -------------------------------------------------------------- NumPy twin --
# Written independently of the C file (vectorised, different evaluation order
# inside float64 sums) so that an error in one restatement shows up as a
# disagreement.  f16 conversion here is NumPy's own IEEE implementation.

def np_f16_rne(x) -> np.ndarray:
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def np_h2f(h) -> np.ndarray:
    return np.asarray(h, dtype=np.uint16).view(np.float16).astype(np.float32)


def np_rope_neox(vec, heads, hd, n_rot, pos, theta) -> np.ndarray:
    """tests/reference/ref_q38.mjs:67-79 / ref_qwen.mjs:32-44 in vectorised float64."""
    v = np.asarray(vec, dtype=np.float32).reshape(heads, hd).astype(np.float64)
    half = n_rot // 2
    i = np.arange(half, dtype=np.float64)
    ang = float(pos) * np.power(float(theta), -(2.0 * i) / float(n_rot))
    c, s = np.cos(ang), np.sin(ang)
    a, b = v[:, :half].copy(), v[:, half:n_rot].copy()
    v[:, :half] = a * c - b * s
    v[:, half:n_rot] = b * c + a * s
    return v.astype(np.float32).reshape(-1)


def np_attn_f64(q, k_cache, v_cache, n_heads, n_kv, hd, pos0, n_cols, gate=None) -> np.ndarray:
    """tests/test_attn_dec.js:72-82 in vectorised float64."""
    G = n_heads // n_kv
    out = np.zeros((n_cols, n_heads * hd), dtype=np.float64)
    Kf = np_h2f(k_cache).astype(np.float64)
    Vf = np_h2f(v_cache).astype(np.float64)
    for c in range(n_cols):
        n = pos0 + c + 1
        for h in range(n_heads):
            g = h // G
            qh = np.asarray(q[c, h * hd:(h + 1) * hd], dtype=np.float64)
            sc = Kf[:n, g * hd:(g + 1) * hd] @ qh / np.sqrt(float(hd))
            p = np.exp(sc - sc.max())
            o = (p @ Vf[:n, g * hd:(g + 1) * hd]) / p.sum()
            if gate is not None:
                o = o * (1.0 / (1.0 + np.exp(-np.asarray(gate[c, h * hd:(h + 1) * hd], dtype=np.float64))))
            out[c, h * hd:(h + 1) * hd] = o
    return out


# ------------------------------------------------ seeded synthetic inputs --
# Counter-based generator shared by tests and the benchmark: splitmix64 of
# (seed, index) -> two uniforms -> Box-Muller in float64.  Stands in for the
# reference's chat / code prompts run through real weights, which are absent.

def _splitmix64(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def normal(seed: int, n: int, offset: int = 0) -> np.ndarray:
    """n draws of N(0,1) in float64, a pure function of (seed, offset + index)."""
    with np.errstate(over="ignore"):
        idx = np.arange(offset, offset + n, dtype=np.uint64)
        base = _splitmix64(np.full(1, seed, dtype=np.uint64))[0]
        a = _splitmix64(base ^ (idx * np.uint64(2)))
        b = _splitmix64(base ^ (idx * np.uint64(2) + np.uint64(1)))
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740993.0
    u2 = (b >> np.uint64(11)).astype(np.float64) / 9007199254740992.0
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def outlier_channels(head: int, hd: int, count: int = 4) -> list[int]:
    """`count` distinct channel indices of one head, a pure function of the head index."""
    out: list[int] = []
    k = 0
    with np.errstate(over="ignore"):
        while len(out) < count:
            c = int(_splitmix64(np.array([0x0071E2 * 1000003 + head * 131 + k], dtype=np.uint64))[0] % np.uint64(hd))
            if c not in out:
                out.append(c)
            k += 1
    return out
