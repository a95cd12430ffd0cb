"""The CPU oracle against independent implementations and the reference tests' own facts (no GPU)."""
import numpy as np
import pytest

from oracle import po


def test_f16_rne_every_half_and_midpoint():
    # every f16 value converts back to itself; every midpoint between neighbours rounds to even;
    # one f32 ulp either side of a midpoint rounds to the nearer neighbour (tests/test_qsa.js:76-119 runs
    # the same sweep on the GPU helper)
    h = np.arange(65536, dtype=np.uint16)
    f = po.h2f(h)
    assert np.array_equal(po.np_h2f(h).view(np.uint32)[~np.isnan(f)], f.view(np.uint32)[~np.isnan(f)])
    finite = np.isfinite(f)
    assert np.array_equal(po.f16_rne(f[finite]), h[finite])
    pos = h[(h < 0x7bff)]
    lo, hi = po.h2f(pos).astype(np.float64), po.h2f(pos + 1).astype(np.float64)
    mid = ((lo + hi) / 2).astype(np.float32)   # exact in f32
    want = np.where(pos & 1, pos + 1, pos).astype(np.uint16)
    assert np.array_equal(po.f16_rne(mid), want)
    assert np.array_equal(po.f16_rne(-mid), want | 0x8000)
    up = np.nextafter(mid, np.float32(np.inf)); dn = np.nextafter(mid, np.float32(-np.inf))
    assert np.array_equal(po.f16_rne(up), pos + 1)
    assert np.array_equal(po.f16_rne(dn), pos)


def test_f16_rne_matches_ieee_on_random_bits():
    rng = np.random.default_rng(7)
    x = rng.integers(0, 2**32, size=2_000_000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    a, b = po.f16_rne(x), po.np_f16_rne(x)
    nan = np.isnan(x)
    assert np.array_equal(a[~nan], b[~nan])
    assert np.all((a[nan] & 0x7c00) == 0x7c00) and np.all((a[nan] & 0x200) != 0)   # quiet NaN
    # edges: overflow to inf, smallest subnormal, underflow to zero
    L = po.lib()
    assert L.po_f16_rne(65520.0) == 0x7c00 and L.po_f16_rne(65519.0) == 0x7bff
    assert L.po_f16_rne(2.0**-24) == 1 and L.po_f16_rne(2.0**-25) == 0 and L.po_f16_rne(np.nextafter(np.float32(2.0**-25), np.float32(1))) == 1


def test_f16_ties_up_known_answers():
    L = po.lib()
    # engine/gguf.js:33-35: a mantissa that rounds up must carry into the exponent (-1.99999 -> -2, not -1)
    assert L.po_f16_ties_up(-1.99999) == 0xC000
    assert L.po_f16_ties_up(1.0) == 0x3C00 and L.po_f16_ties_up(2.0) == 0x4000 and L.po_f16_ties_up(0.5) == 0x3800
    # a tie goes up in magnitude where RNE goes to even: 1 + 2^-11 sits between 0x3c00 (even) and 0x3c01
    t = np.float32(1.0 + 2.0**-11)
    assert L.po_f16_ties_up(t) == 0x3C01 and L.po_f16_rne(t) == 0x3C00


def test_f16_flush_drops_subnormals():
    L = po.lib()
    assert L.po_f16_flush(3e-6) == 0 and L.po_f16_flush(-3e-6) == 0x8000      # tests/test_attn_dec.js:25 "if (e <= 0) return s"
    assert L.po_f16_flush(0.3) == po.np_f16_rne(np.float32(0.3))


def test_lcg_generators_first_values():
    # first values computed by hand from the recurrences in tests/test_attn_dec.js:22-23 and
    # tests/unit/attn_tile_test.js:16-17 (Python integers / floats follow the same IEEE rules as JS numbers)
    import ctypes as C
    s = C.c_uint32(12345)
    py = 12345
    for _ in range(1000):
        py = (py * 1664525 + 1013904223) % 2**32
        assert po.lib().po_lcg_dec_next(C.byref(s)) == py
    s = C.c_uint32(12345)
    js = 12345
    wrap = 12345
    differs = False
    for _ in range(1000):
        x = float(js) * 1103515245.0 + 12345.0      # IEEE double, as JS evaluates it
        js = int(x % 4294967296.0)
        wrap = (wrap * 1103515245 + 12345) % 2**32  # what integer wraparound would give
        differs |= js != wrap
        assert po.lib().po_lcg_tile_next(C.byref(s)) == js
    assert differs, "the double-rounded sequence must differ from integer wraparound"


def test_gen_attn_dec_layout():
    K, V, q, seed = po.gen_attn_dec(12345, 8, 512, 4096)
    s = 12345
    def rnd():
        nonlocal s
        s = (s * 1664525 + 1013904223) % 2**32
        return s / 2**32 - 0.5
    k0 = np.float32(rnd() * 0.6); v0 = np.float32(rnd() * 2); k1 = np.float32(rnd() * 0.6)
    assert K[0, 0] == po.np_f16_rne(k0) and V[0, 0] == po.np_f16_rne(v0) and K[0, 1] == po.np_f16_rne(k1)
    assert q.dtype == np.float32 and np.all(np.abs(q) <= 2.0) and np.abs(po.h2f(K)).max() <= 0.3 + 1e-3


@pytest.mark.parametrize("hd,n_rot,theta,pos", [(128, 128, 1e6, 4096), (256, 64, 1e7, 32768), (256, 64, 1e7, 131072), (64, 32, 1e4, 0)])
def test_rope_c_vs_numpy(hd, n_rot, theta, pos):
    v = po.normal(11, 6 * hd).astype(np.float32)
    a = po.rope_neox_f64(v, 6, hd, n_rot, pos, theta)
    b = po.np_rope_neox(v, 6, hd, n_rot, pos, theta)
    # two libm-based evaluations; identical up to an occasional last-place flip of the f32 store
    assert np.max(np.abs(a.astype(np.float64) - b)) <= 1.5e-7 * max(1.0, np.abs(v).max())
    assert np.array_equal(a.reshape(6, hd)[:, n_rot:], v.reshape(6, hd)[:, n_rot:])   # dims past n_rot untouched
    if pos == 0:
        assert np.array_equal(a, v)


def test_rope_ggml_recurrence():
    # theta_i accumulates in f32: tests/reference/qsa_ref.mjs:99-110
    cs = po.rope_table_f32(64, 1000, 1e7)
    ts = np.float32(np.power(1e7, -2.0 / 64))
    th = np.float32(1000.0)
    for i in range(32):
        assert cs[2 * i] == np.float32(np.cos(np.float64(th))) and cs[2 * i + 1] == np.float32(np.sin(np.float64(th)))
        th = np.float32(th * ts)
    v = po.normal(5, 2 * 256).astype(np.float32)
    r = po.rope_ggml_f32(v, 2, 256, 64, 1000, 1e7)
    a, b = v[:32], v[32:64]
    assert np.array_equal(r[:32], a * cs[0::2] - b * cs[1::2]) and np.array_equal(r[32:64], a * cs[1::2] + b * cs[0::2])


@pytest.mark.parametrize("nH,nKV,hd,pos0,nc", [(16, 2, 256, 0, 1), (16, 2, 256, 130, 4), (24, 4, 256, 63, 5), (16, 8, 128, 200, 1), (8, 2, 64, 17, 8)])
def test_attn_c_vs_numpy(nH, nKV, hd, pos0, nc):
    rows = pos0 + nc
    K = po.np_f16_rne(po.normal(1, rows * nKV * hd) * 0.6).reshape(rows, nKV * hd)
    V = po.np_f16_rne(po.normal(2, rows * nKV * hd)).reshape(rows, nKV * hd)
    q = po.normal(3, nc * (nH * hd + 12)).astype(np.float32).reshape(nc, nH * hd + 12)
    g = po.normal(4, nc * nH * hd).astype(np.float32).reshape(nc, nH * hd)
    for gate in (None, g):
        a = po.attn_f64(q, K, V, nH, nKV, hd, pos0, nc, gate)
        b = po.np_attn_f64(q, K, V, nH, nKV, hd, pos0, nc, gate)
        assert np.max(np.abs(a - b)) < 1e-12
        c = po.attn_f32ref(q, K, V, nH, nKV, hd, pos0, nc, gate)
        d = po.attn_f32_fast(q, K, V, nH, nKV, hd, pos0, nc, gate)
        assert np.max(np.abs(c - a)) < 2e-5 and np.max(np.abs(d - a)) < 2e-5


def test_attn_never_reads_past_the_column_limit():
    # rows at or past a column's own position hold NaN: tests/unit/attn_tile_test.js:43-49
    K, V, q, _ = po.gen_attn_tile(12345, 64, 2 * 64, 20, 4, 8 * 64 + 12)
    assert np.all(K[20:] == 0x7e00) and not np.any(K[:20] == 0x7e00)
    out = po.attn_f64(q, K, V, 8, 2, 64, 16, 4)
    assert np.all(np.isfinite(out))
    # column 0 sees rows [0, 17): poisoning rows 17.. must not change it
    K2, V2 = K.copy(), V.copy(); K2[17:] = 0x7e00; V2[17:] = 0x7e00
    assert np.array_equal(po.attn_f64(q, K2, V2, 8, 2, 64, 16, 1)[0], out[0])


def test_lse_merge_equals_one_pass():
    import ctypes as C
    rng = np.random.default_rng(3)
    n, hd = 300, 64
    s = rng.normal(size=n) * 3; v = rng.normal(size=(n, hd))
    p = np.exp(s - s.max()); want = p @ v / p.sum()
    parts = [(0, 64), (64, 200), (200, 300)]
    o = np.zeros((3, hd)); m = np.zeros(3); l = np.zeros(3)
    for i, (a, b) in enumerate(parts):
        m[i] = s[a:b].max(); w = np.exp(s[a:b] - m[i]); l[i] = w.sum(); o[i] = w @ v[a:b]
    out = np.zeros(hd)
    d = lambda a: a.ctypes.data_as(C.POINTER(C.c_double))
    po.lib().po_lse_merge(d(o), d(m), d(l), 3, hd, d(out))
    assert np.max(np.abs(out - want)) < 1e-13


def test_normal_generator_is_counter_based():
    a = po.normal(42, 1000)
    assert np.array_equal(po.normal(42, 100, offset=300), a[300:400])
    assert abs(a.mean()) < 0.15 and 0.85 < a.std() < 1.15
    b = po.normal(9, 200000)
    assert abs(b.mean()) < 0.01 and abs(b.std() - 1) < 0.01
    ch = po.outlier_channels(3, 256)
    assert len(set(ch)) == 4 and all(0 <= c < 256 for c in ch) and ch == po.outlier_channels(3, 256)


def test_head_norm_c_and_numpy_twins_agree_and_normalise():
    # tests/reference/ref_q38.mjs:50-57: with unit weights the output has mean square 1 (up to eps)
    rng = np.random.default_rng(4)
    for hd, heads in ((128, 8), (256, 16)):
        x = (rng.standard_normal(heads * hd) * 5).astype(np.float32)
        w = (1 + 0.2 * rng.standard_normal(hd)).astype(np.float32)
        a = po.head_norm_f64(x, heads, hd, w, 1e-6)
        b = po.np_head_norm(x, heads, hd, w, 1e-6)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        u = po.head_norm_f64(x, heads, hd, np.ones(hd, np.float32), 1e-6).reshape(heads, hd).astype(np.float64)
        assert np.allclose((u * u).mean(axis=1), 1.0, atol=1e-5)


def test_kv_store_q8_c_and_numpy_agree_and_follow_the_reference_rule():
    # kv_store_q8 (engine/wgsl/qwen35.js:908-946): scale = max|x| / 127 per 32 values, round to nearest even, clamp
    x = (po.normal(77, 200 * 512) * 3).astype(np.float32).reshape(200, 512)
    x[0, :32] = 0.0; x[1, 32:64] = 1e-30; x[2, 5] = 1e6; x[3, :32] = np.arange(32) - 15.5
    q, sc = po.kv_store_q8(x); q2, sc2 = po.np_kv_store_q8(x)
    assert np.array_equal(q, q2) and np.array_equal(sc.view(np.uint32), sc2.view(np.uint32))
    assert np.all(q[0, :32] == 0) and sc[0, 0] == 0.0                       # all-zero block: inv = 0
    assert np.abs(q).max() == 127 and q.min() >= -127                        # the block maximum maps to +-127, never -128
    b = x[3, :32]; s = np.float32(np.abs(b).max() / np.float32(127.0))
    assert np.array_equal(q[3, :32], np.clip(np.rint(b * (np.float32(1.0) / s)), -127, 127).astype(np.int8))
    d = po.dequant_q8(q, sc)
    assert np.all(np.abs(d - x) <= sc.repeat(32, axis=-1) * 0.5 * 1.0001 + 1e-30)   # within half a step of every value


def test_attn_f64_over_f32_values_is_the_same_definition():
    K = po.np_f16_rne(po.normal(2, 100 * 512)).reshape(100, 512); V = po.np_f16_rne(po.normal(3, 100 * 512)).reshape(100, 512)
    q = po.normal(4, 2 * 16 * 256).astype(np.float32).reshape(2, -1); g = po.normal(5, 2 * 16 * 256).astype(np.float32).reshape(2, -1)
    a = po.attn_f64(q, K, V, 16, 2, 256, 98, 2, g); b = po.attn_f64_kv32(q, po.np_h2f(K), po.np_h2f(V), 16, 2, 256, 98, 2, g)
    assert np.array_equal(a, b)
