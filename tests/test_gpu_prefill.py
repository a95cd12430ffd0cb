"""Tiled causal prefill (tcgen05 + TMEM) on the GPU against the float64 oracle, through the C ABI."""
import numpy as np
import pytest

from oracle import po
from tests import util

pytestmark = pytest.mark.gpu


def _engine(nH, nKV, hd, max_seq, act="f32", max_cols=1024, n_rot=64, theta=1e7, rope_mode="none", n_seqs=1):
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    return AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=theta, max_seq=max_seq, n_seqs=n_seqs,
                                 rope_mode=rope_mode, act_dtype=torch.float32 if act == "f32" else torch.float16, max_cols=max_cols))


# ---- the reference's own tile test, retargeted: tests/unit/attn_tile_test.js:118-131 --------------------------------
# (all six cases, in the reference's order: the LCG seed carries over from case to case)
TILE_CASES = [
    dict(name="MoE shape, first pass", hd=256, nH=16, nKV=2, nc=16, basePos=0, maxSeq=512),
    dict(name="MoE shape, 5 splits, partial tile", hd=256, nH=16, nKV=2, nc=16, basePos=301, maxSeq=4096),
    dict(name="27B shape, 2 big splits", hd=256, nH=24, nKV=4, nc=16, basePos=173, maxSeq=512),
    dict(name="27B shape, TK 16", hd=256, nH=24, nKV=4, nc=16, basePos=90, maxSeq=4096),
    dict(name="small head, 1 split target", hd=64, nH=8, nKV=2, nc=16, basePos=219, maxSeq=2048),
    dict(name="8-column batch", hd=128, nH=12, nKV=2, nc=8, basePos=77, maxSeq=1024),
]


def test_attn_tile_js_cases():
    import torch
    seed = 12345
    for t in TILE_CASES:
        hd, nH, nKV, nc, base, max_seq = t["hd"], t["nH"], t["nKV"], t["nc"], t["basePos"], t["maxSeq"]
        s0, s1 = nH * hd + 12, nH * hd + 20                       # padded column strides (attn_tile_test.js:51)
        K, V, q, seed = po.gen_attn_tile(seed, max_seq, nKV * hd, base + nc, nc, s0)
        eng = _engine(nH, nKV, hd, max_seq, act="f32", max_cols=64)
        util.load_cache(eng, 0, 0, K, V)                          # rows at or past base + nc hold the NaN pattern 0x7e00
        out = torch.full((nc, s1), float("nan"), device="cuda")
        eng.prefill(0, 0, base, util.torch_dev(q), out=out)
        eng.sync()
        o = out.cpu().numpy()
        ref = po.attn_f64(q, K, V, nH, nKV, hd, base, nc)
        assert np.all(np.isfinite(o[:, :nH * hd])), t["name"]
        ma, mr = util.assert_close(o[:, :nH * hd], ref, t["name"])
        assert np.all(np.isnan(o[:, nH * hd:])), "wrote into the padding between columns"   # attn_tile_test.js:80
        print(f"{t['name']}: max-abs {ma:.2e} max-rel {mr:.2e}")


def test_head_dims_outside_64_128_256_are_refused():
    # attnTileConfig takes any multiple of 16 up to 256 (engine/wgsl/attn_tile.js:44); the TMA boxes and the tensor-core
    # tiles here are built from 64-element chunks, so 64, 128 and 256 (every shape pooled's models use) are what exists
    from pooled_b200 import PaError
    for hd in (96, 80, 512):
        with pytest.raises(PaError) as e:
            _engine(8, 2, hd, 2048)
        assert e.value.code == -2


@pytest.mark.parametrize("n_cols,pos,act", [(700, 0, "f16"), (130, 219, "f32")])
def test_head_dim_64_prefill_chunks_and_decode(n_cols, pos, act):
    # head_dim 64 (the reference's "small head" case) beyond the 16-column pass of its unit test: several 128-column
    # CTA tiles, a chunk that starts past row 0, and the decode kernel on the same cache
    import torch
    nH, nKV, hd = 8, 2, 64
    td = torch.float16 if act == "f16" else torch.float32
    eng = _engine(nH, nKV, hd, pos + n_cols + 8, act=act, max_cols=1024, n_rot=64, rope_mode="f64")
    q, k, v, g = _inputs(9, nH, nKV, hd, pos + n_cols)
    d = lambda a: util.torch_dev(a, td)
    if pos:
        eng.encode_layer(0, 0, d(q[:pos]), d(k[:pos]), d(v[:pos]), d(g[:pos]), mode="prefill")
    out = eng.encode_layer(0, pos, d(q[pos:]), d(k[pos:]), d(v[pos:]), d(g[pos:]), mode="prefill").float().cpu().numpy()
    eng.sync()
    ref, Kf, Vf = _oracle_layer(q, k, v, g, nH, nKV, hd, 64, 1e7, 0)
    gk, gv = util.read_cache(eng, 0, 0, 0, pos + n_cols)
    assert np.array_equal(gk, Kf) and np.array_equal(gv, Vf), "KV append is not bit-exact"
    util.assert_close(out, ref[pos:], f"head_dim 64 prefill at {pos}")
    for c in (0, pos, pos + n_cols - 1):
        qr = eng.rope(d(q[c:c + 1]), nH, c)
        one = eng.decode(0, [(0, c, 1)], qr, d(g[c:c + 1])).float().cpu().numpy()
        util.assert_close(one[0], ref[c], f"head_dim 64 decode at {c}")
    eng.sync()


def _inputs(cfg_id, nH, nKV, hd, n_cols):
    q = util.normal_f16(0xA11CE + cfg_id, (n_cols, nH * hd)); k = util.normal_f16(0xB0B + cfg_id, (n_cols, nKV * hd))
    v = util.normal_f16(0xC0DE + cfg_id, (n_cols, nKV * hd)); g = util.normal_f16(0x6A7E + cfg_id, (n_cols, nH * hd))
    return q, k, v, g


def _oracle_layer(q, k, v, g, nH, nKV, hd, n_rot, theta, pos, cols=None):
    n = q.shape[0]
    Kf = np.stack([po.f16_rne(po.rope_neox_f64(k[c], nKV, hd, n_rot, pos + c, theta)) for c in range(n)])
    Vf = po.f16_rne(v)
    cols = range(n) if cols is None else cols
    outs = []
    for c in cols:
        qr = po.rope_neox_f64(q[c], nH, hd, n_rot, pos + c, theta)[None]
        outs.append(po.attn_f64(qr, Kf, Vf, nH, nKV, hd, pos + c, 1, None if g is None else g[c:c + 1])[0])
    return np.stack(outs), Kf, Vf


@pytest.mark.parametrize("n_cols,act,gate", [(1024, "f16", False), (300, "f32", True), (129, "f16", True), (1, "f16", False)])
def test_config3_shape_reduced(n_cols, act, gate):
    # 24 q / 4 kv heads, head_dim 256, partial RoPE 64 dims theta 1e7, prompt into an empty cache: RoPE + append + prefill
    import torch
    nH, nKV, hd = 24, 4, 256
    td = torch.float16 if act == "f16" else torch.float32
    eng = _engine(nH, nKV, hd, n_cols + 8, act=act, max_cols=n_cols, rope_mode="f64")
    q, k, v, g = _inputs(3, nH, nKV, hd, n_cols)
    out = eng.encode_layer(0, 0, util.torch_dev(q, td), util.torch_dev(k, td), util.torch_dev(v, td), util.torch_dev(g, td) if gate else None,
                           mode="prefill").float().cpu().numpy()
    eng.sync()
    ref, Kf, Vf = _oracle_layer(q, k, v, g if gate else None, nH, nKV, hd, 64, 1e7, 0)
    gk, gv = util.read_cache(eng, 0, 0, 0, n_cols)
    assert np.array_equal(gk, Kf) and np.array_equal(gv, Vf), "KV append is not bit-exact"
    ma, mr = util.assert_close(out, ref, f"prefill {n_cols}")
    print(f"prefill {n_cols} {act}: max-abs {ma:.2e} max-rel {mr:.2e}")


@pytest.mark.parametrize("nH,nKV,hd", [(24, 4, 256), (16, 8, 128)])
def test_prefill_gives_the_same_bits_twice(nH, nKV, hd):
    # two threads issue the score products of alternate tiles and two softmax groups take alternate tiles: the order of
    # every sum is fixed all the same, so a repeated pass over the same cache carries the same bits
    import torch
    n_cols = 1500
    eng = _engine(nH, nKV, hd, n_cols + 8, act="f16", max_cols=n_cols, rope_mode="f64")
    q, k, v, g = _inputs(5, nH, nKV, hd, n_cols)
    d = lambda a: util.torch_dev(a, torch.float16)
    dq, dk, dv, dg = d(q), d(k), d(v), d(g)
    outs = [eng.encode_layer(0, 0, dq, dk, dv, dg, mode="prefill").cpu().numpy().view(np.uint16) for _ in range(3)]
    eng.sync()
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


def test_chunked_prefill_and_prefill_vs_decode():
    # a second chunk against the first chunk's rows; every column also equals the decode kernel's answer at its position
    import torch
    nH, nKV, hd, n1, n2 = 16, 2, 256, 200, 333
    eng = _engine(nH, nKV, hd, 1024, act="f32", max_cols=512, rope_mode="f64")
    q, k, v, g = _inputs(7, nH, nKV, hd, n1 + n2)
    d = lambda a: util.torch_dev(a)
    o1 = eng.encode_layer(0, 0, d(q[:n1]), d(k[:n1]), d(v[:n1]), d(g[:n1]), mode="prefill").cpu().numpy()
    o2 = eng.encode_layer(0, n1, d(q[n1:]), d(k[n1:]), d(v[n1:]), d(g[n1:]), mode="prefill").cpu().numpy()
    ref, _, _ = _oracle_layer(q, k, v, g, nH, nKV, hd, 64, 1e7, 0)
    util.assert_close(np.concatenate([o1, o2]), ref, "chunked prefill")
    for c in (0, 1, 199, 200, 333, 532):
        qr = eng.rope(d(q[c:c + 1]), nH, c)
        one = eng.decode(0, [(0, c, 1)], qr, d(g[c:c + 1])).cpu().numpy()
        util.assert_close(one[0], ref[c], f"decode at {c}")
    eng.sync()


def test_config3_full_size_properties():
    # the whole 8192-token prompt (0.82 TFLOP): checked on sampled columns against the oracle (the float64 oracle over
    # all 8192 columns takes minutes) and through size-independent properties
    import torch
    nH, nKV, hd, T = 24, 4, 256, 8192
    eng = _engine(nH, nKV, hd, T, act="f16", max_cols=T, rope_mode="f64")
    q, k, v, g = _inputs(3, nH, nKV, hd, T)
    d = lambda a: util.torch_dev(a, torch.float16)
    out = eng.encode_layer(0, 0, d(q), d(k), d(v), None, mode="prefill").float().cpu().numpy()
    eng.sync()
    assert np.all(np.isfinite(out))
    # the first, the last and one interior column of each of the 64 CTA tiles of 128 columns (every CTA of the
    # 24-head x 64-tile schedule has columns under the oracle), plus the first 64-key tile's edges
    rng = np.random.default_rng(3)
    cols = sorted({0, 1, 63, 64} | {t * 128 + o for t in range(T // 128) for o in (0, 127, int(rng.integers(1, 127)))})
    ref, Kf, Vf = _oracle_layer(q, k, v, None, nH, nKV, hd, 64, 1e7, 0, cols)
    ma, mr = util.assert_close(out[cols], ref, "config 3 sampled columns")
    print(f"config 3 full size: {len(cols)} columns, max-abs {ma:.2e} max-rel {mr:.2e}")
    gk, gv = util.read_cache(eng, 0, 0, 0, T)
    assert np.array_equal(gk, Kf) and np.array_equal(gv, Vf), "KV append is not bit-exact at full size"
    # column 0 attends one key: its output is exactly that V row (per kv head), whatever q is
    v0 = po.h2f(Vf[0]).reshape(nKV, hd)
    assert np.allclose(out[0].reshape(nH, hd), np.repeat(v0, nH // nKV, axis=0), atol=1e-3)
    # every output lies inside the range of the V values it can see (a convex combination)
    vmax = np.maximum.accumulate(po.h2f(Vf).reshape(T, nKV, hd), axis=0)[::512]
    o = out[::512].reshape(-1, nKV, nH // nKV, hd)
    assert np.all(o <= vmax[:, :, None, :] + 2e-3)
