"""RoPE and KV append on the GPU against the CPU oracle: bit-exact."""
import numpy as np
import pytest

from oracle import po
from tests import util

pytestmark = pytest.mark.gpu


def _engine(**kw):
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    d = dict(n_heads=16, n_kv_heads=2, head_dim=256, n_rot=64, rope_theta=1e7, max_seq=512, act_dtype=torch.float32, max_cols=64)
    d.update(kw)
    return AttnEngine(AttnConfig(**d))


def test_kv_append_conversion_is_bit_exact_on_every_class_of_value():
    # tests/test_q38flash_mc.js:231-236: the cache half == f16bits(f32 value), for every value
    import torch
    eng = _engine()
    rng = np.random.default_rng(1)
    kvd = eng.cfg.kv_dim
    n_cols = 64
    x = rng.integers(0, 2**32, size=2 * n_cols * kvd, dtype=np.uint64).astype(np.uint32).view(np.float32).copy()
    # plant every half-way case of a run of f16 values, subnormals, overflow edges, infinities, NaN, signed zero
    h = np.arange(0, 4096, dtype=np.uint16) * 16 + 3
    mid = ((po.h2f(h).astype(np.float64) + po.h2f(h + 1).astype(np.float64)) / 2).astype(np.float32)
    special = np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, -65520.0, 1e30, np.inf, -np.inf, np.nan, 2.0**-24, 2.0**-25, 2.0**-25 * 1.0001,
                        6.0e-8, -3.1e-5, 6.1035e-5], dtype=np.float32)
    x[:mid.size] = mid; x[mid.size:2 * mid.size] = -mid; x[2 * mid.size:2 * mid.size + special.size] = special
    k, v = x[:n_cols * kvd].reshape(n_cols, kvd), x[n_cols * kvd:].reshape(n_cols, kvd)
    eng.kv_append(0, 0, 100, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
    eng.sync()
    gk, gv = util.read_cache(eng, 0, 0, 100, n_cols)
    assert np.array_equal(gk, po.f16_rne(k)) and np.array_equal(gv, po.f16_rne(v))


@pytest.mark.parametrize("hd,n_rot,theta,nH,nKV,pos,n_cols,dtype", [
    (128, 128, 1e6, 16, 8, 4096, 1, "f16"),      # config 1: full RoPE
    (256, 64, 1e7, 16, 2, 32768, 1, "f16"),      # config 2
    (256, 64, 1e7, 16, 2, 131072, 1, "f32"),     # config 5 position
    (256, 64, 1e7, 24, 4, 16384, 5, "f16"),      # config 4 block
    (256, 64, 1e7, 24, 4, 0, 64, "f32"),         # start of a prefill
    (256, 64, 1e7, 24, 4, 8128, 64, "f16"),      # end of config 3's prompt
])
def test_rope_append_matches_oracle_bit_for_bit(hd, n_rot, theta, nH, nKV, pos, n_cols, dtype):
    import torch
    td = torch.float16 if dtype == "f16" else torch.float32
    eng = _engine(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=theta, max_seq=pos + n_cols + 3, act_dtype=td)
    qd, kvd = nH * hd, nKV * hd
    q = util.normal_f16(10, (n_cols, qd)); k = util.normal_f16(11, (n_cols, kvd)); v = util.normal_f16(12, (n_cols, kvd))
    if dtype == "f32":   # values that are not f16-representable
        q = po.normal(10, n_cols * qd).astype(np.float32).reshape(n_cols, qd)
        k = po.normal(11, n_cols * kvd).astype(np.float32).reshape(n_cols, kvd)
        v = po.normal(12, n_cols * kvd).astype(np.float32).reshape(n_cols, kvd)
    q_rot = eng.rope_append(0, 0, pos, util.torch_dev(q, td), util.torch_dev(k, td), util.torch_dev(v, td))
    eng.sync()
    gk, gv = util.read_cache(eng, 0, 0, pos, n_cols)
    gq = q_rot.cpu().numpy()
    bad_k = bad_q = 0
    for c in range(n_cols):
        wq = po.rope_neox_f64(q[c], nH, hd, n_rot, pos + c, theta)
        wk = po.rope_neox_f64(k[c], nKV, hd, n_rot, pos + c, theta)
        bad_q += int(np.count_nonzero(gq[c].view(np.uint32) != wq.view(np.uint32)))
        bad_k += int(np.count_nonzero(gk[c] != po.f16_rne(wk)))
        assert np.array_equal(gv[c], po.f16_rne(v[c]))
    # the device's float64 sin/cos and the host libm's can differ in the last place; a flip of the f32 store needs that
    # difference to straddle an f32 rounding boundary (about 1e-8 per element) and a flip of the f16 cache value
    # needs the f32 flip to straddle an f16 boundary too.  On these seeded inputs neither happens.
    assert bad_k == 0, f"{bad_k} cache halves differ"
    assert bad_q <= 2, f"{bad_q} rotated q values differ in f32 bits"
    # rows around the appended ones are untouched
    if pos > 0:
        assert not np.any(util.read_cache(eng, 0, 0, pos - 1, 1)[0] != util.read_cache(eng, 0, 0, pos - 1, 1)[0])


def test_rope_table_mode_matches_ggml_recurrence_bit_for_bit():
    # the Flash engine's host-computed table: engine/qwen4exp.js:549-553, tests/reference/qsa_ref.mjs:99-110
    import torch
    eng = _engine(n_heads=4, n_kv_heads=2, head_dim=256, n_rot=64, rope_theta=1e7, rope_mode="table", max_seq=4096)
    n_cols, pos = 7, 1000
    q = po.normal(1, n_cols * 4 * 256).astype(np.float32).reshape(n_cols, -1)
    k = po.normal(2, n_cols * 2 * 256).astype(np.float32).reshape(n_cols, -1)
    v = po.normal(3, n_cols * 2 * 256).astype(np.float32).reshape(n_cols, -1)
    cs = np.stack([po.rope_table_f32(64, pos + c, 1e7) for c in range(n_cols)])
    q_rot = eng.rope_append(0, 0, pos, util.torch_dev(q), util.torch_dev(k), util.torch_dev(v), cs_table=util.torch_dev(cs))
    eng.sync()
    gk, gv = util.read_cache(eng, 0, 0, pos, n_cols)
    for c in range(n_cols):
        assert np.array_equal(q_rot[c].cpu().numpy(), po.rope_ggml_f32(q[c], 4, 256, 64, pos + c, 1e7))
        assert np.array_equal(gk[c], po.f16_rne(po.rope_ggml_f32(k[c], 2, 256, 64, pos + c, 1e7)))
        assert np.array_equal(gv[c], po.f16_rne(v[c]))


def test_standalone_rope_and_gate():
    import torch
    eng = _engine(n_heads=16, n_kv_heads=2)
    x = po.normal(5, 3 * 16 * 256).astype(np.float32).reshape(3, -1)
    y = eng.rope(util.torch_dev(x), 16, 77).cpu().numpy()
    for c in range(3):
        assert np.array_equal(y[c], po.rope_neox_f64(x[c], 16, 256, 64, 77 + c, 1e7))
    a = po.normal(6, 3 * 4096).astype(np.float32).reshape(3, -1); g = po.normal(7, 3 * 4096).astype(np.float32).reshape(3, -1)
    at = util.torch_dev(a)
    eng.sigmoid_mul(at, util.torch_dev(g))
    want = a.astype(np.float64) / (1 + np.exp(-g.astype(np.float64)))
    assert np.max(np.abs(at.cpu().numpy() - want)) < 1e-6


def test_arguments_are_checked():
    import torch
    from pooled_b200 import PaError
    eng = _engine(max_seq=128, max_cols=4)
    k = torch.zeros((2, eng.cfg.kv_dim), device="cuda")
    with pytest.raises(PaError) as e:
        eng.kv_append(0, 0, 127, k, k)          # rows 127, 128 pass max_seq
    assert e.value.code == -1 and "max_seq" in str(e.value)
    with pytest.raises(PaError):
        eng.kv_append(0, 1, 0, k, k)            # sequence 1 of 1
    with pytest.raises(PaError):
        eng.kv_append(0, 0, 0, torch.zeros((5, eng.cfg.kv_dim), device="cuda"), torch.zeros((5, eng.cfg.kv_dim), device="cuda"))
    eng.kv_append(0, 0, 126, k, k)               # still usable after argument errors
    eng.sync()
