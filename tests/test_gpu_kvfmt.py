"""int8 (kvQ8) and f32 KV caches: the append of kv_store_q8 bit for bit, and attention over those caches against exact
attention over the values the cache holds (engine/wgsl/qwen35.js:97-139, :908-946; engine/wgsl/dense.js:22-136)."""
import numpy as np
import pytest

from oracle import po
from tests import util

pytestmark = pytest.mark.gpu


def _engine(fmt, nH, nKV, hd, max_seq, act="f32", max_cols=8, rope_mode="none", n_layers=1, n_seqs=1):
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    return AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64, rope_theta=1e7, max_seq=max_seq, rope_mode=rope_mode, n_layers=n_layers,
                                 n_seqs=n_seqs, act_dtype=torch.float32 if act == "f32" else torch.float16, max_cols=max_cols, kv_format=fmt))


def _held(eng, fmt, li, rows):
    """The K and V values the cache holds, as float32 [rows][kv_dim]."""
    k, v = eng.cache(li, "k")[0, :rows].cpu().numpy(), eng.cache(li, "v")[0, :rows].cpu().numpy()
    if fmt == "q8":
        ks, vs = eng.cache_scales(li, "k")[0, :rows].cpu().numpy(), eng.cache_scales(li, "v")[0, :rows].cpu().numpy()
        return po.dequant_q8(k, ks), po.dequant_q8(v, vs), (k, ks, v, vs)
    return k, v, None


def test_q8_append_is_kv_store_q8_bit_for_bit():
    import torch
    nH, nKV, hd, n = 16, 2, 256, 40
    eng = _engine("q8", nH, nKV, hd, 64, max_cols=64)
    x = (po.normal(1, 2 * n * nKV * hd) * 2.5).astype(np.float32).reshape(2, n, nKV * hd)
    x[0, 3, :32] = 0.0                       # an all-zero block: scale 0, values 0
    x[0, 4, 32:64] = 1e-30                   # a block whose scale underflows towards zero
    x[1, 5, 7] = 1000.0                      # one outlier sets the block's scale
    x[0, 6, :32] = np.arange(32) - 15.5      # ties: x * inv lands on .5 values for some entries
    eng.kv_append(0, 0, 10, torch.from_numpy(x[0]).cuda(), torch.from_numpy(x[1]).cuda())
    eng.sync()
    _, _, (k, ks, v, vs) = _held(eng, "q8", 0, 64)
    wk, wks = po.kv_store_q8(x[0]); wv, wvs = po.kv_store_q8(x[1])
    assert np.array_equal(k[10:10 + n], wk) and np.array_equal(v[10:10 + n], wv), "int8 values differ from kv_store_q8"
    assert np.array_equal(ks[10:10 + n].view(np.uint32), wks.view(np.uint32)) and np.array_equal(vs[10:10 + n].view(np.uint32), wvs.view(np.uint32))
    nk, nks = po.np_kv_store_q8(x[0])        # the NumPy twin agrees with the C restatement
    assert np.array_equal(nk, wk) and np.array_equal(nks.view(np.uint32), wks.view(np.uint32))


@pytest.mark.parametrize("fmt", ["q8", "f32"])
@pytest.mark.parametrize("nH,nKV,hd", [(16, 2, 256), (16, 8, 128), (8, 2, 64)])
def test_decode_over_the_cache_equals_exact_attention_over_what_it_holds(fmt, nH, nKV, hd):
    import torch
    rows = 3001
    eng = _engine(fmt, nH, nKV, hd, 3100, max_cols=8)
    K = (po.normal(2, rows * nKV * hd) * 0.8).astype(np.float32).reshape(rows, nKV * hd); V = po.normal(3, rows * nKV * hd).astype(np.float32).reshape(rows, nKV * hd)
    for r0 in range(0, rows, 8):             # appended eight rows at a time
        eng.kv_append(0, 0, r0, torch.from_numpy(K[r0:r0 + 8]).cuda(), torch.from_numpy(V[r0:r0 + 8]).cuda())
    eng.sync()
    Kh, Vh, _ = _held(eng, fmt, 0, rows)
    if fmt == "f32":
        assert np.array_equal(Kh, K) and np.array_equal(Vh, V)
    for seq_len, nc in ((1, 1), (64, 1), (65, 1), (rows, 1), (rows, 5), (700, 3)):
        pos = seq_len - nc
        q = po.normal(10 + seq_len, nc * nH * hd).astype(np.float32).reshape(nc, nH * hd); g = po.normal(20 + seq_len, nc * nH * hd).astype(np.float32).reshape(nc, nH * hd)
        out = eng.decode(0, [(0, pos, nc)], util.torch_dev(q), util.torch_dev(g)).cpu().numpy()
        eng.sync()
        ref = po.attn_f64_kv32(q, Kh, Vh, nH, nKV, hd, pos, nc, g)
        assert np.all(np.isfinite(out)) and util.errs(out, ref)[1] < util.REF_REL, f"{fmt} seq_len {seq_len} x {nc}"


@pytest.mark.parametrize("fmt", ["q8", "f32"])
def test_layer_call_and_prefill_on_other_formats(fmt):
    # RoPE + append + attend + gate in one call: k is rotated (float64 expression, f32 result) and then stored in the
    # layer's format; a 300-column prefill chunk, then one token, then a 5-token block
    import torch
    nH, nKV, hd, n_rot, theta = 16, 2, 256, 64, 1e7
    eng = _engine(fmt, nH, nKV, hd, 512, act="f16", max_cols=320, rope_mode="f64")
    T = 306
    q = util.normal_f16(1, (T, nH * hd)); k = util.normal_f16(2, (T, nKV * hd)); v = util.normal_f16(3, (T, nKV * hd)); g = util.normal_f16(4, (T, nH * hd))
    d = lambda a: util.torch_dev(a, torch.float16)
    outs = [eng.encode_layer(0, 0, d(q[:300]), d(k[:300]), d(v[:300]), d(g[:300]), mode="prefill"),
            eng.encode_layer(0, 300, d(q[300:301]), d(k[300:301]), d(v[300:301]), d(g[300:301]), mode="decode"),
            eng.encode_layer(0, 301, d(q[301:]), d(k[301:]), d(v[301:]), d(g[301:]), mode="decode")]
    eng.sync()
    out = torch.cat(outs).float().cpu().numpy()
    k_rot = np.stack([po.rope_neox_f64(k[c], nKV, hd, n_rot, c, theta) for c in range(T)])
    Kh, Vh, held = _held(eng, fmt, 0, T)
    if fmt == "q8":
        wk, wks = po.kv_store_q8(k_rot); wv, wvs = po.kv_store_q8(v)
        assert np.array_equal(held[0], wk) and np.array_equal(held[2], wv) and np.array_equal(held[1].view(np.uint32), wks.view(np.uint32))
    else:
        assert np.array_equal(Kh.view(np.uint32), k_rot.view(np.uint32)) and np.array_equal(Vh, v)
    q_rot = np.stack([po.rope_neox_f64(q[c], nH, hd, n_rot, c, theta) for c in range(T)])
    ref = np.concatenate([po.attn_f64_kv32(q_rot[c:c + 1], Kh, Vh, nH, nKV, hd, c, 1, g[c:c + 1]) for c in range(T)])
    util.assert_close(out, ref, f"{fmt} layer calls")


def test_q8_state_round_trip_and_refusals():
    import torch
    from pooled_b200.lib import PaError
    nH, nKV, hd, pos = 16, 2, 256, 200
    a = _engine("q8", nH, nKV, hd, 256, max_cols=8)
    K = po.normal(5, pos * nKV * hd).astype(np.float32).reshape(pos, nKV * hd)
    for r0 in range(0, pos, 8):
        a.kv_append(0, 0, r0, torch.from_numpy(K[r0:r0 + 8]).cuda(), torch.from_numpy(K[r0:r0 + 8] * 0.5).cuda())
    st = a.export_state(pos)
    assert [len(p) for p in st["parts"]] == [pos * 512, pos * 512, pos * 16 * 4, pos * 16 * 4]      # K, V, K scales, V scales (kvQ8 _stateParts)
    b = _engine("q8", nH, nKV, hd, 256, max_cols=8)
    b.import_state(st)
    q = util.torch_dev(po.normal(6, nH * hd).astype(np.float32).reshape(1, -1))
    oa, ob = a.decode(0, [(0, pos - 1, 1)], q), b.decode(0, [(0, pos - 1, 1)], q)
    a.sync(); b.sync()
    assert torch.equal(oa.view(torch.int32), ob.view(torch.int32))
    with pytest.raises(PaError, match="different model"):
        _engine("f32", nH, nKV, hd, 256).import_state(st)
    with pytest.raises(PaError) as e:
        a.save_slot("x", pos)
    assert e.value.code == -2
    with pytest.raises(PaError) as e:
        a.decode_partial(0, [(0, pos - 1, 1)], q)
    assert e.value.code == -2
