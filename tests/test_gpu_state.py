"""KV state to and from the host, GPU-side slots, and a k-token block that straddles a shard boundary, through the C ABI.

What pooled's engine does with exportState / importState / saveSlot / loadSlot (engine/qwen35.js:129-228) for its
full-attention layers: rows [0, pos) x kv_dim f16 per layer, K then V."""
import ctypes as C

import numpy as np
import pytest

from oracle import po
from tests import util

pytestmark = pytest.mark.gpu


def _engine(nH, nKV, hd, max_seq, n_layers=1, n_seqs=1, act="f16", max_cols=8, **kw):
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    return AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64, rope_theta=1e7, max_seq=max_seq, n_layers=n_layers, n_seqs=n_seqs,
                                 act_dtype=torch.float16 if act == "f16" else torch.float32, max_cols=max_cols, **kw))


def _fill(eng, n_layers, pos, nKV, hd, seed=0):
    Ks, Vs = [], []
    for li in range(n_layers):
        K = po.np_f16_rne(po.normal(seed + 10 + li, pos * nKV * hd) * 0.8).reshape(pos, nKV * hd)
        V = po.np_f16_rne(po.normal(seed + 50 + li, pos * nKV * hd)).reshape(pos, nKV * hd)
        util.load_cache(eng, li, 0, K, V)
        Ks.append(K); Vs.append(V)
    return Ks, Vs


def test_export_import_round_trip_gives_identical_decode_bits():
    import torch
    nH, nKV, hd, pos, n_layers = 16, 2, 256, 1500, 3
    a = _engine(nH, nKV, hd, 2048, n_layers=n_layers)
    Ks, Vs = _fill(a, n_layers, pos, nKV, hd)
    st = a.export_state(pos)
    # the parts are the reference's: per layer K rows [0, pos) then V rows [0, pos), kv_dim * 2 bytes each
    assert len(st["parts"]) == 2 * n_layers and all(len(p) == pos * nKV * hd * 2 for p in st["parts"])
    assert st["parts"][2] == Ks[1].tobytes() and st["parts"][3] == Vs[1].tobytes()
    assert st["held"] == [pos] * (2 * n_layers)
    b = _engine(nH, nKV, hd, 2048, n_layers=n_layers)
    for li in range(n_layers):   # whatever the new engine's caches hold is replaced
        b.cache(li, "k").fill_(0x7e00); b.cache(li, "v").fill_(0x7e00)
    assert b.import_state(st) == pos
    q = util.torch_dev(util.normal_f16(1, (1, nH * hd)), torch.float16); k = util.torch_dev(util.normal_f16(2, (1, nKV * hd)), torch.float16)
    v = util.torch_dev(util.normal_f16(3, (1, nKV * hd)), torch.float16); g = util.torch_dev(util.normal_f16(4, (1, nH * hd)), torch.float16)
    for li in range(n_layers):
        oa = a.encode_layer(li, pos, q, k, v, g, mode="decode")
        ob = b.encode_layer(li, pos, q, k, v, g, mode="decode")
        a.sync(); b.sync()
        assert torch.equal(oa.view(torch.int16), ob.view(torch.int16)), f"layer {li}: decode after import differs"
    # a state of another shape is refused, as importState refuses it
    c = _engine(nH, 4, hd, 2048, n_layers=n_layers)
    with pytest.raises(Exception, match="different model"):
        c.import_state(st)
    st2 = dict(st, parts=st["parts"][:-1])
    with pytest.raises(Exception, match="wrong shape"):
        b.import_state(st2)


def test_slots_switch_between_sessions_on_the_device():
    import torch
    nH, nKV, hd, n_layers = 16, 2, 256, 2
    eng = _engine(nH, nKV, hd, 1024, n_layers=n_layers)
    K1, V1 = _fill(eng, n_layers, 700, nKV, hd, seed=0)
    eng.save_slot("a", 700)
    K2, V2 = _fill(eng, n_layers, 300, nKV, hd, seed=100)       # another session overwrites the first rows
    eng.save_slot("b", 300)
    assert eng.load_slot("a") == 700
    eng.sync()
    for li in range(n_layers):
        gk, gv = util.read_cache(eng, li, 0, 0, 700)
        assert np.array_equal(gk, K1[li]) and np.array_equal(gv, V1[li])
    ex = eng.export_slot("b")                                     # read back without switching to it
    assert ex["pos"] == 300 and ex["parts"][0] == K2[0].tobytes() and ex["parts"][3] == V2[1].tobytes()
    assert eng.load_slot("b") == 300
    eng.sync()
    gk, _ = util.read_cache(eng, 0, 0, 0, 300)
    assert np.array_equal(gk, K2[0])
    eng.drop_slot("a")
    with pytest.raises(Exception, match="no saved slot"):
        eng.load_slot("a")
    eng.drop_all_slots()


def test_shards_export_disjoint_row_ranges_of_one_image():
    # two shards of one 600-row sequence on this GPU: each exports its own rows into the same host image
    import torch
    nH, nKV, hd, chunk, pos = 16, 2, 256, 400, 600
    K = po.np_f16_rne(po.normal(1, pos * nKV * hd)).reshape(pos, nKV * hd)
    image = torch.zeros(pos * nKV * hd * 2, dtype=torch.uint8).pin_memory()
    held = []
    for r in range(2):
        eng = _engine(nH, nKV, hd, chunk)
        eng.set_origin(0, r * chunk)
        lo, hi = r * chunk, min(pos, (r + 1) * chunk)
        util.load_cache(eng, 0, 0, K[lo:hi], K[lo:hi])
        n = C.c_uint32()
        eng._ck(eng.L.pa_cache_export(eng.layers[0], 0, 0, pos, 0, C.c_void_p(image.data_ptr()), C.byref(n), eng._st()))
        eng.sync()
        held.append(n.value)
    assert held == [400, 200]
    assert bytes(image.numpy()) == K.tobytes()


def test_block_straddling_a_shard_boundary_is_appended_by_both_owners():
    # a 5-token block at positions 398..402 over shards [0, 400) and [400, 800): the first shard appends columns 0-1, the
    # second columns 2-4, and each shard's answer is attention over the rows it holds (merged across ranks by the
    # exchange; with one rank per exchange here, the merge is the identity)
    import torch
    nH, nKV, hd, chunk, pos, nc, n_rot, theta = 16, 2, 256, 400, 398, 5, 64, 1e7
    K = po.np_f16_rne(po.normal(1, pos * nKV * hd) * 0.8).reshape(pos, nKV * hd); V = po.np_f16_rne(po.normal(2, pos * nKV * hd)).reshape(pos, nKV * hd)
    q = util.normal_f16(3, (nc, nH * hd)); kn = util.normal_f16(4, (nc, nKV * hd)); vn = util.normal_f16(5, (nc, nKV * hd))
    k_rows = np.stack([po.f16_rne(po.rope_neox_f64(kn[c], nKV, hd, n_rot, pos + c, theta)) for c in range(nc)]); v_rows = po.f16_rne(vn)
    Kf, Vf = np.concatenate([K, k_rows]), np.concatenate([V, v_rows])
    q_rot = np.stack([po.rope_neox_f64(q[c], nH, hd, n_rot, pos + c, theta) for c in range(nc)])
    d = lambda a: util.torch_dev(a, torch.float16)
    POISON = 0x5a5a
    for r in range(2):
        eng = _engine(nH, nKV, hd, chunk)
        eng.set_origin(0, r * chunk)
        eng.cache(0, "k").fill_(POISON); eng.cache(0, "v").fill_(POISON)
        lo, hi = r * chunk, min(pos, (r + 1) * chunk)
        if hi > lo:
            util.load_cache(eng, 0, 0, K[lo:hi], V[lo:hi])
        eng.exchange_setup(0, 1, max_rows=nc * nH)
        out = eng.encode_layer_sharded(0, pos, d(q), d(kn), d(vn)).float().cpu().numpy()
        eng.sync()
        # this shard's part of the block, bit for bit, and nothing else written
        c_lo, c_hi = (0, 2) if r == 0 else (2, 5)
        gk, gv = util.read_cache(eng, 0, 0, pos + c_lo - r * chunk, c_hi - c_lo)
        assert np.array_equal(gk, k_rows[c_lo:c_hi]) and np.array_equal(gv, v_rows[c_lo:c_hi]), f"shard {r}: its columns of the block"
        nxt = util.read_cache(eng, 0, 0, pos + c_hi - r * chunk, 1)[0] if pos + c_hi - r * chunk < chunk else None
        assert nxt is None or np.all(nxt == POISON)
        # attention over the rows this shard holds: global rows [r * chunk, (r + 1) * chunk) up to each column's own
        for c in range(nc):
            n_vis = min(pos + c + 1, (r + 1) * chunk) - r * chunk
            if n_vis <= 0:
                continue
            ref = po.attn_f64(q_rot[c:c + 1], Kf[r * chunk:r * chunk + n_vis], Vf[r * chunk:r * chunk + n_vis], nH, nKV, hd, n_vis - 1, 1, None)
            util.assert_close(out[c][None], ref, f"shard {r} column {c}")
