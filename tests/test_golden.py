"""The committed known-answer vectors (tests/golden/attn_golden.npz) against the C oracle, and on a GPU against the library."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import po
from tests import util

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_golden.npz"))
G2 = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kvfmt_golden.npz"))


def test_oracle_q8_and_listed_rows_vectors():
    q, sc = po.kv_store_q8(G2["x"])
    assert np.array_equal(q, G2["q8"]) and np.array_equal(sc.view(np.uint32), G2["q8_scales"].view(np.uint32))
    nH, nKV, hd = (int(x) for x in G["shape"][:3])
    rows = G2["listed"]
    got = po.attn_f64(G["q"][:1], G["K"][rows], G["V"][rows], nH, nKV, hd, len(rows) - 1, 1)
    assert np.max(np.abs(got - G2["out_listed"])) < 1e-12


def test_oracle_f16_and_lcg_vectors():
    L = po.lib()
    assert np.array_equal(po.f16_rne(G["f16_in"]), G["f16_rne"])
    assert np.array_equal(np.array([L.po_f16_ties_up(float(x)) for x in G["f16_in"]], dtype=np.uint16), G["f16_up"])
    s = C.c_uint32(12345)
    assert [L.po_lcg_dec_next(C.byref(s)) for _ in range(16)] == list(G["lcg_dec"])
    s = C.c_uint32(12345)
    assert [L.po_lcg_tile_next(C.byref(s)) for _ in range(16)] == list(G["lcg_tile"])


def test_oracle_attention_and_rope_vectors():
    nH, nKV, hd, rows, nc, n_rot, pos0 = (int(x) for x in G["shape"])
    theta = float(G["theta"][0])
    assert np.max(np.abs(po.attn_f64(G["q"], G["K"], G["V"], nH, nKV, hd, pos0, nc) - G["out"])) < 1e-12
    assert np.max(np.abs(po.attn_f64(G["q"], G["K"], G["V"], nH, nKV, hd, pos0, nc, G["g"]) - G["out_gated"])) < 1e-12
    assert np.max(np.abs(po.attn_f32ref(G["q"], G["K"], G["V"], nH, nKV, hd, pos0, nc, G["g"]) - G["out_gated"])) < 1e-5
    assert np.max(np.abs(po.rope_neox_f64(G["rope_in"], nH, hd, n_rot, 32768, theta).astype(np.float64) - G["rope_out"])) <= 2.4e-7
    assert np.max(np.abs(po.rope_neox_f64(G["rope_in"], nH, hd, hd, 4096, 1e6).astype(np.float64) - G["rope_full"])) <= 2.4e-7


@pytest.mark.gpu
def test_library_reproduces_the_vectors():
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    nH, nKV, hd, rows, nc, n_rot, pos0 = (int(x) for x in G["shape"])
    eng = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=float(G["theta"][0]), max_seq=128,
                                rope_mode="none", act_dtype=torch.float32, max_cols=8))
    util.load_cache(eng, 0, 0, G["K"], G["V"])
    q, g = util.torch_dev(G["q"]), util.torch_dev(G["g"])
    dec = eng.decode(0, [(0, pos0, nc)], q, g).cpu().numpy()
    assert util.errs(dec, G["out_gated"])[1] < util.REF_REL
    pre = eng.prefill(0, 0, pos0, q).cpu().numpy()
    util.assert_close(pre, G["out"], "prefill vs golden")
    # conversion vectors through the append kernel
    x = np.zeros((1, nKV * hd), dtype=np.float32); n = min(x.size, G["f16_in"].size); x[0, :n] = G["f16_in"][:n]
    eng.kv_append(0, 0, 100, util.torch_dev(x), util.torch_dev(x))
    eng.sync()
    assert np.array_equal(util.read_cache(eng, 0, 0, 100, 1)[0][0, :n], G["f16_rne"][:n])


@pytest.mark.gpu
def test_library_reproduces_the_q8_and_listed_rows_vectors():
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    nH, nKV, hd, rows, nc, n_rot, pos0 = (int(x) for x in G["shape"])
    e8 = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=1e7, max_seq=64, rope_mode="none", act_dtype=torch.float32,
                               max_cols=32, kv_format="q8"))
    x = util.torch_dev(G2["x"])
    e8.kv_append(0, 0, 5, x, x)
    e8.sync()
    assert np.array_equal(e8.cache(0, "k")[0, 5:29].cpu().numpy(), G2["q8"])
    assert np.array_equal(e8.cache_scales(0, "v")[0, 5:29].cpu().numpy().view(np.uint32), G2["q8_scales"].view(np.uint32))
    eng = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=1e7, max_seq=128, rope_mode="none", act_dtype=torch.float32, max_cols=8))
    util.load_cache(eng, 0, 0, G["K"], G["V"])
    lists = np.zeros((1, 16), dtype=np.int32); lists[0, 0] = len(G2["listed"]); lists[0, 1:1 + len(G2["listed"])] = G2["listed"]
    got = eng.decode_gather(0, torch.from_numpy(lists).cuda(), util.torch_dev(G["q"][:1])).cpu().numpy()
    assert util.errs(got, G2["out_listed"])[1] < util.REF_REL
