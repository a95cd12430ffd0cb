"""Gather mode of the decode (pa_decode_gather): a column attends a listed set of cache rows, as pooled's QSA kernels do
(attn_dec with gather = stride, engine/wgsl/attn_dec.js:33-38; attnDecMcWGSL({gather}), engine/wgsl/qwen4exp_batch.js:590-641).
The reference pins two things (tests/test_qsa.js:295-324): the list 0 .. seqLen-1 gives the dense kernel's bits, and a
selection gives exact attention over the selected rows."""
import numpy as np
import pytest

from oracle import po
from tests import util

pytestmark = pytest.mark.gpu


def _engine(nH, nKV, hd, max_seq, act="f32", max_cols=8):
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    return AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64 if hd == 256 else hd, rope_theta=1e7, max_seq=max_seq, rope_mode="none",
                                 act_dtype=torch.float32 if act == "f32" else torch.float16, max_cols=max_cols))


def _lists(rows_per_col, stride):
    import torch
    a = np.zeros((len(rows_per_col), stride), dtype=np.int32)
    for c, rows in enumerate(rows_per_col):
        a[c, 0] = len(rows); a[c, 1:1 + len(rows)] = rows
    return torch.from_numpy(a).cuda()


@pytest.mark.parametrize("nH,nKV,hd", [(16, 2, 256), (16, 8, 128)])
def test_full_list_gives_the_dense_kernels_bits(nH, nKV, hd):
    import torch
    max_seq, stride = 4096, 2052
    eng = _engine(nH, nKV, hd, max_seq)
    K = po.np_f16_rne(po.normal(1, max_seq * nKV * hd) * 0.8).reshape(max_seq, nKV * hd); V = po.np_f16_rne(po.normal(2, max_seq * nKV * hd)).reshape(max_seq, nKV * hd)
    util.load_cache(eng, 0, 0, K, V)
    for lens in ([1], [63], [64], [65], [300], [2051], [1, 64, 700, 2051], [500, 500, 500]):
        nc = len(lens)
        q = po.normal(10 + nc, nc * nH * hd).astype(np.float32).reshape(nc, nH * hd); g = po.normal(20 + nc, nc * nH * hd).astype(np.float32).reshape(nc, nH * hd)
        qd, gd = util.torch_dev(q), util.torch_dev(g)
        dense = eng.decode(0, [(0, n - 1, 1) for n in lens], qd, gd)
        got = eng.decode_gather(0, _lists([np.arange(n) for n in lens], stride), qd, gd)
        eng.sync()
        assert torch.equal(dense.view(torch.int32), got.view(torch.int32)), f"lengths {lens}: gather over 0..n-1 differs from the dense decode"
        ref = np.concatenate([po.attn_f64(q[c:c + 1], K, V, nH, nKV, hd, lens[c] - 1, 1, g[c:c + 1]) for c in range(nc)])
        assert util.errs(got.cpu().numpy(), ref)[1] < util.REF_REL


@pytest.mark.parametrize("act", ["f32", "f16"])
def test_selected_blocks_equal_exact_attention_over_the_listed_rows(act):
    import torch
    nH, nKV, hd, max_seq, stride = 16, 2, 256, 20000, 2052
    td = torch.float32 if act == "f32" else torch.float16
    eng = _engine(nH, nKV, hd, max_seq, act=act)
    K = po.np_f16_rne(po.normal(3, max_seq * nKV * hd) * 0.8).reshape(max_seq, nKV * hd); V = po.np_f16_rne(po.normal(4, max_seq * nKV * hd)).reshape(max_seq, nKV * hd)
    util.load_cache(eng, 0, 0, K, V)
    rng = np.random.default_rng(7)
    sels = []
    for c, (n_blocks, tail) in enumerate([(32, 3), (8, 0), (1, 1), (31, 67)]):   # 64-row blocks + the column's newest rows
        blocks = np.sort(rng.choice(max_seq // 64 - 2, size=n_blocks, replace=False))
        rows = np.concatenate([np.arange(b * 64, b * 64 + 64) for b in blocks] + [np.arange(max_seq - 100, max_seq - 100 + tail)])
        sels.append(np.sort(rows).astype(np.int64))
    nc = len(sels)
    q = util.normal_f16(30, (nc, nH * hd)); g = util.normal_f16(31, (nc, nH * hd))
    got = eng.decode_gather(0, _lists(sels, stride), util.torch_dev(q, td), util.torch_dev(g, td)).float().cpu().numpy()
    eng.sync()
    for c, rows in enumerate(sels):
        ref = po.attn_f64(q[c:c + 1], K[rows], V[rows], nH, nKV, hd, len(rows) - 1, 1, g[c:c + 1])
        if act == "f32":
            assert util.errs(got[c:c + 1], ref)[1] < util.REF_REL, f"column {c}"
        else:
            util.assert_close(got[c:c + 1], ref, f"column {c}")


def test_empty_list_and_bad_arguments():
    import torch
    from pooled_b200.lib import PaError
    nH, nKV, hd = 16, 2, 256
    eng = _engine(nH, nKV, hd, 1024)
    eng.cache(0, "k").fill_(0x7e00); eng.cache(0, "v").fill_(0x7e00)       # NaN everywhere: nothing may be read into the result
    K = po.np_f16_rne(po.normal(5, 10 * nKV * hd)).reshape(10, nKV * hd)
    util.load_cache(eng, 0, 0, K, K)
    q = util.torch_dev(po.normal(6, 2 * nH * hd).astype(np.float32).reshape(2, nH * hd))
    out = eng.decode_gather(0, _lists([np.arange(0), np.array([2, 5, 9])], 16), q).cpu().numpy()
    eng.sync()
    assert np.all(out[0] == 0.0)
    ref = po.attn_f64(q.cpu().numpy()[1:2], K[[2, 5, 9]], K[[2, 5, 9]], nH, nKV, hd, 2, 1)
    assert util.errs(out[1:2], ref)[1] < util.REF_REL
    # lists wide enough for the call to merge its own records (no combine kernel behind it): the empty column still
    # reads zero, over whatever the output held before
    wide = torch.full((2, nH * hd), 7.0, dtype=torch.float32, device="cuda")
    eng.decode_gather(0, _lists([np.arange(0), np.array([2, 5, 9])], 2052), q, out=wide)
    eng.sync()
    wide = wide.cpu().numpy()
    assert np.all(wide[0] == 0.0)
    assert np.array_equal(wide[1], out[1])
    with pytest.raises(PaError):
        eng.decode_gather(0, torch.zeros((2, 1), dtype=torch.int32, device="cuda"), q)      # no room for a row
