"""pa_decode_static — the decode entry point for callers that may not allocate device memory (stream-capture regions,
allocator-free threads, hosts that own the memory pool and hand over raw pointers).  It keeps its split partials in a
fixed array inside the library instead of a context's buffers, so this test calls it through the C ABI with nothing but
pointers and checks it against the ordinary pa_decode on the same inputs — twice in a row with different positions and
queries, because the array is shared between calls and keeps the previous call's records.

Collected last on purpose: a failure here must not hide any other test in a run that stops at the first failure."""
import ctypes as C

import numpy as np
import pytest

from oracle import po
from tests import util

pytestmark = pytest.mark.gpu


def _call(lib, eng, pos, n_cols, q, gate, nH, nKV, hd, rows, out=None):
    import torch
    if out is None:
        out = torch.full((n_cols, nH * hd), float("nan"), device="cuda")
    msg = C.create_string_buffer(256)
    rc = lib.pa_decode_static(0, lib.pa_cache_ptr(eng.layers[0], 0), lib.pa_cache_ptr(eng.layers[0], 1), rows, nH, nKV, hd, pos, n_cols,
                              C.c_void_p(q.data_ptr()), C.c_void_p(gate.data_ptr()) if gate is not None else None, C.c_void_p(out.data_ptr()),
                              C.c_void_p(torch.cuda.current_stream().cuda_stream), msg, 256)
    return rc, msg.value.decode(), out


@pytest.mark.parametrize("nH,nKV,hd", [(16, 2, 256), (16, 8, 128)])
def test_static_scratch_decode_matches_pa_decode_twice_in_a_row(nH, nKV, hd):
    import torch
    from pooled_b200 import AttnConfig, AttnEngine, load
    lib = load()
    rows = 9000
    eng = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64, rope_theta=1e7, max_seq=rows, rope_mode="none",
                                act_dtype=torch.float32, max_cols=8))
    K = po.np_f16_rne(po.normal(31, rows * nKV * hd) * 0.7).reshape(rows, nKV * hd)
    V = po.np_f16_rne(po.normal(32, rows * nKV * hd)).reshape(rows, nKV * hd)
    util.load_cache(eng, 0, 0, K, V)
    # first call: one token at a long context with a gate; second call: a 3-token block at a short context, no gate.
    # The second call uses fewer records than the first left behind.
    for pos, n_cols, gated, seed in [(8191, 1, True, 41), (300, 3, False, 42)]:
        q = util.torch_dev(po.normal(seed, n_cols * nH * hd).astype(np.float32).reshape(n_cols, nH * hd))
        g = util.torch_dev(po.normal(seed + 100, n_cols * nH * hd).astype(np.float32).reshape(n_cols, nH * hd)) if gated else None
        want = eng.decode(0, [(0, pos, n_cols)], q, g)
        # the one-time set-up of this row-count class (address look-up, kernel attributes, the driver loading the
        # kernel) happens in a call of its own, so that the measured call below is an ordinary one
        rc, msg, _ = _call(lib, eng, pos, n_cols, q, g, nH, nKV, hd, rows)
        torch.cuda.synchronize()
        assert rc == 0, msg
        out_buf = torch.full((n_cols, nH * hd), float("nan"), device="cuda")     # allocated before the measurement
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc, msg, got = _call(lib, eng, pos, n_cols, q, g, nH, nKV, hd, rows, out=out_buf)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory: something was allocated"
        word = C.c_uint32(123)
        assert lib.pa_decode_static_status(0, C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(word)) == 0 and word.value == 0
        a, b = got.cpu().numpy(), want.cpu().numpy()
        assert np.all(np.isfinite(a))
        assert util.errs(a, b)[1] < util.REF_REL, f"pos {pos}: differs from pa_decode"
        ref = po.attn_f64(q.cpu().numpy(), K, V, nH, nKV, hd, pos, n_cols, None if g is None else g.cpu().numpy())
        assert util.errs(a, ref)[1] < util.REF_REL


def test_static_scratch_decode_refuses_what_does_not_fit():
    import torch
    from pooled_b200 import AttnConfig, AttnEngine, load
    lib = load()
    eng = AttnEngine(AttnConfig(n_heads=16, n_kv_heads=2, head_dim=256, n_rot=64, rope_theta=1e7, max_seq=512, rope_mode="none", act_dtype=torch.float32))
    q = torch.zeros((16, 4096), device="cuda")
    rc, msg, _ = _call(lib, eng, 100, 9, q, None, 16, 2, 256, 512)          # 9 columns x 8 heads per kv head > 64 query rows
    assert rc == -2 and "64" in msg
    rc, msg, _ = _call(lib, eng, 510, 4, q, None, 16, 2, 256, 512)          # positions pass the cache
    assert rc == -1 and "cache_rows" in msg
    rc, msg, _ = _call(lib, eng, 100, 1, q, None, 16, 2, 96, 512)
    assert rc == -2 and "head_dim" in msg
