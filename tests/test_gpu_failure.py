"""A bounded device-side wait that runs out: the kernel returns by itself with a status the host reads, the context
latches until pa_reset, and the next step is correct again.  The failure is made on the host side of the protocol: a
two-rank exchange in which the second rank never publishes (its buffer lives on this GPU and nothing writes to it),
with a short polling limit.  Nothing traps, faults or hangs."""
import ctypes as C

import numpy as np
import pytest

from oracle import po
from tests import util

pytestmark = pytest.mark.gpu


def test_exchange_wait_runs_out_then_reset_recovers():
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    from pooled_b200.lib import PaError
    nH, nKV, hd, rows = 16, 2, 256, 3000
    eng = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64, rope_theta=1e7, max_seq=4096, rope_mode="none", act_dtype=torch.float32))
    L = eng.L
    K = po.np_f16_rne(po.normal(1, rows * nKV * hd) * 0.7).reshape(rows, nKV * hd); V = po.np_f16_rne(po.normal(2, rows * nKV * hd)).reshape(rows, nKV * hd)
    util.load_cache(eng, 0, 0, K, V)
    q = po.normal(3, nH * hd).astype(np.float32).reshape(1, -1)
    qd = util.torch_dev(q)
    # world 2, this process is rank 0; "rank 1" is a second buffer on this GPU that no one ever writes
    nbytes = L.pa_exchange_bytes(eng.ctx, 2, 64)
    bufs = (C.c_void_p * 2)()
    for r in range(2):
        p = C.c_void_p()
        eng._ck(L.pa_alloc(eng.ctx, nbytes, C.byref(p)))
        bufs[r] = p.value
    # zero both buffers through torch (plain device memory)
    from pooled_b200.attn import _DevArray
    for r in range(2):
        torch.as_tensor(_DevArray(bufs[r], (nbytes,), "|u1"), device="cuda").zero_()
    torch.cuda.synchronize()
    eng._ck(L.pa_exchange_init(eng.ctx, 0, 2, bufs, 64))
    eng.set_wait_limit(3000)                       # a few milliseconds instead of about a second
    out = eng.decode_exchange(0, [(0, rows - 1, 1)], qd)
    with pytest.raises(PaError) as ei:
        eng.sync()                                 # the kernel came back by itself; the host reads its status
    assert ei.value.code == -5                     # PA_ETIMEOUT
    with pytest.raises(PaError) as ei:
        eng.decode(0, [(0, rows - 1, 1)], qd)      # latched: every call is refused until reset
    assert ei.value.code == -6                     # PA_ESTATE
    eng.reset()
    eng.set_wait_limit(0)
    got = eng.decode(0, [(0, rows - 1, 1)], qd).cpu().numpy()
    eng.sync()
    ref = po.attn_f64(q, K, V, nH, nKV, hd, rows - 1, 1)
    assert util.errs(got, ref)[1] < util.REF_REL
    # the unfinished exchange left its partial answer: finite, and the merge over the one rank that did publish
    assert np.all(np.isfinite(out.cpu().numpy()))
    for r in range(2):
        L.pa_free(eng.ctx, C.c_void_p(bufs[r]))
