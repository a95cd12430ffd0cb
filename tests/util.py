"""Shared helpers of the GPU parity tests: seeded inputs, cache loading, tolerances."""
from __future__ import annotations

import numpy as np

from oracle import po

# Tolerance on f16 outputs: max-abs 2e-3 and max-rel 1e-2, the relative error taken as the reference's
# own tests take it: max |diff| / max |ref| (tests/test_attn_dec.js:87-88)
MAX_ABS, MAX_REL = 2e-3, 1e-2
# the reference's own bound for attn_dec with f32 q and f32 outputs (tests/test_attn_dec.js:98)
REF_REL = 2e-5


def errs(got: np.ndarray, ref: np.ndarray):
    d = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    return float(d.max()), float(d.max() / max(np.abs(ref).max(), 1e-30))


def assert_close(got, ref, what=""):
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    ma, mr = errs(got, ref)
    assert ma <= MAX_ABS and mr <= MAX_REL, f"{what}: max-abs {ma:.3e} (<= {MAX_ABS}), max-rel {mr:.3e} (<= {MAX_REL})"
    return ma, mr


def torch_dev(a: np.ndarray, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def load_cache(eng, li: int, seq: int, K: np.ndarray, V: np.ndarray, row0: int = 0):
    """Copy uint16 [rows][kv_dim] arrays into rows row0.. of the layer's caches."""
    import torch
    kc, vc = eng.cache(li, "k"), eng.cache(li, "v")
    kc[seq, row0:row0 + K.shape[0]] = torch.from_numpy(K.view(np.int16)).cuda()
    vc[seq, row0:row0 + V.shape[0]] = torch.from_numpy(V.view(np.int16)).cuda()


def read_cache(eng, li: int, seq: int, row0: int, rows: int):
    k = eng.cache(li, "k")[seq, row0:row0 + rows].cpu().numpy().view(np.uint16)
    v = eng.cache(li, "v")[seq, row0:row0 + rows].cpu().numpy().view(np.uint16)
    return k, v


def normal_f16(seed: int, shape, scale: float = 1.0) -> np.ndarray:
    """N(0, scale^2) rounded to f16, returned as float32 values exactly representable in f16."""
    n = int(np.prod(shape))
    return po.np_h2f(po.np_f16_rne(po.normal(seed, n) * scale)).reshape(shape)


def with_outliers(x: np.ndarray, n_heads: int, hd: int, factor: float = 20.0) -> np.ndarray:
    """x [..., n_heads*hd]: 4 seeded channels per head scaled by `factor` (then re-rounded to f16 values)."""
    y = x.reshape(*x.shape[:-1], n_heads, hd).copy()
    for h in range(n_heads):
        for c in po.outlier_channels(h, hd):
            y[..., h, c] *= factor
    return po.np_h2f(po.np_f16_rne(y)).reshape(x.shape)
