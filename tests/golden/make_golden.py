"""Writes tests/golden/attn_golden.npz: small known-answer vectors for the attention path.

The reference (JavaScript + WGSL) cannot run in the build image, so the vectors come from the NumPy restatement in
oracle/po.py (np_* functions, NumPy's own IEEE f16 conversion) and from plain Python integer / float arithmetic for the
reference tests' LCGs.  The C oracle and the CUDA library are then checked against them.
    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import po  # noqa: E402


def ties_up_bits(x: np.float32) -> int:
    """engine/gguf.js:17-37 in Python integers."""
    u = int(np.float32(x).view(np.uint32))
    sign = (u >> 16) & 0x8000
    e, m = (u >> 23) & 0xff, u & 0x7fffff
    if e == 0xff:
        return sign | 0x7c00 | (0x200 if m else 0)
    e = e - 127 + 15
    if e >= 0x1f:
        return sign | 0x7c00
    if e <= 0:
        if e < -10:
            return sign
        m = (m | 0x800000) >> (1 - e)
        return sign | ((m + 0x1000) >> 13)
    return sign | ((e << 10) + ((m + 0x1000) >> 13))


def main():
    rng = np.random.default_rng(20261125)
    f16_in = np.concatenate([
        rng.integers(0, 2**32, size=512, dtype=np.uint64).astype(np.uint32).view(np.float32),
        np.array([0.0, -0.0, 1.0, -1.99999, 65504.0, 65519.99, 65520.0, 1e30, np.inf, -np.inf, 2.0**-24, 2.0**-25, 6.0e-8, 6.1035e-5,
                  1.0 + 2.0**-11, 1.0 + 3 * 2.0**-11], dtype=np.float32)])
    f16_in = f16_in[~np.isnan(f16_in)]
    f16_rne = po.np_f16_rne(f16_in)
    f16_up = np.array([ties_up_bits(x) for x in f16_in], dtype=np.uint16)

    s, lcg_dec = 12345, []
    for _ in range(16):
        s = (s * 1664525 + 1013904223) % 2**32; lcg_dec.append(s)
    s, lcg_tile = 12345, []
    for _ in range(16):
        s = int((float(s) * 1103515245.0 + 12345.0) % 4294967296.0); lcg_tile.append(s)

    nH, nKV, hd, rows, nc, n_rot, theta, pos0 = 4, 2, 128, 70, 3, 64, 1e7, 67
    K = po.np_f16_rne(po.normal(101, rows * nKV * hd) * 0.8).reshape(rows, nKV * hd)
    V = po.np_f16_rne(po.normal(102, rows * nKV * hd)).reshape(rows, nKV * hd)
    q = po.normal(103, nc * nH * hd).astype(np.float32).reshape(nc, nH * hd)
    g = po.normal(104, nc * nH * hd).astype(np.float32).reshape(nc, nH * hd)
    out = po.np_attn_f64(q, K, V, nH, nKV, hd, pos0, nc)
    out_gated = po.np_attn_f64(q, K, V, nH, nKV, hd, pos0, nc, g)
    rope_in = po.normal(105, nH * hd).astype(np.float32)
    rope_out = po.np_rope_neox(rope_in, nH, hd, n_rot, 32768, theta)
    rope_full = po.np_rope_neox(rope_in, nH, hd, hd, 4096, 1e6)

    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz"),
                        f16_in=f16_in, f16_rne=f16_rne, f16_up=f16_up, lcg_dec=np.array(lcg_dec, dtype=np.uint32), lcg_tile=np.array(lcg_tile, dtype=np.uint32),
                        shape=np.array([nH, nKV, hd, rows, nc, n_rot, pos0]), theta=np.array([theta]), K=K, V=V, q=q, g=g, out=out, out_gated=out_gated,
                        rope_in=rope_in, rope_out=rope_out, rope_full=rope_full)

    # the "next" rows of the path: int8 KV (kv_store_q8, NumPy twin) and gathered attention (exact attention over listed rows)
    x = (po.normal(201, 24 * 256) * 2.0).astype(np.float32).reshape(24, 256)
    x[1, :32] = 0.0; x[2, 40] = 900.0; x[3, :32] = np.arange(32) - 15.5
    q8, q8_scales = po.np_kv_store_q8(x)
    listed = np.array([0, 3, 4, 17, 40, 41, 69], dtype=np.int32)
    out_listed = po.np_attn_f64(q[:1], K[listed], V[listed], nH, nKV, hd, len(listed) - 1, 1)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "kvfmt_golden.npz"),
                        x=x, q8=q8, q8_scales=q8_scales, listed=listed, out_listed=out_listed)


if __name__ == "__main__":
    main()
