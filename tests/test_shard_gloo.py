"""Host logic of the KV-sequence-sharded decode (pooled_b200/shard.py) with world size 2 on CPU (gloo): which rank appends,
what each rank's partial covers, the all-gather layout and the merge.  The engine is a stand-in that computes the
(o, m, l) records with NumPy where the real one launches CUDA kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import po
from pooled_b200.shard import ShardPlan, ShardedDecoder

NH, NKV, HD, CHUNK = 4, 2, 64, 96


class _Cfg:
    n_heads, n_kv_heads, head_dim, n_layers, q_dim, max_seq = NH, NKV, HD, 1, NH * HD, CHUNK


class FakeEngine:
    """AttnEngine's sharding-relevant surface over NumPy: caches of CHUNK rows starting at a global origin."""

    def __init__(self):
        self.cfg, self.origin = _Cfg(), 0
        self.K = np.zeros((CHUNK, NKV * HD), dtype=np.uint16); self.V = np.zeros_like(self.K)

    def set_origin(self, li, origin):
        self.origin = origin

    def rope(self, x, n_heads, pos):
        return torch.from_numpy(np.stack([po.rope_neox_f64(x[c].numpy(), n_heads, HD, 32, pos + c, 1e4) for c in range(x.shape[0])]))

    def rope_append(self, li, seq, pos, q, k, v):
        row = pos - self.origin
        assert 0 <= row < CHUNK, "append outside this shard"
        self.K[row] = po.f16_rne(po.rope_neox_f64(k[0].numpy(), NKV, HD, 32, pos, 1e4)); self.V[row] = po.f16_rne(v[0].numpy())
        return self.rope(q, NH, pos)

    def decode_partial(self, li, items, q_rot):
        rows = len(items) * NH
        o = np.zeros((rows, HD), dtype=np.float32); ml = np.zeros((rows, 2), dtype=np.float32)
        Kf, Vf = po.h2f(self.K).astype(np.float64), po.h2f(self.V).astype(np.float64)
        for i, (seq, pos, nc) in enumerate(items):
            n = int(np.clip(pos + 1 - self.origin, 0, CHUNK))
            for h in range(NH):
                g = h // (NH // NKV)
                if n == 0:
                    ml[i * NH + h] = (-3.0e38, 0.0); continue
                s = Kf[:n, g * HD:(g + 1) * HD] @ q_rot[i, h * HD:(h + 1) * HD].numpy().astype(np.float64) / np.sqrt(HD)
                m = s.max(); p = np.exp(s - m)
                o[i * NH + h] = p @ Vf[:n, g * HD:(g + 1) * HD]; ml[i * NH + h] = (m, p.sum())
        return torch.from_numpy(np.concatenate([o.reshape(-1), ml.reshape(-1)]))

    def merge(self, parts, n_cols, gate=None, out=None):
        P, rows = parts.shape[0], n_cols * NH
        a = parts.numpy().astype(np.float64)
        o = a[:, :rows * HD].reshape(P, rows, HD); ml = a[:, rows * HD:].reshape(P, rows, 2)
        M = ml[:, :, 0].max(axis=0); w = np.exp(ml[:, :, 0] - M)
        res = (o * w[:, :, None]).sum(axis=0) / (ml[:, :, 1] * w).sum(axis=0)[:, None]
        res = res.reshape(n_cols, NH * HD)
        if gate is not None:
            res = res / (1 + np.exp(-gate.numpy().astype(np.float64)))
        return torch.from_numpy(res)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        total = 150                                   # context before the step: rank 0 holds 96 rows, rank 1 holds 54
        K = po.np_f16_rne(po.normal(1, total * NKV * HD) * 0.7).reshape(total, NKV * HD)
        V = po.np_f16_rne(po.normal(2, total * NKV * HD)).reshape(total, NKV * HD)
        eng = FakeEngine()
        sd = ShardedDecoder(eng, ShardPlan(world, CHUNK), rank, dist)
        assert eng.origin == rank * CHUNK
        lo, hi = rank * CHUNK, min(total, (rank + 1) * CHUNK)
        eng.K[:hi - lo], eng.V[:hi - lo] = K[lo:hi], V[lo:hi]
        f = lambda s, n: torch.from_numpy(po.normal(s, n).astype(np.float32)).reshape(1, n)
        q, k, v, g = f(3, NH * HD), f(4, NKV * HD), f(5, NKV * HD), f(6, NH * HD)
        out = sd.step(0, [(0, total)], q, k, v, g).numpy()
        # reference: unsharded attention over the 150 rows + the appended one
        Kf = np.concatenate([K, po.f16_rne(po.rope_neox_f64(k[0].numpy(), NKV, HD, 32, total, 1e4))[None]])
        Vf = np.concatenate([V, po.f16_rne(v[0].numpy())[None]])
        ref = po.attn_f64(po.rope_neox_f64(q[0].numpy(), NH, HD, 32, total, 1e4)[None], Kf, Vf, NH, NKV, HD, total, 1, g.numpy())
        err = float(np.abs(out - ref).max())
        appended = bool(np.any(eng.K[total - lo] != 0)) if lo <= total < lo + CHUNK else False
        ret[rank] = (err, appended)
    finally:
        dist.destroy_process_group()


def test_shard_plan():
    p = ShardPlan(4, 100)
    assert [p.owner(x) for x in (0, 99, 100, 399)] == [0, 0, 1, 3]
    with pytest.raises(ValueError):
        p.owner(400)
    assert [p.local_rows(r, 250) for r in range(4)] == [100, 100, 50, 0] and p.local_pos(2, 250) == 50


def test_block_columns_cover_a_straddling_block_once():
    p = ShardPlan(4, 100)
    assert p.block_columns(0, 97, 5) == (0, 3) and p.block_columns(1, 97, 5) == (3, 5)       # rows 97..99 | 100..101
    assert p.block_columns(2, 97, 5)[0] >= p.block_columns(2, 97, 5)[1]                      # nothing for rank 2
    assert p.block_columns(1, 100, 5) == (0, 5) and p.block_columns(0, 100, 5)[1] == 0
    for pos in (0, 95, 99, 100, 196, 299, 395):
        for n in (1, 4, 5, 8):
            if pos + n > 400:
                continue
            got = sorted(c for r in range(4) for c in range(*p.block_columns(r, pos, n)))
            assert got == list(range(n)), (pos, n)                                             # every column exactly once
            for r in range(4):
                lo, hi = p.block_columns(r, pos, n)
                assert all(p.owner(pos + c) == r for c in range(lo, hi))


def test_sharded_decoder_refuses_caches_longer_than_a_chunk():
    eng = FakeEngine()
    eng.cfg = type("C", (), dict(vars(_Cfg), max_seq=CHUNK + 64))()
    with pytest.raises(ValueError, match="one chunk"):
        ShardedDecoder(eng, ShardPlan(2, CHUNK), 0, None)


def test_sharded_decode_world2_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert set(ret.keys()) == {0, 1}
    assert ret[0][0] < 1e-6 and ret[1][0] < 1e-6, dict(ret)      # both ranks end with the full result
    assert ret[1][1] and not ret[0][1]                            # the owner of position 150 (rank 1) appended, rank 0 did not
