"""KV-sequence-sharded decode over two GPUs with the merge fused into the combine kernel (peer stores over NVLink +
flags), against the float64 oracle.  Needs two GPUs: skipped elsewhere."""
import os
import socket

import numpy as np
import pytest

from oracle import po

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    from pooled_b200 import AttnConfig, AttnEngine
    from pooled_b200.shard import ShardPlan, ShardedDecoder
    from tests import util
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        nH, nKV, hd, chunk, steps = 16, 2, 256, 4096, 6
        total = chunk + 1000                       # rank 0 holds 4096 rows, rank 1 holds 1000 and grows
        K = util.normal_f16(1, (total + steps, nKV * hd)); V = util.normal_f16(2, (total + steps, nKV * hd))
        Kc, Vc = po.np_f16_rne(K), po.np_f16_rne(V)
        eng = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64, rope_theta=1e7, max_seq=chunk, act_dtype=torch.float16), device=rank)
        eng.exchange_setup(rank, world, dist, max_rows=64)
        errs = []
        for mode in ("peer", "nccl"):
            sd = ShardedDecoder(eng, ShardPlan(world, chunk), rank, dist, exchange=mode)
            lo, hi = rank * chunk, min(total, (rank + 1) * chunk)
            eng.cache(0, "k")[0, :hi - lo] = torch.from_numpy(Kc[lo:hi].view(np.int16)).cuda()
            eng.cache(0, "v")[0, :hi - lo] = torch.from_numpy(Vc[lo:hi].view(np.int16)).cuda()
            Kf, Vf = Kc[:total].copy(), Vc[:total].copy()
            for t in range(steps):
                pos = total + t
                q = util.normal_f16(100 + t, (1, nH * hd)); g = util.normal_f16(200 + t, (1, nH * hd))
                d = lambda a: torch.from_numpy(a).to(torch.float16).cuda()
                out = sd.step(0, [(0, pos)], d(q), d(K[pos:pos + 1]), d(V[pos:pos + 1]), d(g)).float().cpu().numpy()
                eng.sync()
                Kf = np.concatenate([Kf, po.f16_rne(po.rope_neox_f64(K[pos], nKV, hd, 64, pos, 1e7))[None]])
                Vf = np.concatenate([Vf, Vc[pos][None]])
                ref = po.attn_f64(po.rope_neox_f64(q[0], nH, hd, 64, pos, 1e7)[None], Kf, Vf, nH, nKV, hd, pos, 1, g)
                errs.append(float(np.abs(out - ref).max()))
        # a short context that rank 1 holds nothing of (its decode kernel does not run: the call still takes its number
        # in the exchange), single tokens and a 5-token block (the tensor-core verify kernel on rank 0)
        eng0 = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64, rope_theta=1e7, max_seq=chunk, act_dtype=torch.float16), device=rank)
        eng0.exchange_setup(rank, world, dist, max_rows=128)
        sd0 = ShardedDecoder(eng0, ShardPlan(world, chunk), rank, dist, exchange="peer")
        short = 500
        K0 = util.normal_f16(51, (short + 16, nKV * hd)); V0 = util.normal_f16(52, (short + 16, nKV * hd))
        Kf, Vf = po.np_f16_rne(K0[:short]).copy(), po.np_f16_rne(V0[:short]).copy()
        if rank == 0:
            eng0.cache(0, "k")[0, :short] = torch.from_numpy(Kf.view(np.int16)).cuda()
            eng0.cache(0, "v")[0, :short] = torch.from_numpy(Vf.view(np.int16)).cuda()
        d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.float16).cuda()
        pos = short
        for n_new in (1, 1, 5, 1):
            q = util.normal_f16(500 + pos, (n_new, nH * hd)); g = util.normal_f16(600 + pos, (n_new, nH * hd))
            out = eng0.encode_layer_sharded(0, pos, d(q), d(K0[pos:pos + n_new]), d(V0[pos:pos + n_new]), d(g)).float().cpu().numpy()
            eng0.sync()
            for c in range(n_new):
                Kf = np.concatenate([Kf, po.f16_rne(po.rope_neox_f64(K0[pos + c], nKV, hd, 64, pos + c, 1e7))[None]])
                Vf = np.concatenate([Vf, po.np_f16_rne(V0[pos + c])[None]])
            qr = np.stack([po.rope_neox_f64(q[c], nH, hd, 64, pos + c, 1e7) for c in range(n_new)])
            ref = po.attn_f64(qr, Kf, Vf, nH, nKV, hd, pos, n_new, g)
            errs.append(float(np.abs(out - ref).max()))
            pos += n_new
        # a batch of three sequences, one token each per step: one whose rows all sit on rank 0's shard (rank 1 holds
        # nothing of it), two that have grown into rank 1's; the peer form is one library call per step
        totals, n_seqs = [300, chunk + 77, chunk + 1900], 3
        eng2 = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64, rope_theta=1e7, max_seq=chunk, n_seqs=n_seqs, act_dtype=torch.float16),
                          device=rank)
        eng2.exchange_setup(rank, world, dist, max_rows=64)
        Ks = [util.normal_f16(10 + s, (totals[s] + 2 * steps, nKV * hd)) for s in range(n_seqs)]
        Vs = [util.normal_f16(20 + s, (totals[s] + 2 * steps, nKV * hd)) for s in range(n_seqs)]
        full = [[po.np_f16_rne(Ks[s][:totals[s]]), po.np_f16_rne(Vs[s][:totals[s]])] for s in range(n_seqs)]
        for s in range(n_seqs):
            lo, hi = rank * chunk, min(totals[s], (rank + 1) * chunk)
            if hi > lo:
                eng2.cache(0, "k")[s, :hi - lo] = torch.from_numpy(full[s][0][lo:hi].view(np.int16)).cuda()
                eng2.cache(0, "v")[s, :hi - lo] = torch.from_numpy(full[s][1][lo:hi].view(np.int16)).cuda()
        t0 = 0
        for mode in ("peer", "nccl"):
            sd = ShardedDecoder(eng2, ShardPlan(world, chunk), rank, dist, exchange=mode)
            for t in range(t0, t0 + steps):
                sp = [(s, totals[s] + t) for s in range(n_seqs)]
                q = util.normal_f16(300 + t, (n_seqs, nH * hd)); g = util.normal_f16(400 + t, (n_seqs, nH * hd))
                kn = np.stack([Ks[s][totals[s] + t] for s in range(n_seqs)]); vn = np.stack([Vs[s][totals[s] + t] for s in range(n_seqs)])
                d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.float16).cuda()
                out = sd.step(0, sp, d(q), d(kn), d(vn), d(g)).float().cpu().numpy()
                eng2.sync()
                for s, pos in sp:
                    full[s][0] = np.concatenate([full[s][0], po.f16_rne(po.rope_neox_f64(kn[s], nKV, hd, 64, pos, 1e7))[None]])
                    full[s][1] = np.concatenate([full[s][1], po.np_f16_rne(vn[s])[None]])
                    ref = po.attn_f64(po.rope_neox_f64(q[s], nH, hd, 64, pos, 1e7)[None], full[s][0], full[s][1], nH, nKV, hd, pos, 1, g[s:s + 1])
                    errs.append(float(np.abs(out[s:s + 1] - ref).max()))
            t0 += steps
        ret[rank] = max(errs)
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharded_decode_peer_and_nccl():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert set(ret.keys()) == {0, 1} and max(ret.values()) <= 2e-3, dict(ret)
