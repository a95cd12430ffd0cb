"""RoPE and KV append on the GPU against the CPU oracle: bit-exact."""
import numpy as np
import pytest

from oracle import po
from tests import util

pytestmark = pytest.mark.gpu


def _engine(**kw):
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    d = dict(n_heads=16, n_kv_heads=2, head_dim=256, n_rot=64, rope_theta=1e7, max_seq=512, act_dtype=torch.float32, max_cols=64)
    d.update(kw)
    return AttnEngine(AttnConfig(**d))


def test_kv_append_conversion_is_bit_exact_on_every_class_of_value():
    # tests/test_q38flash_mc.js:231-236: the cache half == f16bits(f32 value), for every value
    import torch
    eng = _engine()
    rng = np.random.default_rng(1)
    kvd = eng.cfg.kv_dim
    n_cols = 64
    x = rng.integers(0, 2**32, size=2 * n_cols * kvd, dtype=np.uint64).astype(np.uint32).view(np.float32).copy()
    # plant every half-way case of a run of f16 values, subnormals, overflow edges, infinities, NaN, signed zero
    h = np.arange(0, 4096, dtype=np.uint16) * 16 + 3
    mid = ((po.h2f(h).astype(np.float64) + po.h2f(h + 1).astype(np.float64)) / 2).astype(np.float32)
    special = np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, -65520.0, 1e30, np.inf, -np.inf, np.nan, 2.0**-24, 2.0**-25, 2.0**-25 * 1.0001,
                        6.0e-8, -3.1e-5, 6.1035e-5], dtype=np.float32)
    x[:mid.size] = mid; x[mid.size:2 * mid.size] = -mid; x[2 * mid.size:2 * mid.size + special.size] = special
    k, v = x[:n_cols * kvd].reshape(n_cols, kvd), x[n_cols * kvd:].reshape(n_cols, kvd)
    eng.kv_append(0, 0, 100, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
    eng.sync()
    gk, gv = util.read_cache(eng, 0, 0, 100, n_cols)
    assert np.array_equal(gk, po.f16_rne(k)) and np.array_equal(gv, po.f16_rne(v))


@pytest.mark.parametrize("hd,n_rot,theta,nH,nKV,pos,n_cols,dtype", [
    (128, 128, 1e6, 16, 8, 4096, 1, "f16"),      # config 1: full RoPE
    (256, 64, 1e7, 16, 2, 32768, 1, "f16"),      # config 2
    (256, 64, 1e7, 16, 2, 131072, 1, "f32"),     # config 5 position
    (256, 64, 1e7, 24, 4, 16384, 5, "f16"),      # config 4 block
    (256, 64, 1e7, 24, 4, 0, 64, "f32"),         # start of a prefill
    (256, 64, 1e7, 24, 4, 8128, 64, "f16"),      # end of config 3's prompt
])
def test_rope_append_matches_oracle_bit_for_bit(hd, n_rot, theta, nH, nKV, pos, n_cols, dtype):
    import torch
    td = torch.float16 if dtype == "f16" else torch.float32
    eng = _engine(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=theta, max_seq=pos + n_cols + 3, act_dtype=td)
    qd, kvd = nH * hd, nKV * hd
    q = util.normal_f16(10, (n_cols, qd)); k = util.normal_f16(11, (n_cols, kvd)); v = util.normal_f16(12, (n_cols, kvd))
    if dtype == "f32":   # values that are not f16-representable
        q = po.normal(10, n_cols * qd).astype(np.float32).reshape(n_cols, qd)
        k = po.normal(11, n_cols * kvd).astype(np.float32).reshape(n_cols, kvd)
        v = po.normal(12, n_cols * kvd).astype(np.float32).reshape(n_cols, kvd)
    # the rows on either side of the appended ones carry a pattern no conversion produces here
    POISON = 0x5a5a
    for name in ("k", "v"):
        c = eng.cache(0, name)
        if pos > 0:
            c[0, pos - 1] = POISON
        c[0, pos + n_cols:pos + n_cols + 3] = POISON
    q_rot = eng.rope_append(0, 0, pos, util.torch_dev(q, td), util.torch_dev(k, td), util.torch_dev(v, td))
    eng.sync()
    gk, gv = util.read_cache(eng, 0, 0, pos, n_cols)
    gq = q_rot.cpu().numpy()
    bad_k = bad_q = 0
    for c in range(n_cols):
        wq = po.rope_neox_f64(q[c], nH, hd, n_rot, pos + c, theta)
        wk = po.rope_neox_f64(k[c], nKV, hd, n_rot, pos + c, theta)
        bad_q += int(np.count_nonzero(gq[c].view(np.uint32) != wq.view(np.uint32)))
        bad_k += int(np.count_nonzero(gk[c] != po.f16_rne(wk)))
        assert np.array_equal(gv[c], po.f16_rne(v[c]))
    # the device's float64 sin/cos and the host libm's can differ in the last place; a flip of the f32 store needs that
    # difference to straddle an f32 rounding boundary (about 1e-8 per element) and a flip of the f16 cache value
    # needs the f32 flip to straddle an f16 boundary too.  On these seeded inputs neither happens.
    assert bad_k == 0, f"{bad_k} cache halves differ"
    assert bad_q <= 2, f"{bad_q} rotated q values differ in f32 bits"
    # rows around the appended ones are untouched: the poison is still there
    after_k, after_v = util.read_cache(eng, 0, 0, pos + n_cols, 3)
    assert np.all(after_k == POISON) and np.all(after_v == POISON), "rows past the appended ones were written"
    if pos > 0:
        before_k, before_v = util.read_cache(eng, 0, 0, pos - 1, 1)
        assert np.all(before_k == POISON) and np.all(before_v == POISON), "the row before the appended ones was written"


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_one_token_rope_is_the_float64_expression_bit_for_bit(dtype):
    # One-token calls take cos / sin from the host's libm (as the oracle does) and rotate with f32-pair arithmetic that
    # must reproduce fl32(fl64(fl64(a cos) -/+ fl64(b sin))) exactly, falling back to float64 instructions near a
    # rounding boundary (about one output in 2^17): 2.4M rotated values per dtype, no differing bit allowed.
    import torch
    td = torch.float16 if dtype == "f16" else torch.float32
    nH, nKV, hd, n_rot, theta = 16, 8, 128, 128, 1e6
    eng = _engine(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=theta, max_seq=40000, act_dtype=td)
    qd, kvd = nH * hd, nKV * hd
    rng = np.random.default_rng(5)
    n_calls = 800
    scales = [1.0, 20.0, 1e-3, 300.0]
    bad_q = bad_k = 0
    for it in range(n_calls):
        pos = int(rng.integers(0, 39000))
        sc = scales[it % len(scales)]
        q = (rng.standard_normal(qd) * sc).astype(np.float32); k = (rng.standard_normal(kvd) * sc).astype(np.float32)
        v = rng.standard_normal(kvd).astype(np.float32)
        if dtype == "f16":
            q, k, v = (po.h2f(po.f16_rne(x)) for x in (q, k, v))
        if it % 7 == 0:
            q[rng.integers(0, qd, 64)] = 0.0; k[rng.integers(0, kvd, 64)] = 0.0
        q_rot = eng.rope_append(0, 0, pos, util.torch_dev(q[None], td), util.torch_dev(k[None], td), util.torch_dev(v[None], td))
        gq = q_rot.cpu().numpy()[0]
        gk, _ = util.read_cache(eng, 0, 0, pos, 1)
        wq = po.rope_neox_f64(q, nH, hd, n_rot, pos, theta)
        wk = po.rope_neox_f64(k, nKV, hd, n_rot, pos, theta)
        bad_q += int(np.count_nonzero(gq.view(np.uint32) != wq.view(np.uint32)))
        bad_k += int(np.count_nonzero(gk[0] != po.f16_rne(wk)))
    assert bad_q == 0 and bad_k == 0, f"{bad_q} rotated q values and {bad_k} cache halves differ"


def test_angle_table_is_refilled_when_a_graph_replay_may_have_rewritten_it():
    # Wide calls (more than 64 angles) read cos / sin from a device table that the library fills once per (position,
    # width) and reuses across layers.  A captured graph refills it on replay, so a stand-alone call that follows must
    # not trust what it wrote there before the replay.
    import torch
    nH, nKV, hd, n_rot, theta, n_cols = 4, 2, 128, 128, 1e6, 32
    eng = _engine(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=theta, max_seq=4096, act_dtype=torch.float32, max_cols=n_cols)
    qd, kvd = nH * hd, nKV * hd
    q = po.normal(3, n_cols * qd).astype(np.float32).reshape(n_cols, qd)
    k = po.normal(4, n_cols * kvd).astype(np.float32).reshape(n_cols, kvd)
    dq, dk, dv = (util.torch_dev(x) for x in (q, k, k))
    want = lambda pos: np.stack([po.rope_neox_f64(q[c], nH, hd, n_rot, pos + c, theta) for c in range(n_cols)])
    close = lambda got, pos: int(np.count_nonzero(got.view(np.uint32) != want(pos).view(np.uint32))) <= 4   # device vs host sin/cos, last place
    pos_a, pos_b = 1000, 2000
    eng.rope_append(0, 0, pos_a, dq, dk, dv)
    torch.cuda.synchronize()
    cs = torch.cuda.Stream()
    cs.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(cs):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=cs):
            out_a = eng.rope_append(0, 0, pos_a, dq, dk, dv)
            out_a2 = eng.rope_append(0, 0, pos_a, dq, dk, dv)      # same capture, same columns: shares the table
    torch.cuda.current_stream().wait_stream(cs)
    out_b = eng.rope_append(0, 0, pos_b, dq, dk, dv).cpu().numpy()
    assert close(out_b, pos_b)
    g.replay()                                                     # rewrites the table for pos_a
    torch.cuda.synchronize()
    assert close(out_a.cpu().numpy(), pos_a) and close(out_a2.cpu().numpy(), pos_a)
    out_b2 = eng.rope_append(0, 0, pos_b, dq, dk, dv).cpu().numpy()   # same key as before the replay
    assert close(out_b2, pos_b)
    g.replay()
    torch.cuda.synchronize()
    assert close(out_a.cpu().numpy(), pos_a)


def test_rope_table_mode_matches_ggml_recurrence_bit_for_bit():
    # the Flash engine's host-computed table: engine/qwen4exp.js:549-553, tests/reference/qsa_ref.mjs:99-110
    import torch
    eng = _engine(n_heads=4, n_kv_heads=2, head_dim=256, n_rot=64, rope_theta=1e7, rope_mode="table", max_seq=4096)
    n_cols, pos = 7, 1000
    q = po.normal(1, n_cols * 4 * 256).astype(np.float32).reshape(n_cols, -1)
    k = po.normal(2, n_cols * 2 * 256).astype(np.float32).reshape(n_cols, -1)
    v = po.normal(3, n_cols * 2 * 256).astype(np.float32).reshape(n_cols, -1)
    cs = np.stack([po.rope_table_f32(64, pos + c, 1e7) for c in range(n_cols)])
    q_rot = eng.rope_append(0, 0, pos, util.torch_dev(q), util.torch_dev(k), util.torch_dev(v), cs_table=util.torch_dev(cs))
    eng.sync()
    gk, gv = util.read_cache(eng, 0, 0, pos, n_cols)
    for c in range(n_cols):
        assert np.array_equal(q_rot[c].cpu().numpy(), po.rope_ggml_f32(q[c], 4, 256, 64, pos + c, 1e7))
        assert np.array_equal(gk[c], po.f16_rne(po.rope_ggml_f32(k[c], 2, 256, 64, pos + c, 1e7)))
        assert np.array_equal(gv[c], po.f16_rne(v[c]))


def test_standalone_rope_and_gate():
    import torch
    eng = _engine(n_heads=16, n_kv_heads=2)
    x = po.normal(5, 3 * 16 * 256).astype(np.float32).reshape(3, -1)
    y = eng.rope(util.torch_dev(x), 16, 77).cpu().numpy()
    for c in range(3):
        assert np.array_equal(y[c], po.rope_neox_f64(x[c], 16, 256, 64, 77 + c, 1e7))
    a = po.normal(6, 3 * 4096).astype(np.float32).reshape(3, -1); g = po.normal(7, 3 * 4096).astype(np.float32).reshape(3, -1)
    at = util.torch_dev(a)
    eng.sigmoid_mul(at, util.torch_dev(g))
    want = a.astype(np.float64) / (1 + np.exp(-g.astype(np.float64)))
    assert np.max(np.abs(at.cpu().numpy() - want)) < 1e-6


def test_arguments_are_checked():
    import torch
    from pooled_b200 import PaError
    eng = _engine(max_seq=128, max_cols=4)
    k = torch.zeros((2, eng.cfg.kv_dim), device="cuda")
    with pytest.raises(PaError) as e:
        eng.kv_append(0, 0, 127, k, k)          # rows 127, 128 pass max_seq
    assert e.value.code == -1 and "max_seq" in str(e.value)
    with pytest.raises(PaError):
        eng.kv_append(0, 1, 0, k, k)            # sequence 1 of 1
    with pytest.raises(PaError):
        eng.kv_append(0, 0, 0, torch.zeros((5, eng.cfg.kv_dim), device="cuda"), torch.zeros((5, eng.cfg.kv_dim), device="cuda"))
    eng.kv_append(0, 0, 126, k, k)               # still usable after argument errors
    eng.sync()


@pytest.mark.parametrize("hd,heads,n_cols,dtype", [(256, 16, 1, "f32"), (256, 2, 5, "f32"), (128, 24, 33, "f32"), (256, 6, 4, "f16")])
def test_head_norm_matches_the_reference_arithmetic_bit_for_bit(hd, heads, n_cols, dtype):
    # tests/reference/ref_q38.mjs:50-57, :163-164: serial float64 sum of squares, inv = 1/sqrt(ss/n + eps), f32((x*inv)*w);
    # padded column stride and interleaved heads (q_full layout: head stride 2*hd) as the engine hands them over
    import torch
    td = torch.float16 if dtype == "f16" else torch.float32
    eng = _engine(n_heads=heads, n_kv_heads=1 if heads % 2 else 2, head_dim=hd, n_rot=64, act_dtype=td)
    hs, cs = 2 * hd, heads * 2 * hd + 12
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((n_cols, cs)) * 3).astype(np.float32)
    x[0, :hd] *= 1e-3; x[-1, hd * 2:hd * 3] *= 40
    if dtype == "f16":
        x = po.h2f(po.f16_rne(x))
    w = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    dx = util.torch_dev(x, td)
    out = torch.zeros_like(dx)
    eng.head_norm(dx, heads, util.torch_dev(w), 1e-6, head_stride=hs, out=out)
    got = out.float().cpu().numpy()
    for c in range(n_cols):
        for h in range(heads):
            want = po.head_norm_f64(x[c, h * hs:h * hs + hd], 1, hd, w, 1e-6)
            g = got[c, h * hs:h * hs + hd]
            if dtype == "f16":
                assert np.array_equal(po.f16_rne(g), po.f16_rne(want))
            else:
                assert np.array_equal(g.view(np.uint32), want.view(np.uint32)), (c, h)
            assert not got[c, h * hs + hd:(h + 1) * hs].any()      # the gate half of q_full is not touched
    # in place
    eng.head_norm(dx, heads, util.torch_dev(w), 1e-6, head_stride=hs)
    assert torch.equal(dx[:, :heads * hs].view(n_cols, heads, hs)[:, :, :hd], out[:, :heads * hs].view(n_cols, heads, hs)[:, :, :hd])


def test_rope_append_items_equals_per_sequence_calls():
    # one token of each of 8 sequences at different positions in one launch == 8 pa_rope_append calls, bit for bit; with a
    # shard origin set, items outside the shard are rotated but not appended
    import torch
    nH, nKV, hd, n_rot, theta, n_seqs = 16, 2, 256, 64, 1e7, 8
    mk = lambda: _engine(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=theta, max_seq=600, act_dtype=torch.float16, n_seqs=n_seqs, max_cols=8)
    a, b = mk(), mk()
    rng = np.random.default_rng(3)
    q = po.h2f(po.f16_rne(rng.standard_normal((n_seqs, nH * hd)).astype(np.float32)))
    k = po.h2f(po.f16_rne(rng.standard_normal((n_seqs, nKV * hd)).astype(np.float32)))
    v = po.h2f(po.f16_rne(rng.standard_normal((n_seqs, nKV * hd)).astype(np.float32)))
    dq, dk, dv = (util.torch_dev(x, torch.float16) for x in (q, k, v))
    seqs_pos = [(s, 37 * s + 5) for s in range(n_seqs)]
    qa = a.rope_append_items(0, seqs_pos, dq, dk, dv).cpu().numpy()
    qb = np.concatenate([b.rope_append(0, s, p, dq[i:i + 1], dk[i:i + 1], dv[i:i + 1]).cpu().numpy() for i, (s, p) in enumerate(seqs_pos)])
    assert np.array_equal(qa.view(np.uint32), qb.view(np.uint32))
    for s, p in seqs_pos:
        ka, va = util.read_cache(a, 0, s, p, 1); kb, vb = util.read_cache(b, 0, s, p, 1)
        assert np.array_equal(ka, kb) and np.array_equal(va, vb)
        assert np.array_equal(ka[0], po.f16_rne(po.rope_neox_f64(k[s], nKV, hd, n_rot, p, theta)))
    # a shard that starts at global position 100: items below it leave the caches alone
    c = mk(); c.set_origin(0, 100)
    before = c.cache(0, "k").clone()
    qc = c.rope_append_items(0, seqs_pos, dq, dk, dv).cpu().numpy()
    assert np.array_equal(qc.view(np.uint32), qa.view(np.uint32))
    after = c.cache(0, "k")
    for s, p in seqs_pos:
        if p >= 100:
            assert np.array_equal(after[s, p - 100].cpu().numpy().view(np.uint16), util.read_cache(a, 0, s, p, 1)[0][0])
    touched = (after != before).any(dim=2).sum().item()
    assert touched <= sum(1 for _, p in seqs_pos if p >= 100)
