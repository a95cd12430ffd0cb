"""Split-K decode / verify, combine and gate on the GPU against the float64 oracle, through the C ABI."""
import numpy as np
import pytest

from oracle import po
from tests import util

pytestmark = pytest.mark.gpu


def _engine(nH, nKV, hd, max_seq, act="f32", n_seqs=1, max_cols=8, n_rot=64, theta=1e7, rope_mode="f64", **kw):
    import torch
    from pooled_b200 import AttnConfig, AttnEngine
    return AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=n_rot, rope_theta=theta, max_seq=max_seq, n_seqs=n_seqs,
                                 rope_mode=rope_mode, act_dtype=torch.float32 if act == "f32" else torch.float16, max_cols=max_cols, **kw))


# ---- the reference's own kernel test, retargeted: tests/test_attn_dec.js ------------------------------

REF_RUNS = [  # (nH, nKV, maxSeq, cases) as in tests/test_attn_dec.js:106-107 (QUICK sizes first in CI there)
    (16, 2, 70000, [1, 2, 5, 63, 64, 65, 127, 128, 129, 300, 1000, 4096, 8192, 8193, 16385, 33000, 69999]),
    (24, 4, 40000, [1, 3, 64, 129, 257, 1000, 4097, 16384, 32769, 39999]),
]


@pytest.fixture(scope="module")
def ref_inputs():
    """The LCG stream of tests/test_attn_dec.js: the seed carries over from the first run to the second."""
    seed = 12345
    out = []
    for nH, nKV, max_seq, cases in REF_RUNS:
        K, V, q, seed = po.gen_attn_dec(seed, max_seq, nKV * 256, nH * 256)
        out.append((nH, nKV, max_seq, cases, K, V, q))
    return out


@pytest.mark.parametrize("run", [0, 1])
def test_attn_dec_js_cases(ref_inputs, run):
    import torch
    nH, nKV, max_seq, cases, K, V, q = ref_inputs[run]
    eng = _engine(nH, nKV, 256, max_seq, act="f32", max_cols=4, rope_mode="none")
    util.load_cache(eng, 0, 0, K, V)
    qd = util.torch_dev(q)
    worst = 0.0
    for seq_len in cases:
        pos = seq_len - 1
        one = eng.decode(0, [(0, pos, 1)], qd[0:1]).cpu().numpy()
        ref = po.attn_f64(q[0:1], K, V, nH, nKV, 256, pos, 1)
        ma, rel = util.errs(one, ref)
        worst = max(worst, rel)
        assert np.all(np.isfinite(one)) and rel < util.REF_REL, f"seqLen {seq_len}: relDiff vs f64 {rel:.2e}"
        if seq_len >= 4:
            # verify vs decode: a 4-column pass ending here against one-column passes at each position.  The reference
            # makes these bitwise equal by deriving split boundaries from each column's own position; here the
            # columns of a pass share one K/V stream, so the bound is the same 2e-5 against float64 instead.
            multi = eng.decode(0, [(0, pos - 3, 4)], qd[0:4]).cpu().numpy()
            refm = po.attn_f64(q[0:4], K, V, nH, nKV, 256, pos - 3, 4)
            assert util.errs(multi, refm)[1] < util.REF_REL
            for c in range(4):
                single = eng.decode(0, [(0, pos - 3 + c, 1)], qd[c:c + 1]).cpu().numpy()
                assert util.errs(single[0], multi[c])[1] < util.REF_REL
    eng.sync()
    print(f"run {run}: worst relDiff vs f64 {worst:.2e}")


# ---- the five benchmark configurations -------------------------------------------------------------------------

def _config_inputs(cfg_id, nH, nKV, hd, rows, n_cols, outliers=False):
    K = util.normal_f16(0xB0B + cfg_id, (rows, nKV * hd)); V = util.normal_f16(0xC0DE + cfg_id, (rows, nKV * hd))
    q = util.normal_f16(0xA11CE + cfg_id, (n_cols, nH * hd)); g = util.normal_f16(0x6A7E + cfg_id, (n_cols, nH * hd))
    if outliers:
        K = util.with_outliers(K, nKV, hd)
        # q heads of one kv head share that head's outlier channels
        G = nH // nKV
        qq = q.reshape(n_cols, nH, hd).copy()
        for h in range(nH):
            for c in po.outlier_channels(h // G, hd):
                qq[:, h, c] *= 20.0
        q = po.np_h2f(po.np_f16_rne(qq)).reshape(n_cols, nH * hd)
    return q, K, V, g


def _layer_step_vs_oracle(eng, cfgid, nH, nKV, hd, n_rot, theta, ctx, n_cols, gate, outliers, act):
    """Cache rows [0, ctx) pre-rotated; the new tokens' q, k, v go through RoPE + append + attend + gate."""
    import torch
    td = torch.float16 if act == "f16" else torch.float32
    q, K, V, g = _config_inputs(cfgid, nH, nKV, hd, ctx + n_cols, n_cols, outliers)
    Kc, Vc = po.np_f16_rne(K[:ctx]), po.np_f16_rne(V[:ctx])
    util.load_cache(eng, 0, 0, Kc, Vc)
    k_new, v_new = K[ctx:], V[ctx:]
    out = eng.encode_layer(0, ctx, util.torch_dev(q, td), util.torch_dev(k_new, td), util.torch_dev(v_new, td),
                           util.torch_dev(g, td) if gate else None, mode="decode").float().cpu().numpy()
    eng.sync()
    # oracle: the same steps on the CPU
    Kf = np.concatenate([Kc, np.stack([po.f16_rne(po.rope_neox_f64(k_new[c], nKV, hd, n_rot, ctx + c, theta)) for c in range(n_cols)])])
    Vf = np.concatenate([Vc, po.f16_rne(v_new)])
    gk, gv = util.read_cache(eng, 0, 0, ctx, n_cols)
    assert np.array_equal(gk, Kf[ctx:]) and np.array_equal(gv, Vf[ctx:]), "KV append is not bit-exact"
    q_rot = np.stack([po.rope_neox_f64(q[c], nH, hd, n_rot, ctx + c, theta) for c in range(n_cols)])
    ref = po.attn_f64(q_rot, Kf, Vf, nH, nKV, hd, ctx, n_cols, g if gate else None)
    return out, ref, (q_rot, Kf, Vf, g)


def test_config1_qwen3_17b_decode():
    # 16 q / 8 kv heads, head_dim 128, full RoPE theta 1e6 at position 4096, context 4096
    eng = _engine(16, 8, 128, 4200, act="f16", n_rot=128, theta=1e6)
    out, ref, _ = _layer_step_vs_oracle(eng, 1, 16, 8, 128, 128, 1e6, 4096, 1, False, False, "f16")
    ma, mr = util.assert_close(out, ref, "config 1")
    print(f"config 1: max-abs {ma:.2e} max-rel {mr:.2e}")


def test_config2_moe_decode_with_outliers_and_gate():
    # 16 q / 2 kv heads, head_dim 256, partial RoPE 64 dims theta 1e7, context 32768, outlier channels x20, sigmoid gate
    eng = _engine(16, 2, 256, 32768 + 8, act="f16")
    out, ref, _ = _layer_step_vs_oracle(eng, 2, 16, 2, 256, 64, 1e7, 32768, 1, True, True, "f16")
    ma, mr = util.assert_close(out, ref, "config 2")
    print(f"config 2: max-abs {ma:.2e} max-rel {mr:.2e}")


def test_config4_verify_block_equals_sequential_decodes():
    # 24 q / 4 kv heads, 5-token block against a 16384-token cache: equal to 5 sequential decodes within tolerance
    import torch
    eng = _engine(24, 4, 256, 16384 + 8, act="f16")
    out, ref, (q_rot, Kf, Vf, g) = _layer_step_vs_oracle(eng, 4, 24, 4, 256, 64, 1e7, 16384, 5, False, False, "f16")
    ma, mr = util.assert_close(out, ref, "config 4 block")
    qd = util.torch_dev(q_rot)
    for c in range(5):
        single = eng.decode(0, [(0, 16384 + c, 1)], qd[c:c + 1]).float().cpu().numpy()
        util.assert_close(single[0], ref[c], f"config 4 sequential decode {c}")
        util.assert_close(single[0], out[c], f"config 4 block column {c} vs decode")
    print(f"config 4: max-abs {ma:.2e} max-rel {mr:.2e}")


def test_config5_batched_long_context_reduced():
    # config 5's shape (8 sequences, gate) at 1/16 of its context so the float64 oracle finishes in seconds
    import torch
    n_seqs, ctx, nH, nKV, hd = 8, 8192 + 37, 16, 2, 256
    eng = _engine(nH, nKV, hd, ctx + 4, act="f16", n_seqs=n_seqs, max_cols=8)
    qs, gs, refs = [], [], []
    for s in range(n_seqs):
        q, K, V, g = _config_inputs(50 + s, nH, nKV, hd, ctx - s * 100, 1)
        Kc, Vc = po.np_f16_rne(K), po.np_f16_rne(V)
        util.load_cache(eng, 0, s, Kc, Vc)
        refs.append(po.attn_f64(q, Kc, Vc, nH, nKV, hd, ctx - s * 100 - 1, 1, g)[0]); qs.append(q[0]); gs.append(g[0])
    items = [(s, ctx - s * 100 - 1, 1) for s in range(n_seqs)]
    out = eng.decode(0, items, util.torch_dev(np.stack(qs), torch.float16), util.torch_dev(np.stack(gs), torch.float16)).float().cpu().numpy()
    eng.sync()
    util.assert_close(out, np.stack(refs), "config 5 (reduced)")


def test_config5_full_size_batched_step():
    # config 5 at its own size: 8 sequences x 131072-row context in one layer (2.1 GB of K and V), one token each at position
    # 131072 through the batched front (pa_rope_append_items) and one batched decode call.  Row offsets pass 2^30 bytes,
    # TMA row coordinates pass 10^6, the plan is 9 splits over 2049 tiles.  Sequences 0 and 7 are checked against the
    # float64 oracle (the criterion of tests/test_attn_dec.js:87-98) and their appended rows bit for bit; the other
    # sequences hold the same K/V content as sequence 0 shifted by one row each, so their outputs must be finite and
    # differ from sequence 0's.
    import torch
    n_seqs, ctx, nH, nKV, hd, n_rot, theta = 8, 131072, 16, 2, 256, 64, 1e7
    kvd, qd = nKV * hd, nH * hd
    eng = _engine(nH, nKV, hd, ctx + 8, act="f16", n_seqs=n_seqs, max_cols=8)
    base = po.np_f16_rne(po.normal(0xB0B + 5, (ctx + 8) * kvd) * 0.9).reshape(ctx + 8, kvd)
    vbase = po.np_f16_rne(po.normal(0xC0DE + 5, (ctx + 8) * kvd)).reshape(ctx + 8, kvd)
    tk, tv = torch.from_numpy(base.view(np.int16)).cuda(), torch.from_numpy(vbase.view(np.int16)).cuda()
    for s in range(n_seqs):
        eng.cache(0, "k")[s, :ctx] = tk[s:s + ctx]
        eng.cache(0, "v")[s, :ctx] = tv[s:s + ctx]
    q = util.normal_f16(0xA11CE + 5, (n_seqs, qd)); kn = util.normal_f16(71, (n_seqs, kvd)); vn = util.normal_f16(72, (n_seqs, kvd))
    g = util.normal_f16(0x6A7E + 5, (n_seqs, qd))
    d = lambda a: util.torch_dev(a, torch.float16)
    seqs_pos = [(s, ctx) for s in range(n_seqs)]
    q_rot = eng.rope_append_items(0, seqs_pos, d(q), d(kn), d(vn))
    out = eng.decode(0, [(s, ctx, 1) for s in range(n_seqs)], q_rot, d(g)).float().cpu().numpy()
    eng.sync()
    assert np.all(np.isfinite(out))
    for s in (0, n_seqs - 1):
        k_row = po.f16_rne(po.rope_neox_f64(kn[s], nKV, hd, n_rot, ctx, theta)); v_row = po.f16_rne(vn[s])
        gk, gv = util.read_cache(eng, 0, s, ctx, 1)
        assert np.array_equal(gk[0], k_row) and np.array_equal(gv[0], v_row), f"sequence {s}: appended row differs"
        Kf = np.concatenate([base[s:s + ctx], k_row[None]]); Vf = np.concatenate([vbase[s:s + ctx], v_row[None]])
        ref = po.attn_f64(po.rope_neox_f64(q[s], nH, hd, n_rot, ctx, theta)[None], Kf, Vf, nH, nKV, hd, ctx, 1, g[s][None])
        ma, mr = util.assert_close(out[s][None], ref, f"config 5 full size, sequence {s}")
        print(f"config 5 full size, sequence {s}: max-abs {ma:.2e} max-rel {mr:.2e}")
    assert all(np.abs(out[s] - out[0]).max() > 1e-3 for s in range(1, n_seqs))
    eng.destroy()


# ---- edges ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("nH,nKV,hd", [(16, 2, 256), (24, 4, 256), (16, 8, 128), (8, 8, 128), (32, 2, 256), (8, 2, 64)])
@pytest.mark.parametrize("seq_len", [1, 2, 63, 64, 65, 127, 128, 129, 1000, 4097])
def test_short_and_ragged_contexts(nH, nKV, hd, seq_len):
    eng = _engine(nH, nKV, hd, 4200, act="f32", rope_mode="none")
    q, K, V, g = _config_inputs(7, nH, nKV, hd, seq_len, 1)
    Kc, Vc = po.np_f16_rne(K), po.np_f16_rne(V)
    util.load_cache(eng, 0, 0, Kc, Vc)
    out = eng.decode(0, [(0, seq_len - 1, 1)], util.torch_dev(q), util.torch_dev(g)).cpu().numpy()
    ref = po.attn_f64(q, Kc, Vc, nH, nKV, hd, seq_len - 1, 1, g)
    assert util.errs(out, ref)[1] < util.REF_REL


def test_rows_past_a_columns_position_never_count_even_when_nan():
    # tests/unit/attn_tile_test.js:43-49: rows at or past the pass's end hold NaN and must not be used
    import torch
    nH, nKV, hd, base, nc = 16, 2, 256, 301, 8
    eng = _engine(nH, nKV, hd, 4096, act="f32", rope_mode="none")
    kc = eng.cache(0, "k"); vc = eng.cache(0, "v")
    kc.fill_(0x7e00); vc.fill_(0x7e00)
    q, K, V, _ = _config_inputs(9, nH, nKV, hd, base + nc, nc)
    Kc, Vc = po.np_f16_rne(K), po.np_f16_rne(V)
    util.load_cache(eng, 0, 0, Kc, Vc)
    out = eng.decode(0, [(0, base, nc)], util.torch_dev(q)).cpu().numpy()
    ref = po.attn_f64(q, Kc, Vc, nH, nKV, hd, base, nc)
    assert np.all(np.isfinite(out)) and util.errs(out, ref)[1] < util.REF_REL
    # column 0 must not see the later columns' rows either: poison them too and decode it alone
    kc[0, base + 1:] = 0x7e00; vc[0, base + 1:] = 0x7e00
    one = eng.decode(0, [(0, base, 1)], util.torch_dev(q[0:1])).cpu().numpy()
    assert util.errs(one[0], ref[0])[1] < util.REF_REL


def test_padded_strides_and_interleaved_gate():
    # column strides padded as in tests/unit/attn_tile_test.js:51 (nH*hd + 12 / + 20); q and gate interleaved per head as
    # q_full [nH][2*hd] (engine/wgsl/attn_dec.js:282-283)
    import torch
    nH, nKV, hd, ctx, nc = 16, 2, 256, 700, 3
    eng = _engine(nH, nKV, hd, 1024, act="f32", rope_mode="none")
    q, K, V, g = _config_inputs(3, nH, nKV, hd, ctx + nc, nc)
    Kc, Vc = po.np_f16_rne(K), po.np_f16_rne(V)
    util.load_cache(eng, 0, 0, Kc, Vc)
    ref = po.attn_f64(q, Kc, Vc, nH, nKV, hd, ctx, nc, g)
    s0, s1 = 2 * nH * hd + 12, nH * hd + 20
    qfull = torch.full((nc, s0), float("nan"), device="cuda")
    qfull[:, :2 * nH * hd] = torch.from_numpy(np.stack([q.reshape(nc, nH, hd), g.reshape(nc, nH, hd)], axis=2).reshape(nc, -1)).cuda()
    out = torch.full((nc, s1), float("nan"), device="cuda")
    eng.decode(0, [(0, ctx, nc)], qfull, gate=qfull[:, hd:], out=out, q_head_stride=2 * hd, gate_head_stride=2 * hd)
    o = out.cpu().numpy()
    assert util.errs(o[:, :nH * hd], ref)[1] < util.REF_REL
    assert np.all(np.isnan(o[:, nH * hd:])), "wrote into the padding between columns"


def test_fast_mode_stays_inside_the_baseline_tolerance():
    eng = _engine(16, 2, 256, 8300, act="f16", fast=True)
    out, ref, _ = _layer_step_vs_oracle(eng, 2, 16, 2, 256, 64, 1e7, 8192, 1, True, False, "f16")
    util.assert_close(out, ref, "fast mode")


def test_sharded_partials_merge_to_the_full_result():
    # the KV sequence cut into 4 contiguous shards, one layer per "rank"; merged records equal the unsharded decode
    import torch
    nH, nKV, hd, ctx, P = 16, 2, 256, 8192 + 11, 4
    q, K, V, g = _config_inputs(5, nH, nKV, hd, ctx, 2)
    Kc, Vc = po.np_f16_rne(K), po.np_f16_rne(V)
    ref = po.attn_f64(q[:1], Kc, Vc, nH, nKV, hd, ctx - 1, 1, g[:1])
    eng = _engine(nH, nKV, hd, ctx, act="f16", rope_mode="none", n_seqs=1)
    from pooled_b200 import AttnConfig, AttnEngine
    shard = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64, rope_theta=1e7, max_seq=ctx, n_layers=P,
                                  rope_mode="none", act_dtype=torch.float16))
    bounds = [(r * ctx) // P for r in range(P + 1)]
    parts = []
    qd = util.torch_dev(q[:1], torch.float16)
    for r in range(P):
        a, b = bounds[r], bounds[r + 1]
        util.load_cache(shard, r, 0, Kc[a:b], Vc[a:b])
        parts.append(shard.decode_partial(r, [(0, b - a - 1, 1)], qd))
    merged = shard.merge(torch.stack(parts), 1, util.torch_dev(g[:1], torch.float16)).float().cpu().numpy()
    util.assert_close(merged, ref, "sharded merge")
    # merging one record is the identity (normalise + gate)
    util.load_cache(eng, 0, 0, Kc, Vc)
    full = eng.decode(0, [(0, ctx - 1, 1)], qd, util.torch_dev(g[:1], torch.float16)).float().cpu().numpy()
    one = eng.merge(eng.decode_partial(0, [(0, ctx - 1, 1)], qd)[None], 1, util.torch_dev(g[:1], torch.float16)).float().cpu().numpy()
    assert np.array_equal(full, one)
    util.assert_close(full, merged, "sharded vs unsharded")


def test_determinism_same_bits_twice():
    eng = _engine(16, 2, 256, 9000, act="f32", rope_mode="none")
    q, K, V, g = _config_inputs(8, 16, 2, 256, 8193, 1)
    util.load_cache(eng, 0, 0, po.np_f16_rne(K), po.np_f16_rne(V))
    a = eng.decode(0, [(0, 8192, 1)], util.torch_dev(q)).cpu().numpy()
    b = eng.decode(0, [(0, 8192, 1)], util.torch_dev(q)).cpu().numpy()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_unsupported_shapes_are_refused_with_a_message():
    import torch
    from pooled_b200 import PaError
    eng = _engine(16, 2, 256, 1024, act="f32", max_cols=16, rope_mode="none")
    q = torch.zeros((9, 4096), device="cuda")
    with pytest.raises(PaError) as e:
        eng.decode(0, [(0, 100, 9)], q)     # 9 columns x 8 heads = 72 query rows per kv head
    assert e.value.code == -2 and "pa_prefill" in str(e.value)
    assert eng.stats()["calls"] == 0
    # the batched layer call: one sequence past the layer's rows, and more items than the context was created for
    eng2 = _engine(16, 2, 256, 1024, act="f32", n_seqs=2, max_cols=2)
    z = lambda n, w: torch.zeros((n, w), device="cuda")
    with pytest.raises(PaError) as e:
        eng2.encode_items(0, [(0, 10), (1, 1024)], z(2, 4096), z(2, 512), z(2, 512))
    assert "max_seq" in str(e.value)
    with pytest.raises(PaError) as e:
        eng2.encode_items(0, [(0, 10), (1, 11), (0, 12)], z(3, 4096), z(3, 512), z(3, 512))
    assert "max_cols" in str(e.value)
    assert eng2.stats()["calls"] == 0


def test_host_buffer_entry_points_match_the_device_path():
    # pa_attn_layer_host (one layer) and pa_attn_step_host (all layers of a token step) against pa_attn_layer
    import torch
    nH, nKV, hd, ctx, layers = 16, 2, 256, 3000, 3
    from pooled_b200 import AttnConfig, AttnEngine
    eng = AttnEngine(AttnConfig(n_heads=nH, n_kv_heads=nKV, head_dim=hd, n_rot=64, rope_theta=1e7, max_seq=ctx + 8, n_layers=layers,
                                act_dtype=torch.float16, max_cols=8))
    for li in range(layers):
        _, K, V, _ = _config_inputs(20 + li, nH, nKV, hd, ctx, 1)
        util.load_cache(eng, li, 0, po.np_f16_rne(K), po.np_f16_rne(V))
    mk = lambda seed, n: torch.from_numpy(util.normal_f16(seed, (layers, 2, n))).to(torch.float16).pin_memory()
    hq, hk, hv, hg = mk(1, nH * hd), mk(2, nKV * hd), mk(3, nKV * hd), mk(4, nH * hd)
    want = torch.stack([eng.encode_layer(li, ctx, hq[li].cuda(), hk[li].cuda(), hv[li].cuda(), hg[li].cuda(), mode="decode") for li in range(layers)]).cpu()
    eng.sync()
    hout = torch.empty((layers, 2, nH * hd), dtype=torch.float16).pin_memory()
    eng.encode_step_host(ctx, hq, hk, hv, hg, hout, mode="decode")
    assert torch.equal(hout, want)
    one = torch.empty((2, nH * hd), dtype=torch.float16).pin_memory()
    eng.encode_layer_host(1, ctx, hq[1], hk[1], hv[1], hg[1], one, mode="decode")
    assert torch.equal(one, want[1])


def test_exchange_merge_with_one_rank_matches_decode_over_many_calls():
    # the peer-exchange combine with world = 1 (the rank publishes to and reads from its own buffer): the call counter,
    # the two buffer parities and the flags are exercised by consecutive calls of different sizes
    import torch
    nH, nKV, hd, ctx = 16, 2, 256, 5000
    eng = _engine(nH, nKV, hd, ctx + 8, act="f32", rope_mode="none", max_cols=8)
    q, K, V, g = _config_inputs(11, nH, nKV, hd, ctx + 8, 4)
    Kc, Vc = po.np_f16_rne(K), po.np_f16_rne(V)
    util.load_cache(eng, 0, 0, Kc, Vc)
    eng.exchange_setup(0, 1, max_rows=64)
    qd, gd = util.torch_dev(q), util.torch_dev(g)
    for pos, nc in [(4999, 1), (100, 4), (4096, 2), (63, 1), (4999, 1), (2000, 3)]:
        want = eng.decode(0, [(0, pos, nc)], qd[:nc], gd[:nc]).cpu().numpy()
        got = eng.decode_exchange(0, [(0, pos, nc)], qd[:nc], gd[:nc]).cpu().numpy()
        eng.sync()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"pos {pos} nc {nc}"
    from pooled_b200 import PaError
    with pytest.raises(PaError):
        eng.decode_exchange(0, [(0, 100, 8)], torch.zeros((8, nH * hd), device="cuda"))   # 128 rows > max_rows 64


@pytest.mark.parametrize("nH,nKV,hd,n_rot,theta", [(16, 2, 256, 64, 1e7), (16, 8, 128, 128, 1e6), (8, 2, 128, 128, 1e6)])
@pytest.mark.parametrize("act", ["f16", "f32"])
def test_fused_front_equals_the_three_kernel_chain_bit_for_bit(act, nH, nKV, hd, n_rot, theta, monkeypatch):
    # One-token calls of the 64-rotary-dim / head_dim 256 shape rotate q and k and append inside the decode kernel.
    # Same cos / sin (host libm), same rotation arithmetic, same decode kernel: the cache rows and the outputs must
    # carry the same bits as the RoPE/append -> decode -> combine chain (POOLED_ATTN_NO_FUSE=1), token after token on
    # ONE layer, where each call's early K/V fetch must stay clear of the row the call before may still be writing.
    import torch
    ctx0, steps = 700, 40
    td = torch.float16 if act == "f16" else torch.float32
    rng = np.random.default_rng(11)
    K0 = util.normal_f16(21, (ctx0, nKV * hd)); V0 = util.normal_f16(22, (ctx0, nKV * hd))
    q = rng.standard_normal((steps, nH * hd)).astype(np.float32); k = rng.standard_normal((steps, nKV * hd)).astype(np.float32)
    v = rng.standard_normal((steps, nKV * hd)).astype(np.float32); g = rng.standard_normal((steps, nH * hd)).astype(np.float32)
    if act == "f16":
        q, k, v, g = (po.h2f(po.f16_rne(x)) for x in (q, k, v, g))
    outs, caches = {}, {}
    for mode in ("fused", "chain"):
        if mode == "chain":
            monkeypatch.setenv("POOLED_ATTN_NO_FUSE", "1")
        else:
            monkeypatch.delenv("POOLED_ATTN_NO_FUSE", raising=False)
        eng = _engine(nH, nKV, hd, ctx0 + steps + 8, act=act, n_rot=n_rot, theta=theta)
        util.load_cache(eng, 0, 0, po.f16_rne(K0), po.f16_rne(V0))
        dq, dk, dv, dg = (util.torch_dev(x, td) for x in (q, k, v, g))
        out = torch.empty((steps, nH * hd), dtype=td, device="cuda")
        for t in range(steps):     # back to back, no synchronisation in between
            eng.encode_layer(0, ctx0 + t, dq[t:t + 1], dk[t:t + 1], dv[t:t + 1], dg[t:t + 1], out[t:t + 1], mode="decode")
        eng.sync()
        outs[mode] = out.float().cpu().numpy()
        caches[mode] = util.read_cache(eng, 0, 0, ctx0, steps)
    assert np.array_equal(caches["fused"][0], caches["chain"][0]) and np.array_equal(caches["fused"][1], caches["chain"][1])
    assert np.array_equal(outs["fused"].view(np.uint32), outs["chain"].view(np.uint32))
    # and against the oracle: the appended rows bit for bit
    wk = np.stack([po.f16_rne(po.rope_neox_f64(k[t], nKV, hd, n_rot, ctx0 + t, theta)) for t in range(steps)])
    assert np.array_equal(caches["fused"][0], wk) and np.array_equal(caches["fused"][1], po.f16_rne(v))


@pytest.mark.parametrize("nH,nKV,hd,n_rot,theta", [(16, 2, 256, 64, 1e7), (16, 8, 128, 128, 1e6)])
@pytest.mark.parametrize("act", ["f16", "f32"])
def test_batched_layer_call_equals_append_items_then_decode_bit_for_bit(act, nH, nKV, hd, n_rot, theta):
    # pa_attn_items: one token of each of several sequences, every one at its own position, in ONE call per step (the
    # decode kernel's fused front per item) against pa_rope_append_items + pa_decode: same cache rows, same output bits,
    # step after step on one layer without synchronisation; the last step against the float64 oracle.
    import torch
    n_seqs, steps = 5, 12
    ctx0 = [700, 64, 1, 1290, 333]      # ragged: a sequence whose new row opens a tile, one of a single row
    td = torch.float16 if act == "f16" else torch.float32
    rng = np.random.default_rng(23)
    K0 = [util.normal_f16(31 + s, (ctx0[s], nKV * hd)) for s in range(n_seqs)]
    V0 = [util.normal_f16(41 + s, (ctx0[s], nKV * hd)) for s in range(n_seqs)]
    mk = lambda n: rng.standard_normal((steps, n_seqs, n)).astype(np.float32)
    q, k, v, g = mk(nH * hd), mk(nKV * hd), mk(nKV * hd), mk(nH * hd)
    if act == "f16":
        q, k, v, g = (po.h2f(po.f16_rne(x)) for x in (q, k, v, g))
    outs, caches = {}, {}
    for mode in ("one_call", "two_calls"):
        eng = _engine(nH, nKV, hd, max(ctx0) + steps + 8, act=act, n_seqs=n_seqs, n_rot=n_rot, theta=theta)
        for s in range(n_seqs):
            util.load_cache(eng, 0, s, po.f16_rne(K0[s]), po.f16_rne(V0[s]))
        dq, dk, dv, dg = (util.torch_dev(x, td) for x in (q, k, v, g))
        out = torch.empty((steps, n_seqs, nH * hd), dtype=td, device="cuda")
        for t in range(steps):
            sp = [(s, ctx0[s] + t) for s in range(n_seqs)]
            if mode == "one_call":
                eng.encode_items(0, sp, dq[t], dk[t], dv[t], dg[t], out[t])
            else:
                q_rot = eng.rope_append_items(0, sp, dq[t], dk[t], dv[t])
                eng.decode(0, [(s, p, 1) for s, p in sp], q_rot, dg[t], out[t])
        eng.sync()
        outs[mode] = out.float().cpu().numpy()
        caches[mode] = [util.read_cache(eng, 0, s, 0, ctx0[s] + steps) for s in range(n_seqs)]
    for s in range(n_seqs):
        assert np.array_equal(caches["one_call"][s][0], caches["two_calls"][s][0]) and np.array_equal(caches["one_call"][s][1], caches["two_calls"][s][1])
    assert np.array_equal(outs["one_call"].view(np.uint32), outs["two_calls"].view(np.uint32))
    t = steps - 1
    for s in range(n_seqs):
        Kc, Vc = caches["one_call"][s]
        qr = po.rope_neox_f64(q[t, s], nH, hd, n_rot, ctx0[s] + t, theta).astype(np.float32)[None]
        ref = po.attn_f64(qr, Kc, Vc, nH, nKV, hd, ctx0[s] + t, 1, gate=g[t, s][None])
        util.assert_close(outs["one_call"][t, s][None], ref, f"sequence {s}")
        wk = po.f16_rne(po.rope_neox_f64(k[t, s], nKV, hd, n_rot, ctx0[s] + t, theta))
        assert np.array_equal(caches["one_call"][s][0][ctx0[s] + t], wk)


@pytest.mark.parametrize("n_cols,mode", [(1, "decode"), (5, "decode"), (160, "prefill")])
def test_layer_call_with_head_norm_is_attn_glue_kv_plus_core_plus_gate(n_cols, mode):
    # engine/wgsl/layer_fuse.js:87-146 + attn core + gate in one call: q_full (q and gate interleaved per head) and k go in
    # un-normed; the library norms q and k (tests/reference/ref_q38.mjs:163-164), rotates, appends, attends, gates.
    # f32 activations: the normed values are not f16 numbers, so the cache rows are checked bit for bit after the oracle's
    # own norm -> rope -> f16 chain.
    import torch
    nH, nKV, hd, n_rot, theta, ctx0, eps = 16, 2, 256, 64, 1e7, 500, 1e-6
    eng = _engine(nH, nKV, hd, ctx0 + n_cols + 8, act="f32", max_cols=max(8, n_cols))
    rng = np.random.default_rng(17)
    K0 = util.normal_f16(31, (ctx0, nKV * hd)); V0 = util.normal_f16(32, (ctx0, nKV * hd))
    util.load_cache(eng, 0, 0, po.f16_rne(K0), po.f16_rne(V0))
    q_full = (rng.standard_normal((n_cols, nH * 2 * hd)) * 2).astype(np.float32)      # [head][q hd | gate hd]
    k = (rng.standard_normal((n_cols, nKV * hd)) * 3).astype(np.float32)
    v = rng.standard_normal((n_cols, nKV * hd)).astype(np.float32)
    qw = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32); kw = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    dqw, dkw = util.torch_dev(qw), util.torch_dev(kw)
    eng.set_head_norm(0, dqw, dkw, eps)
    dqf = util.torch_dev(q_full)
    out = eng.encode_layer(0, ctx0, dqf, util.torch_dev(k), util.torch_dev(v), dqf[:, hd:], mode=mode, q_head_stride=2 * hd,
                           gate_head_stride=2 * hd).cpu().numpy()
    eng.sync()
    qv = q_full.reshape(n_cols, nH, 2 * hd)
    q_plain, g = np.ascontiguousarray(qv[:, :, :hd]).reshape(n_cols, -1), np.ascontiguousarray(qv[:, :, hd:]).reshape(n_cols, -1)
    q_rot = np.stack([po.rope_neox_f64(po.head_norm_f64(q_plain[c], nH, hd, qw, eps), nH, hd, n_rot, ctx0 + c, theta) for c in range(n_cols)])
    k_rot = np.stack([po.rope_neox_f64(po.head_norm_f64(k[c], nKV, hd, kw, eps), nKV, hd, n_rot, ctx0 + c, theta) for c in range(n_cols)])
    Kf = np.concatenate([po.f16_rne(K0), po.f16_rne(k_rot)]); Vf = np.concatenate([po.f16_rne(V0), po.f16_rne(v)])
    gk, gv = util.read_cache(eng, 0, 0, ctx0, n_cols)
    bad = int(np.count_nonzero(gk != Kf[ctx0:]))
    assert bad <= (0 if n_cols * (n_rot // 2) <= 64 else 2), f"{bad} cache halves differ"     # wide calls: device sin/cos, last place
    assert np.array_equal(gv, Vf[ctx0:])
    cols = range(n_cols) if n_cols <= 8 else [0, 1, 63, 64, 127, 159]
    ref = np.stack([po.attn_f64(q_rot[c:c + 1], Kf, Vf, nH, nKV, hd, ctx0 + c, 1, g[c:c + 1])[0] for c in cols])
    util.assert_close(out[list(cols)], ref, f"head-norm layer call, {n_cols} columns")
    # switched off again: the same call without the norm differs
    eng.set_head_norm(0, None, None)
    out2 = eng.encode_layer(0, ctx0, dqf, util.torch_dev(k), util.torch_dev(v), dqf[:, hd:], mode=mode, q_head_stride=2 * hd,
                            gate_head_stride=2 * hd).cpu().numpy()
    assert np.abs(out2 - out).max() > 1e-3


@pytest.mark.parametrize("n_cols,nH,nKV", [(5, 24, 4), (3, 16, 2), (8, 16, 2)])
def test_token_blocks_back_to_back_on_one_layer(n_cols, nH, nKV):
    # 30 k-token blocks of f16 activations, one after another without synchronisation on ONE layer: each block's early K/V
    # fetch must stay clear of rows still being written, and the blocks' rows straddle tile and split boundaries somewhere
    # along the way.  Cache rows against the oracle (device sin/cos for these wide calls: last-place slack), the last block's
    # output against float64 attention over everything before it.
    import torch
    hd, ctx0, blocks = 256, 1000, 30
    rng = np.random.default_rng(23)
    T = n_cols * blocks
    K0 = util.normal_f16(41, (ctx0, nKV * hd)); V0 = util.normal_f16(42, (ctx0, nKV * hd))
    f16 = lambda x: po.h2f(po.f16_rne(x.astype(np.float32)))
    q, g = f16(rng.standard_normal((T, nH * hd))), f16(rng.standard_normal((T, nH * hd)))
    k, v = f16(rng.standard_normal((T, nKV * hd)) * 2), f16(rng.standard_normal((T, nKV * hd)))
    eng = _engine(nH, nKV, hd, ctx0 + T + 8, act="f16", max_cols=8)
    util.load_cache(eng, 0, 0, po.f16_rne(K0), po.f16_rne(V0))
    dq, dk, dv, dg = (util.torch_dev(x, torch.float16) for x in (q, k, v, g))
    out = torch.empty((T, nH * hd), dtype=torch.float16, device="cuda")
    for b in range(blocks):
        s = slice(b * n_cols, (b + 1) * n_cols)
        eng.encode_layer(0, ctx0 + b * n_cols, dq[s], dk[s], dv[s], dg[s], out[s], mode="decode")
    eng.sync()
    o = out.float().cpu().numpy()
    gk, gv = util.read_cache(eng, 0, 0, ctx0, T)
    wk = np.stack([po.f16_rne(po.rope_neox_f64(k[t], nKV, hd, 64, ctx0 + t, 1e7)) for t in range(T)])
    assert int(np.count_nonzero(gk != wk)) <= 2 and np.array_equal(gv, po.f16_rne(v))
    Kf = np.concatenate([po.f16_rne(K0), gk]); Vf = np.concatenate([po.f16_rne(V0), gv])
    p0 = ctx0 + T - n_cols
    q_rot = np.stack([po.rope_neox_f64(q[T - n_cols + c], nH, hd, 64, p0 + c, 1e7) for c in range(n_cols)])
    ref = po.attn_f64(q_rot, Kf, Vf, nH, nKV, hd, p0, n_cols, g[T - n_cols:])
    util.assert_close(o[T - n_cols:], ref, "token blocks, last block")
