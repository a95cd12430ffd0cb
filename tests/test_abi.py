"""The C-ABI library without a GPU: it loads, exports every declared symbol, its host mirrors agree with the
reference's arithmetic, and it refuses to run without a device instead of falling back."""
import ctypes as C
import os
import re

import pytest

import pooled_b200
from pooled_b200 import lib as L
from pooled_b200 import attn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pa():
    from pooled_b200 import build
    build.build()
    return L.load()


def test_exports_every_declared_symbol(pa):
    hdr = open(os.path.join(ROOT, "include", "pooled_attn.h")).read()
    declared = set(re.findall(r"PA_API\s+[\w\s\*]+?\b(pa_\w+)\s*\(", hdr))
    assert len(declared) >= 25
    assert declared == set(L.SYMBOLS), (declared ^ set(L.SYMBOLS))
    for name in declared:
        assert getattr(pa.dll, name) is not None
    assert b"sm_100a" in pa.pa_version()


def test_js_binding_table_names_every_export():
    # js/pooled_attn.js is the Deno FFI table a maintainer copies; it must list exactly the header's exports, with as
    # many parameters as the ctypes table that the GPU tests call through
    js = open(os.path.join(ROOT, "js", "pooled_attn.js")).read()
    table = js[js.index("export const SYMBOLS = {"):js.index("\n};")]
    entries = dict(re.findall(r"^\s+(pa_\w+): \{ parameters: \[(.*?)\], result:", table, flags=re.M))
    assert set(entries) == set(L.SYMBOLS), set(entries) ^ set(L.SYMBOLS)
    for name, params in entries.items():
        n = len([x for x in params.split(",") if x.strip()])
        assert n == len(L.SYMBOLS[name][1]), name


def test_struct_layouts_match_the_header():
    assert C.sizeof(L.PaConfig) == 4 * 4 + 8 + 5 * 4 + 5 * 4 + 4 or C.sizeof(L.PaConfig) % 8 == 0
    assert C.sizeof(L.PaItem) == 16 and C.sizeof(L.PaStats) == 24
    assert L.PaConfig.rope_theta.offset == 16 and L.PaConfig.rope_mode.offset == 24


def test_split_mirrors_match_reference_values(pa):
    # the values the reference's rule gives at the benchmark shapes (engine/wgsl/attn_dec.js:40-48)
    assert pa.pa_dec_config(256, 8, 2, 0) == 128 and pa.pa_dec_config(256, 6, 4, 0) == 64
    assert pa.pa_dec_config(128, 2, 8, 0) == 0           # head_dim 128: the reference's split-K decode refuses it
    assert pa.pa_dec_config(256, 9, 2, 0) == 0 and pa.pa_dec_config(256, 8, 2, 40) == 40
    assert (pa.pa_dec_split_len(32768, 128), pa.pa_dec_splits(32768, 128)) == (256, 128)
    assert (pa.pa_dec_split_len(32769, 128), pa.pa_dec_splits(32769, 128)) == (320, 103)
    assert (pa.pa_dec_split_len(16385, 64), pa.pa_dec_splits(16385, 64)) == (320, 52)
    assert pa.pa_dec_split_len(1, 128) == 64 and pa.pa_dec_splits(1, 128) == 1
    for S in (16, 64, 128):
        for s in list(range(1, 700)) + [4096, 8193, 69999, 131073]:
            assert pa.pa_dec_split_len(s, S) == attn.dec_split_len(s, S)
            assert pa.pa_dec_splits(s, S) == attn.dec_splits(s, S)
            sl = attn.dec_split_len(s, S)
            assert sl % 64 == 0 and attn.dec_splits(s, S) <= S and sl * attn.dec_splits(s, S) >= s
    assert attn.attn_dec_config(256, 8, 2) == {"HD": 256, "G": 8, "S": 128, "R": 1}
    assert attn.attn_dec_config(128, 2, 8) is None and attn.attn_dec_config(256, 8, 2, kvQ8=True) is None


def test_tile_mirrors(pa):
    # tests/unit/attn_tile_test.js:84-100: a multiple of 64, at least 64, at most faSplit, never more than faSplits splits
    for max_seq in (256, 512, 2048, 4096, 16384, 65536, 262144):
        fa_split = max(256, -(-max_seq // 128 // 64) * 64)
        fa_splits = -(-max_seq // fa_split)
        for target in (1, 8, 32, 64):
            c = attn.attn_tile_config(256, 8, fa_split, fa_splits, target=target)
            for seq_end in range(1, max_seq + 1, max(1, max_seq // 499)):
                tl = attn.tile_split_len(seq_end, c)
                assert tl % 64 == 0 and 64 <= tl <= fa_split and -(-seq_end // tl) <= fa_splits
                assert pa.pa_tile_split_len(seq_end, fa_split, fa_splits, target) == tl
    # tests/unit/attn_tile_test.js:113-114
    assert attn.attn_tile_config(256, 8, 256, 64, wgMem=32768)["TK"] == 16 and attn.attn_tile_config(256, 8, 256, 64, wgMem=16384)["TK"] == 8
    assert attn.attn_tile_config(256, 6, 256, 64)["CW"] == 10 and attn.attn_tile_config(250, 6, 256, 64) is None


def test_no_device_is_an_error_not_a_fallback(pa):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    cfg = L.PaConfig(n_heads=16, n_kv_heads=2, head_dim=256, n_rot=64, rope_theta=1e7, rope_mode=1, act_dtype=1, max_cols=8)
    h = C.c_void_p()
    rc = pa.pa_create(0, C.byref(cfg), C.byref(h))
    assert rc == -4 and not h.value
    assert b"no CPU fallback" in pa.pa_last_error(None)
    with pytest.raises(L.PaError):
        attn.AttnEngine(attn.AttnConfig(16, 2, 256, 64, 1e7, max_seq=128))


def test_bad_config_is_rejected_before_touching_the_device(pa):
    h = C.c_void_p()
    bad = L.PaConfig(n_heads=16, n_kv_heads=3, head_dim=256, n_rot=64, rope_theta=1e7, rope_mode=1, act_dtype=1, max_cols=8)
    assert pa.pa_create(0, C.byref(bad), C.byref(h)) == -1
    bad = L.PaConfig(n_heads=16, n_kv_heads=2, head_dim=96, n_rot=64, rope_theta=1e7, rope_mode=1, act_dtype=1, max_cols=8)
    assert pa.pa_create(0, C.byref(bad), C.byref(h)) == -2 and b"head_dim 96" in pa.pa_last_error(None)
    assert pa.pa_create(0, None, C.byref(h)) == -1


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(L.PaError) as e:
        L.Lib(str(tmp_path / "libpooled_attn.so"))
    assert "no CPU or PyTorch fallback" in str(e.value)


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "pooled_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cc", ".mjs", ".js")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("pooled's CPU reference", ""), f"{f} mentions the oracle"
    assert pooled_b200.__doc__
