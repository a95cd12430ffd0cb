"""ctypes binding of libpooled_attn.so (include/pooled_attn.h).  Fails loudly when the library is missing."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "libpooled_attn.so")

PA_F32, PA_F16 = 0, 1
PA_ROPE_NONE, PA_ROPE_F64, PA_ROPE_TABLE = 0, 1, 2
PA_KV_F16, PA_KV_Q8, PA_KV_F32 = 0, 1, 2
PA_FLAG_FAST = 1
PA_MODE_AUTO, PA_MODE_DECODE, PA_MODE_PREFILL = 0, 1, 2
STATUS = {0: "PA_OK", -1: "PA_EINVAL", -2: "PA_EUNSUPPORTED", -3: "PA_ENOMEM", -4: "PA_ECUDA", -5: "PA_ETIMEOUT", -6: "PA_ESTATE"}


class PaError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{STATUS.get(code, code)}: {msg}")
        self.code = code


class PaConfig(C.Structure):
    _fields_ = [("n_heads", C.c_uint32), ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("n_rot", C.c_uint32),
                ("rope_theta", C.c_double), ("rope_mode", C.c_uint32), ("act_dtype", C.c_uint32), ("max_cols", C.c_uint32),
                ("splits", C.c_uint32), ("flags", C.c_uint32), ("reserved", C.c_uint32 * 5)]


class PaItem(C.Structure):
    _fields_ = [("seq", C.c_uint32), ("pos", C.c_uint32), ("n_cols", C.c_uint32), ("reserved", C.c_uint32)]


class PaStats(C.Structure):
    _fields_ = [("kernel_launches", C.c_uint64), ("kv_bytes_streamed", C.c_uint64), ("calls", C.c_uint64)]


# name -> (restype, argtypes): every symbol include/pooled_attn.h declares
_vp, _u32, _u64, _i, _sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_size_t
SYMBOLS = {
    "pa_create": (_i, [_i, C.POINTER(PaConfig), C.POINTER(_vp)]),
    "pa_destroy": (_i, [_vp]),
    "pa_layer_create": (_i, [_vp, _u32, _u32, C.POINTER(_vp)]),
    "pa_layer_create_fmt": (_i, [_vp, _u32, _u32, _i, C.POINTER(_vp)]),
    "pa_layer_destroy": (_i, [_vp]),
    "pa_layer_set_origin": (_i, [_vp, _u32]),
    "pa_layer_set_next": (_i, [_vp, _vp]),
    "pa_cache_ptr": (_vp, [_vp, _i]),
    "pa_cache_export": (_i, [_vp, _u32, _u32, _u32, _i, _vp, C.POINTER(_u32), _vp]),
    "pa_cache_import": (_i, [_vp, _u32, _u32, _u32, _i, _vp, C.POINTER(_u32), _vp]),
    "pa_slot_save": (_i, [_vp, _u32, _u32, C.POINTER(_vp), _vp]),
    "pa_slot_load": (_i, [_vp, _u32, _vp, C.POINTER(_u32), _vp]),
    "pa_slot_export": (_i, [_vp, _i, _vp, _vp]),
    "pa_slot_info": (_i, [_vp, C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32)]),
    "pa_slot_drop": (_i, [_vp]),
    "pa_last_error": (C.c_char_p, [_vp]),
    "pa_version": (C.c_char_p, []),
    "pa_sync": (_i, [_vp, _vp]),
    "pa_reset": (_i, [_vp]),
    "pa_alloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "pa_free": (_i, [_vp, _vp]),
    "pa_alloc_host": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "pa_free_host": (_i, [_vp, _vp]),
    "pa_upload": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "pa_download": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "pa_dec_config": (_u32, [_u32, _u32, _u32, _u32]),
    "pa_dec_split_len": (_u32, [_u32, _u32]),
    "pa_dec_splits": (_u32, [_u32, _u32]),
    "pa_tile_split_len": (_u32, [_u32, _u32, _u32, _u32]),
    "pa_plan_splits": (_u32, [_vp, _u32, _u32]),
    "pa_rope": (_i, [_vp, _vp, _u64, _u64, _u32, _u32, _u32, _vp, _vp, _u64, _vp]),
    "pa_kv_append": (_i, [_vp, _u32, _u32, _u32, _vp, _vp, _u64, _i, _vp]),
    "pa_rope_append": (_i, [_vp, _u32, _u32, _u32, _vp, _u64, _u64, _vp, _vp, _u64, _vp, _vp, _vp]),
    "pa_rope_append_items": (_i, [_vp, _vp, _u32, _vp, _u64, _u64, _vp, _vp, _u64, _vp, _vp]),
    "pa_decode": (_i, [_vp, C.POINTER(PaItem), _u32, _vp, _i, _u64, _u64, _vp, _u64, _u64, _vp, _u64, _vp]),
    "pa_decode_gather": (_i, [_vp, _u32, _u32, _vp, _u32, _vp, _i, _u64, _u64, _vp, _u64, _u64, _vp, _u64, _vp]),
    "pa_decode_partial": (_i, [_vp, C.POINTER(PaItem), _u32, _vp, _i, _u64, _u64, _vp, _vp]),
    "pa_merge": (_i, [_vp, _vp, _u32, _u32, _vp, _u64, _u64, _vp, _u64, _vp]),
    "pa_exchange_bytes": (_sz, [_vp, _u32, _u32]),
    "pa_shared_alloc": (_i, [_vp, _sz, C.POINTER(_vp), _vp]),
    "pa_shared_open": (_i, [_vp, _vp, C.POINTER(_vp)]),
    "pa_shared_close": (_i, [_vp, _vp]),
    "pa_exchange_init": (_i, [_vp, _u32, _u32, C.POINTER(_vp), _u32]),
    "pa_decode_exchange": (_i, [_vp, C.POINTER(PaItem), _u32, _vp, _i, _u64, _u64, _vp, _u64, _u64, _vp, _u64, _vp]),
    "pa_attn_items": (_i, [_vp, _vp, _u32, _vp, _u64, _u64, _vp, _vp, _u64, _vp, _u64, _u64, _vp, _u64, C.c_int, _vp]),
    "pa_attn_layer_sharded": (_i, [_vp, _u32, _u32, _u32, _vp, _u64, _u64, _vp, _vp, _u64, _vp, _u64, _u64, _vp, _vp, _u64, _vp]),
    "pa_prefill": (_i, [_vp, _u32, _u32, _u32, _vp, _i, _u64, _u64, _vp, _u64, _u64, _vp, _u64, _vp]),
    "pa_sigmoid_mul": (_i, [_vp, _vp, _u64, _vp, _u64, _u64, _u32, _vp]),
    "pa_layer_set_head_norm": (_i, [_vp, _vp, _vp, C.c_double]),
    "pa_head_norm": (_i, [_vp, _vp, _u64, _u64, _u32, _u32, _vp, C.c_double, _vp, _u64, _u64, _vp]),
    "pa_attn_layer": (_i, [_vp, _u32, _u32, _u32, _i, _vp, _u64, _u64, _vp, _vp, _u64, _vp, _u64, _u64, _vp, _vp, _u64, _vp]),
    "pa_attn_layer_host": (_i, [_vp, _u32, _u32, _u32, _i, _vp, _u64, _u64, _vp, _vp, _u64, _vp, _u64, _u64, _vp, _vp, _u64, _vp]),
    "pa_attn_step_host": (_i, [C.POINTER(_vp), _u32, _u32, _u32, _u32, _i, _vp, _u64, _u64, _u64, _vp, _vp, _u64, _u64, _vp, _u64, _u64, _u64, _vp, _u64, _u64, _vp]),
    "pa_decode_static": (_i, [_i, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, C.c_char_p, _sz]),
    "pa_decode_static_status": (_i, [_i, _vp, C.POINTER(_u32)]),
    "pa_set_wait_limit": (_i, [_vp, _u32]),
    "pa_get_stats": (_i, [_vp, C.POINTER(PaStats)]),
    "pa_timing_begin": (_i, [_vp, _u32]),
    "pa_set_core_only": (_i, [_vp, _i]),
    "pa_timing_end": (_i, [_vp, C.POINTER(C.c_double), C.POINTER(_u64)]),
}


class Lib:
    """The loaded shared library with typed entry points."""

    def __init__(self, path: str = SO_PATH):
        if not os.path.exists(path):
            raise PaError(-4, f"{path} is missing: build it with `python -m pooled_b200.build` (nvcc, sm_100a). "
                              "There is no CPU or PyTorch fallback for the attention path.")
        self.path = path
        self.dll = C.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(self.dll, name)   # AttributeError when the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
            setattr(self, name, fn)

    def check(self, rc: int, ctx=None):
        if rc != 0:
            msg = self.pa_last_error(ctx)
            raise PaError(rc, msg.decode() if msg else "")


_lib: Lib | None = None


def load() -> Lib:
    global _lib
    if _lib is None:
        _lib = Lib()
    return _lib
