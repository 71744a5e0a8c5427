"""ctypes binding of librwkv_b200.so (the C ABI declared in include/rwkv_b200.h).

The library is the only compute path: when it is missing this module raises, there is no
CPU or pure-torch fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librwkv_b200.so")

OK = 0
F32, F16, BF16 = 0, 1, 2
PRO_PLAIN, PRO_LN_MIX, PRO_WKV4 = 0, 1, 2
ERR_UNSUPPORTED = -5
MM8_WIDE_BUILD = 1
EPI_ACC_F32, EPI_STORE, EPI_SIGMOID, EPI_RELU_SQ, EPI_RESIDUAL, EPI_MUL_RESIDUAL, EPI_STORE_F32, EPI_SILU = range(8)


class RwkvB200Error(RuntimeError):
    pass


class Mm8Problem(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("w_stride", C.c_int64),
        ("mx", C.c_void_p), ("rx", C.c_void_p), ("my", C.c_void_p), ("ry", C.c_void_p),
        ("y", C.c_void_p), ("aux", C.c_void_p), ("aux2", C.c_void_p),
        ("N", C.c_int32), ("M", C.c_int32), ("epilogue", C.c_int32), ("out_scale", C.c_float),
        ("prologue", C.c_int32), ("mode", C.c_int32),
        ("ln_w", C.c_void_p), ("ln_b", C.c_void_p), ("sx", C.c_void_p), ("mix", C.c_void_p), ("xx_out", C.c_void_p),
        ("k", C.c_void_p), ("v", C.c_void_p), ("t_decay", C.c_void_p), ("t_first", C.c_void_p),
        ("aa", C.c_void_p), ("bb", C.c_void_p), ("pp", C.c_void_p),
        ("aa_out", C.c_void_p), ("bb_out", C.c_void_p), ("pp_out", C.c_void_p),
    ]


class Mm8Exchange(C.Structure):
    """rwkv_mm8_exchange: where a column-sharded launch also stores its results (the other ranks'
    buffers) and the arrival words it waits on and publishes."""
    _fields_ = [
        ("peer_y", (C.c_void_p * 7) * 4),
        ("arrived", C.c_void_p), ("peer_arrived", C.c_void_p * 7),
        ("done_counter", C.c_void_p), ("error", C.c_void_p), ("seq_base", C.c_void_p),
        ("wait_seq", C.c_uint32), ("signal_seq", C.c_uint32),
        ("world", C.c_int32), ("rank", C.c_int32),
    ]


PEER_HANDLE_BYTES = 64
_vp, _i64, _i32, _sz, _f = C.c_void_p, C.c_int64, C.c_int, C.c_size_t, C.c_float

# name -> (restype, argtypes); every symbol include/rwkv_b200.h declares.
SIGNATURES = {
    "rwkv_b200_version": (_i32, []),
    "rwkv_b200_error_string": (C.c_char_p, [_i32]),
    "rwkv_quantize_weight_workspace_bytes": (_sz, [_i64, _i64]),
    "rwkv_quantize_weight": (_i32, [_vp, _i32, _i64, _i64, _f, _i64, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _vp, _sz, _vp]),
    "rwkv_mm8_one_workspace_bytes": (_sz, [_i64, _i64]),
    "rwkv_mm8_one": (_i32, [_i64, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _sz, _vp]),
    "rwkv_mm8_one_static": (_i32, [_i64, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _vp, _vp]),
    "rwkv_mm8_one_batch_workspace_bytes": (_sz, [C.POINTER(Mm8Problem), _i32]),
    "rwkv_mm8_one_batch": (_i32, [C.POINTER(Mm8Problem), _i32, _i32, _vp, _sz, _vp]),
    "rwkv_mm8_one_batch_exchange": (_i32, [C.POINTER(Mm8Problem), _i32, C.POINTER(Mm8Exchange), _i32, _vp, _sz, _vp]),
    "rwkv_sample_logits": (_i32, [_i64, _vp, C.c_float, C.c_float, _i64, _vp, _vp, _vp, _vp, C.c_float, C.c_float, C.c_float,
                                  _vp, _i64, _vp, _vp, _vp, _vp]),
    "rwkv_mm8_one_set_lean": (None, [_i32]),
    "rwkv_mm8_one_take_error": (_i32, [_vp, C.POINTER(C.c_int)]),
    "rwkv_mm8_one_batch_flags": (_i32, [C.POINTER(Mm8Problem), _i32, C.POINTER(Mm8Exchange), _i32, _i32, _vp, _sz, _vp]),
    "rwkv_peer_alloc": (_i32, [_sz, C.POINTER(_vp)]),
    "rwkv_peer_free": (_i32, [_vp]),
    "rwkv_peer_export": (_i32, [_vp, _vp]),
    "rwkv_peer_open": (_i32, [_vp, C.POINTER(_vp)]),
    "rwkv_peer_close": (_i32, [_vp]),
    "rwkv_peer_wait": (_i32, [_vp, _i32, C.c_uint32, _vp, _vp, _vp]),
    "rwkv_peer_advance": (_i32, [_vp, C.c_uint32, _vp]),
    "rwkv_mm8_one_set_split": (None, [_i32]),
    "rwkv_mm8_one_set_variant": (None, [_i32]),
    "rwkv_mm8_one_set_cluster": (None, [_i32, _i32]),
    "rwkv_mm8_one_set_plan": (None, [_i64, _i32]),
    "rwkv_mm8_stream_ctas": (_i32, []),
    "rwkv_mm8_stream_set_planes": (None, [_i32]),
    "rwkv_mm8_stream_weight_bytes": (_sz, [C.POINTER(Mm8Problem), _i32, _i32]),
    "rwkv_mm8_stream_pack": (_i32, [C.POINTER(Mm8Problem), _i32, _i32, _vp, _sz, _vp]),
    "rwkv_mm8_stream_table_bytes": (_sz, [_i32]),
    "rwkv_mm8_stream_plan": (_i32, [C.POINTER(Mm8Problem), C.POINTER(C.c_int32), _i32, _i32, _i32, _vp, _sz]),
    "rwkv_mm8_stream_run": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "rwkv_mm8_stream_take_error": (_i32, [_vp, _vp, C.POINTER(C.c_int)]),
    "rwkv_mm8_seq_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "rwkv_mm8_seq_set_path": (None, [_i32]),
    "rwkv_mm8_seq_tc_take_error": (_i32, [_vp, _vp, C.POINTER(C.c_int)]),
    "rwkv_mm8_seq": (_i32, [_i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _vp, _i64, _vp, _sz, _vp]),
    "rwkv_mm8_seq_epi": (_i32, [_i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _vp, _i64, _i32, _vp, _i64, _vp, _i64,
                                _f, _vp, _sz, _vp]),
    "rwkv_wkv4_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "rwkv_wkv4_seq": (_i32, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _sz, _vp]),
    "rwkv_wkv4_forward": (_i32, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp]),
    "rwkv_wkv5_forward": (_i32, [_i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp]),
    "rwkv_wkv6_forward": (_i32, [_i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp]),
    "rwkv_wkv56_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "rwkv_wkv56_seq": (_i32, [_i32, _i64, _i64, _i64, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _vp, _sz, _vp]),
    "rwkv_v6_seq_mix": (_i32, [_i64, _i64, _vp, _i64, _vp, _i64, _vp, C.POINTER(_vp), C.POINTER(_vp), _vp]),
    "rwkv_tanh_regroup_f16": (_i32, [_i64, _i64, _i64, _vp, _vp, _vp]),
    "rwkv_v6_seq_decay": (_i32, [_i64, _i64, _vp, _vp, _vp, _vp]),
    "rwkv_v56_seq_gn_gate": (_i32, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _f, _vp]),
    "rwkv_ln_mix": (_i32, [_i64, _i64, _vp, _i64, _vp, _vp, _vp, _i32, _i32, C.POINTER(_vp), _i64, C.POINTER(_vp), _i64, _vp, _i64, _vp, _vp]),
    "rwkv_ln_mix_rows": (_i32, [_i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i32, _i32, C.POINTER(_vp), _i64, C.POINTER(_vp), _i64, _vp, _i64,
                                _vp, _vp]),
    "rwkv_embed_row": (_i32, [_i64, _i64, _vp, _i64, _vp, _vp, _vp]),
    "rwkv_wkv4_one": (_i32, [_i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "rwkv_v6_scratch_bytes": (_sz, [_i64, _i64]),
    "rwkv_v6_att_pre": (_i32, [_i64, _i64, _i64] + [_vp] * 17),
    "rwkv_v6_token_shift": (_i32, [_i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp, _vp, _vp]),
    "rwkv_v6_decay": (_i32, [_i64, _i64, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "rwkv_wkv56_one": (_i32, [_i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
}

_lib = None


def lib():
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RwkvB200Error(
                f"{LIB_PATH} not found: build it with `python -m chatrwkv_b200.build` "
                "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code, what=""):
    if code != OK:
        msg = lib().rwkv_b200_error_string(code).decode()
        raise RwkvB200Error(f"{what}: {msg} (code {code})")
