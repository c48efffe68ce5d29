"""ctypes binding of libmbema.so (the C ABI declared in include/mbema.h).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmbema.so")

F32, BF16 = 0, 1
FLAG_SILU, FLAG_LISTED_ONLY, FLAG_CBASE_EXTRA_DECAY, FLAG_FP32_BACKWARD, FLAG_INDEX_READY = 1, 2, 4, 8, 16
FLAG_TEST_WITHHOLD_ARRIVE = 1 << 30
MODE_FP32, MODE_TC_BF16 = 0, 1
TILE_T = 128

_i64, _i32, _vp, _sz, _f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float

# name -> (restype, argtypes); kept in the order of include/mbema.h
SIGNATURES = {
    "mbema_version": (_i32, []),
    "mbema_strerror": (ctypes.c_char_p, [_i32]),
    "mbema_last_cuda_error": (ctypes.c_char_p, []),
    "mbema_query_scan_workspace_bytes": (_sz, [_i64, _i64]),
    "mbema_query_scan": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "mbema_query_scan_static": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "mbema_tile_states_workspace_bytes": (_sz, [_i64, _i64]),
    "mbema_tile_states": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp, _sz, _vp]),
    "mbema_qgate_fwd": (_i32, [_vp, _i32, _vp, _i32, _vp, _vp, _vp, _f32, _vp, _i32, _vp, _vp, _i64, _i64, _i32, _vp]),
    "mbema_qgate_bwd_workspace_bytes": (_sz, [_i64, _i64]),
    "mbema_qgate_bwd": (_i32, [_vp, _i32, _vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                               _i64, _i64, _i32, _vp, _sz, _vp]),
    "mbema_flash_tc_supported": (_i32, [_i64, _i64, _i64]),
    "mbema_flash_fwd_workspace_bytes": (_sz, [_i64] * 6 + [_i32]),
    "mbema_flash_fwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                               _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _vp, _sz, _vp]),
    "mbema_flash_bwd_workspace_bytes": (_sz, [_i64] * 6 + [_i32]),
    "mbema_flash_bwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32,
                               _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _vp, _sz, _vp]),
    "mbema_flash_fwd_rows": (_i32, [_vp, _i32, _vp, _vp, _vp, _i32, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                    _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _vp, _sz, _vp]),
    "mbema_flash_bwd_rows": (_i32, [_vp, _i32, _vp, _vp, _vp, _i32, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                    _vp, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32,
                                    _vp, _sz, _vp]),
    "mbema_decode_attend": (_i32, [_vp, _i32, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                   _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _vp]),
    "mbema_decode_attend_tc_workspace_bytes": (_sz, [_i64] * 3),
    "mbema_decode_attend_tc": (_i32, [_vp, _i32, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                      _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _vp, _sz, _vp]),
    "mbema_decode_update": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp]),
    "mbema_decode_advance": (_i32, [_vp, _vp]),
    "mbema_slot_ln_fwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _f32, _vp, _i32, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mbema_slot_ln_bwd": (_i32, [_vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mbema_slot_state_gather": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "mbema_ce_rows": (_i32, [_vp, _i32, _vp, _f32, _vp, _i64, _i64, _i64, _vp]),
    "mbema_slot_grad_scatter": (_i32, [_vp, _vp, _i32, _vp, _vp, _i64, _i64, _i64, _vp]),
}

_lib = None


class MbemaError(RuntimeError):
    pass


def load():
    """Load libmbema.so once; raises if it has not been built (python -m mathbrain_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MbemaError("libmbema.so not found at %s: build it with `python -m mathbrain_b200.build` "
                             "(there is no fallback implementation)" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc, what):
    if rc != 0:
        lib = load()
        msg = lib.mbema_strerror(rc).decode()
        if rc == 5:
            msg += ": " + lib.mbema_last_cuda_error().decode()
        raise MbemaError("%s failed: %s (code %d)" % (what, msg, rc))
