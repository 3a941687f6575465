"""ctypes binding of libt2sc.so (include/t2sc.h).  There is no fallback: if the library is missing or
cannot create a context the import / call raises."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# T2SC_LIBRARY names another build of the same sources inside this package (the diagnostic build libt2sc_diag.so, which
# the bounded-wait test loads in a process of its own); the default is the shipped library
LIB_PATH = os.path.join(HERE, os.path.basename(os.environ.get("T2SC_LIBRARY", "libt2sc.so")))

F32, F16, BF16, U8 = 0, 1, 2, 5
ACT_NONE, ACT_SILU, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2, 3
VARIANT_AUTO, VARIANT_SIMT, VARIANT_UMMA, VARIANT_UMMA_PAIR = 0, 1, 2, 3
STATIC_MAX_ROWS = 65536
PEER_SHIFT = 28
PART = {"all": 0, "interior": 1, "boundary": 2}

# every symbol include/t2sc.h declares: (name, restype, argtypes)
_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
_pp = ctypes.POINTER(ctypes.c_void_p)
_pi64 = ctypes.POINTER(ctypes.c_int64)
_pi32 = ctypes.POINTER(ctypes.c_int)


class Epilogue(ctypes.Structure):
    """Mirror of t2sc_epilogue."""
    _fields_ = [("bias", _vp), ("ln", _i32), ("ln_gamma", _vp), ("ln_beta", _vp), ("ln_eps", _f32), ("act", _i32),
                ("residual", _vp), ("skip_x", _vp), ("skip_src", _vp), ("skip_cin", _i32), ("skip_rep", _i32)]


SYMBOLS = [
    ("t2sc_ctx_create", _i32, [_i32, _vp, _pp]),
    ("t2sc_ctx_destroy", _i32, [_vp]),
    ("t2sc_ctx_sync", _i32, [_vp]),
    ("t2sc_last_error", ctypes.c_char_p, [_vp]),
    ("t2sc_launch_count", _i64, [_vp]),
    ("t2sc_device_status", _i32, [_vp, _pi32]),
    ("t2sc_build_neighbors", _i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    ("t2sc_build_neighbors_range", _i32, [_vp, _vp, _i64, _i32, _i32, _i32, _i64, _i64, _vp, _vp]),
    ("t2sc_voxel_lookup", _i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp, _i64, _vp]),
    ("t2sc_build_neighbors_static", _i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp]),
    ("t2sc_valid_taps", _i32, [_vp, _vp, _vp, _i64, _i32, _vp, _vp, _pi64]),
    ("t2sc_subdivide_count", _i32, [_vp, _vp, _i32, _i64, _vp, _pi64]),
    ("t2sc_subdivide_emit", _i32, [_vp, _vp, _i32, _vp, _vp, _i64, _vp, _vp]),
    ("t2sc_gather_rows", _i32, [_vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    ("t2sc_add_skip", _i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32]),
    ("t2sc_plan_create", _i32, [_vp, _vp, _vp, _i64, _vp, _i64, _i64, _i32, _pp]),
    ("t2sc_plan_create_split", _i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _pp]),
    ("t2sc_plan_parts", _i32, [_vp, _vp, _pi64, _pi64]),
    ("t2sc_plan_destroy", _i32, [_vp, _vp]),
    ("t2sc_plan_set_input_rows", _i32, [_vp, _vp, _i64]),
    ("t2sc_plan_check", _i32, [_vp, _vp, _i64]),
    ("t2sc_plan_stats", _i32, [_vp, _vp, _pi64, _pi64, _pi64]),
    ("t2sc_plan_order", _i32, [_vp, _vp, _vp]),
    ("t2sc_subm_conv", _i32, [_vp, _vp, _vp, _vp, ctypes.POINTER(Epilogue), _vp, _i32, _i64, _i32, _i32, _i32]),
    ("t2sc_subm_conv_part", _i32, [_vp, _vp, _vp, _vp, ctypes.POINTER(Epilogue), _vp, _i32, _i64, _i32, _i32, _i32, _i32]),
    ("t2sc_subm_conv_peers_part", _i32, [_vp, _vp, _vp, ctypes.POINTER(ctypes.c_void_p), _pi64, _i32, _i32, _vp, ctypes.POINTER(Epilogue), _vp, _i32, _i32, _i32, _i32]),
    ("t2sc_peer_barrier", _i32, [_vp, ctypes.POINTER(ctypes.c_void_p), _i32, _i32, _i32, _i32]),
    ("t2sc_subm_conv_peers", _i32, [_vp, _vp, ctypes.POINTER(ctypes.c_void_p), _pi64, _i32, _i32, _vp, ctypes.POINTER(Epilogue), _vp, _i32, _i32, _i32]),
    ("t2sc_linear", _i32, [_vp, _vp, _vp, ctypes.POINTER(Epilogue), _vp, _i32, _i64, _i32, _i32]),
    ("t2sc_row_epilogue", _i32, [_vp, _vp, ctypes.POINTER(Epilogue), _vp, _i64, _i32, _i32]),
    ("t2sc_subm_conv_host", _i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32]),
]

_lib = None


def load():
    """Loads the library and binds every declared symbol; raises if the file or a symbol is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} not found: build it with `python -m trellis2_cuda_b200.build` "
                              "(there is no CPU or PyTorch fallback for these operators)")
        L = ctypes.CDLL(LIB_PATH)
        for name, res, args in SYMBOLS:
            f = getattr(L, name)          # AttributeError if the symbol is not exported
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


class T2scError(RuntimeError):
    """A non-zero status from the C ABI; carries the library's last-error message (the reference raises
    std::runtime_error with the same kind of message, src/core.cu:10-15)."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"t2sc error {code}: {msg}")
        self.code = code
