"""ctypes access to oracle/_ref/libt2ref.so: the reference's own CUDA kernels behind the harness
oracle/ref_driver.cu.  Test infrastructure; needs a GPU.  ``available()`` is False when the library was
not built (no reference checkout at build time) or there is no CUDA device."""
from __future__ import annotations

import ctypes
import os

import numpy as np

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_SO = os.path.join(_DIR, "libt2ref.so")
_SO_DROPIN = os.path.join(_DIR, "libt2ref_dropin.so")      # the reference's decoder code on this repository's kernels
_libs = {}
_use_dropin = False


def use_dropin(flag: bool) -> None:
    """Route the calls below through libt2ref_dropin.so (reference sdec/ops/gemm/core + the t2sc binding in place of
    the reference's spconv.cu) instead of the all-reference library."""
    global _use_dropin
    _use_dropin = bool(flag)


def available(dropin: bool = False) -> bool:
    if not os.path.exists(_SO_DROPIN if dropin else _SO):
        return False
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def lib():
    key = _use_dropin
    if key not in _libs:
        L = ctypes.CDLL(_SO_DROPIN if key else _SO)
        L.ref_last_error.restype = ctypes.c_char_p
        _libs[key] = L
    return _libs[key]


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _check(rc):
    if rc:
        raise RuntimeError("reference: " + lib().ref_last_error().decode())


def build_neighbors(coords, W=4096, H=4096, D=4096, B1=0):
    coords = np.ascontiguousarray(coords, np.int32)
    n = coords.shape[0]
    nbr, gray, srt = np.empty((n, 27), np.uint32), np.empty(n, np.int32), np.empty(n, np.int32)
    nb = (n + B1 - 1) // B1 if B1 else 0
    seg, lst, ln = np.zeros(nb + 1, np.int32), np.zeros(max(27 * nb, 1), np.int32), ctypes.c_int(0)
    _check(lib().ref_build_neighbors(_p(coords), n, W, H, D, _p(nbr), _p(gray), _p(srt), B1, _p(seg), _p(lst), ctypes.byref(ln)))
    return (nbr, gray, srt, seg, lst[:ln.value].copy()) if B1 else (nbr, gray, srt)


def subm_conv(coords, x, w, bias, reps=0):
    """fp16 arrays -> (y fp16, conv ms, build_neighbors ms)."""
    coords = np.ascontiguousarray(coords, np.int32)
    x, w = np.ascontiguousarray(x, np.float16), np.ascontiguousarray(w, np.float16)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float16)
    n, Ci, Co = x.shape[0], x.shape[1], w.shape[0]
    y = np.empty((n, Co), np.float16)
    cms, nms = ctypes.c_float(0), ctypes.c_float(0)
    _check(lib().ref_subm_conv(_p(coords), n, _p(x), _p(w), _p(bias), Ci, Co, _p(y), reps, ctypes.byref(cms), ctypes.byref(nms)))
    return y, cms.value, nms.value


def c2s(coords, sub):
    coords = np.ascontiguousarray(coords, np.int32)
    sub = np.ascontiguousarray(sub, np.float16)
    n = coords.shape[0]
    cc, src, m = np.empty((8 * n, 4), np.int32), np.empty(8 * n, np.int32), ctypes.c_int(0)
    _check(lib().ref_c2s(_p(coords), n, _p(sub), _p(cc), _p(src), ctypes.byref(m)))
    return cc[:m.value].copy(), src[:m.value].copy()


def conv_block(coords, x, w, bias, ln=None, act=0, residual=None):
    coords = np.ascontiguousarray(coords, np.int32)
    x, w = np.ascontiguousarray(x, np.float16), np.ascontiguousarray(w, np.float16)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float16)
    residual = None if residual is None else np.ascontiguousarray(residual, np.float16)
    n, Ci, Co = x.shape[0], x.shape[1], w.shape[0]
    g = b = None
    eps = 0.0
    if ln is not None:
        g = None if ln[0] is None else np.ascontiguousarray(ln[0], np.float32)
        b = None if ln[1] is None else np.ascontiguousarray(ln[1], np.float32)
        eps = ln[2]
    y = np.empty((n, Co), np.float16)
    _check(lib().ref_conv_block(_p(coords), n, _p(x), _p(w), _p(bias), Ci, Co, int(ln is not None), _p(g), _p(b),
                                ctypes.c_float(eps), act, _p(residual), _p(y)))
    return y


def up_tail(coords, x, sub, w1, b1, w2, b2):
    coords = np.ascontiguousarray(coords, np.int32)
    f = lambda a: np.ascontiguousarray(a, np.float16)
    x, sub, w1, b1, w2, b2 = map(f, (x, sub, w1, b1, w2, b2))
    n, Ci, Cc = x.shape[0], x.shape[1], w2.shape[0]
    hc, out, m = np.empty((8 * n, Cc), np.float16), np.empty((8 * n, Cc), np.float16), ctypes.c_int(0)
    _check(lib().ref_up_tail(_p(coords), n, _p(x), _p(sub), _p(w1), _p(b1), _p(w2), _p(b2), Ci, Cc, _p(hc), _p(out), ctypes.byref(m)))
    return hc[:m.value].copy(), out[:m.value].copy()
