"""CPU oracle (test infrastructure).  Only tests/, the repository's smoke check and the benchmark's
cpu_baseline / reference legs may import this package; the shipped library never does.

Thin ctypes wrapper over ``oracle.c`` plus the storage-dtype rounding the reference applies between
kernels (fp32 -> fp16 / bf16 round-to-nearest-even via torch on CPU).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")
_lib = None

EMPTY = 0xFFFFFFFF
ACT = {"none": 0, None: 0, "silu": 1, "gelu_tanh": 2, "gelu": 3, "gelu_erf": 3}


def build(force: bool = False) -> str:
    """gcc -O3 -fopenmp oracle.c -> liboracle.so (scalar code: no intrinsics, no fast-math)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-ffp-contract=off", "-o", _SO, src, "-lm"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(build())
        i64, i32, f32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p
        L.orc_build_neighbors.argtypes = [vp, i64, i32, i32, i32, vp, vp, vp, vp]
        L.orc_build_neighbors.restype = i32
        L.orc_valid_taps.argtypes = [vp, vp, i64, i32, vp, vp]
        L.orc_valid_taps.restype = i64
        for f in (L.orc_subm_conv_f32, L.orc_subm_conv_f64):
            f.argtypes = [vp, vp, vp, vp, vp, vp, i64, i32, i32, vp]
            f.restype = None
        L.orc_c2s_count.argtypes = [vp, i64, vp]
        L.orc_c2s_count.restype = i64
        L.orc_c2s_emit.argtypes = [vp, vp, vp, i64, vp, vp]
        L.orc_gather_rows.argtypes = [vp, vp, i64, i32, vp]
        L.orc_add_skip.argtypes = [vp, vp, vp, i64, i32, i32, i32]
        L.orc_layer_norm.argtypes = [vp, vp, vp, f32, i64, i32, vp]
        L.orc_act.argtypes = [vp, i64, i32, vp]
        L.orc_add.argtypes = [vp, vp, i64, vp]
        L.orc_num_threads.restype = i32
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_threads(n: int) -> None:
    """OpenMP thread count for the timed baselines (1 = the scalar baseline)."""
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        omp = ctypes.CDLL("libgomp.so.1")
        omp.omp_set_num_threads(int(n))
    except OSError:
        pass


# ------------------------------------------------------------------------------------ integer path
def build_neighbors(coords, W=4096, H=4096, D=4096, want_sorted=True):
    """-> (nbr uint32 [N,27], gray int32 [N], bin int32 [N], sorted int32 [N] or None)."""
    coords = _c(coords, np.int32)
    n = coords.shape[0]
    nbr = np.empty((n, 27), np.uint32)
    gray = np.empty(n, np.int32)
    bin_ = np.empty(n, np.int32)
    srt = np.empty(n, np.int32) if want_sorted else None
    rc = lib().orc_build_neighbors(_p(coords), n, W, H, D, _p(nbr), _p(gray), _p(bin_), _p(srt))
    if rc:
        raise MemoryError("orc_build_neighbors")
    return nbr, gray, bin_, srt


def valid_taps(gray, srt, B1):
    n = gray.shape[0]
    nb = (n + B1 - 1) // B1
    seg = np.zeros(nb + 1, np.int32)
    lst = np.zeros(max(27 * nb, 1), np.int32)
    tot = lib().orc_valid_taps(_p(_c(gray, np.int32)), _p(_c(srt, np.int32)), n, B1, _p(seg), _p(lst))
    return lst[:tot].copy(), seg


def subdivide(coords, keep):
    """keep: bool/uint8 [n,8] -> (child coords int32 [m,4], src int32 [m])."""
    coords = _c(coords, np.int32)
    keep = _c(np.asarray(keep) != 0, np.uint8)
    n = coords.shape[0]
    off = np.zeros(n + 1, np.int32)
    m = lib().orc_c2s_count(_p(keep), n, _p(off))
    nco = np.empty((m, 4), np.int32)
    src = np.empty(m, np.int32)
    lib().orc_c2s_emit(_p(keep), _p(coords), _p(off), n, _p(nco), _p(src))
    return nco, src


# ------------------------------------------------------------------------------------ float path
def subm_conv(x, w, bias, nbr, nrow=None, wsel=None, Co=None, f64=False):
    """x float32 [Nin,Ci]; w float32 [Wrows,27,Ci]; nbr uint32 [*,27]; -> float32 (or float64) [n_out,Co].
    n_out = len(nrow) if given else nbr.shape[0]; Co defaults to w.shape[0]."""
    x, w, bias = _c(x, np.float32), _c(w, np.float32), _c(bias, np.float32)
    nbr = _c(nbr, np.uint32)
    nrow, wsel = _c(nrow, np.int32), _c(wsel, np.int32)
    n_out = nrow.shape[0] if nrow is not None else nbr.shape[0]
    Ci = x.shape[1]
    Co = w.shape[0] if Co is None else Co
    assert w.shape[1] == 27 and w.shape[2] == Ci
    y = np.empty((n_out, Co), np.float64 if f64 else np.float32)
    f = lib().orc_subm_conv_f64 if f64 else lib().orc_subm_conv_f32
    f(_p(x), _p(w), _p(bias), _p(nbr), _p(nrow), _p(wsel), n_out, Ci, Co, _p(y))
    return y


def gather_rows(x, src, C):
    x = _c(x, np.float32)
    src = _c(src, np.int32)
    y = np.empty((src.shape[0], C), np.float32)
    lib().orc_gather_rows(_p(x), _p(src), src.shape[0], C, _p(y))
    return y


def add_skip(h, x, src, rep):
    h = _c(h, np.float32).copy()
    x = _c(x, np.float32)
    src = _c(src, np.int32)
    lib().orc_add_skip(_p(h), _p(x), _p(src), h.shape[0], h.shape[1], x.shape[1], rep)
    return h


def layer_norm(x, g, b, eps):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    lib().orc_layer_norm(_p(x), _p(_c(g, np.float32)), _p(_c(b, np.float32)), eps, x.shape[0], x.shape[1], _p(y))
    return y


def act(x, kind):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    lib().orc_act(_p(x), x.size, ACT[kind], _p(y))
    return y


def add(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    y = np.empty_like(a)
    lib().orc_add(_p(a), _p(b), a.size, _p(y))
    return y


# ------------------------------------------------------------------------------------ storage rounding
def round_to(a: np.ndarray, dtype: str) -> np.ndarray:
    """Round float32 values to the storage dtype ("f32" | "f16" | "bf16") and widen back to float32."""
    a = np.asarray(a, dtype=np.float32)
    if dtype == "f32":
        return a
    if dtype == "f16":
        return a.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        u = a.view(np.uint32).astype(np.uint64)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16          # round to nearest even on the top 16 bits
        out = r.astype(np.uint32).view(np.float32).reshape(a.shape)
        return np.where(np.isnan(a), a, out)
    raise ValueError(dtype)


def conv_block(x, w, bias, nbr, dtype, ln=None, act_kind=None, residual=None, nrow=None, wsel=None, Co=None,
               skip=None):
    """The unfused reference chain with its rounding points, as one call:
    conv (fp32 accumulate) -> round -> (+bias in storage dtype, rounded; src/spconv.cu:141-143)
    -> LN in fp32, rounded (src/ops.cu:73-76) -> act, rounded -> + residual in fp32, rounded (src/ops.cu:105-113).
    ln = (gamma or None, beta or None, eps); skip = (x_parent, src, rep) for the up block's add (src/sdec.cu:39-43).
    Inputs are float32 arrays already holding storage-representable values."""
    y = subm_conv(x, w, None, nbr, nrow=nrow, wsel=wsel, Co=Co)
    y = round_to(y, dtype)
    if bias is not None:
        b = np.asarray(bias, np.float32)
        if wsel is not None:
            Co_ = y.shape[1]
            b = b[np.asarray(wsel)[:, None] + np.arange(Co_)[None, :]]
        y = round_to(y + round_to(b, dtype), dtype)
    if ln is not None:
        y = round_to(layer_norm(y, ln[0], ln[1], ln[2]), dtype)
    if act_kind not in (None, "none"):
        y = round_to(act(y, act_kind), dtype)
    if residual is not None:
        y = round_to(add(y, residual), dtype)
    if skip is not None:
        y = round_to(add_skip(y, skip[0], skip[1], skip[2]), dtype)
    return y
