"""CPU checks of the drop-in boundary: the library is built in-tree, loads, and exports exactly the
symbols include/t2sc.h declares; without a GPU every entry refuses loudly instead of falling back."""
import ctypes
import os
import re

import pytest
import torch

from trellis2_cuda_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "t2sc.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(t2sc_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    build.build_library()
    L = _lib.load()
    names = declared()
    assert len(names) >= 18
    assert names == sorted(n for n, _, _ in _lib.SYMBOLS)
    for n in names:
        assert getattr(L, n) is not None


def test_epilogue_struct_layout_matches_header():
    # pointer, int, pointer, pointer, float, int, 3 pointers, 2 ints with natural alignment
    assert ctypes.sizeof(_lib.Epilogue) == 72
    assert _lib.Epilogue.ln_eps.offset == 32 and _lib.Epilogue.residual.offset == 40 and _lib.Epilogue.skip_cin.offset == 64


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_gpu_means_error_not_fallback():
    L = _lib.load()
    h = ctypes.c_void_p()
    rc = L.t2sc_ctx_create(0, None, ctypes.byref(h))
    assert rc != 0 and not h.value
    assert b"no CUDA device" in L.t2sc_last_error(None)
    import trellis2_cuda_b200 as sp
    with pytest.raises(RuntimeError, match="no CPU path"):
        sp.context()
