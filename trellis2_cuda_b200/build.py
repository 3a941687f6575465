"""Builds libt2sc.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m trellis2_cuda_b200.build [--force] [--verbose] [--diag]

Cross-compiles without a GPU.  Object files go to trellis2_cuda_b200/build/, the library next to this
file; both are git-ignored.  ``--diag`` builds libt2sc_diag.so instead: the same sources with -DT2SC_DIAG, which adds
the measurement switches, per-role wait timers and the settable wait limit that the shipped library does not contain
(loaded by setting T2SC_LIBRARY=libt2sc_diag.so; used by the bounded-wait test and for kernel studies).
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libt2sc.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
         "-Xcompiler", "-fPIC"]


def _deps_mtime() -> float:
    files = glob.glob(os.path.join(CSRC, "*")) + [os.path.join(HERE, "..", "include", "t2sc.h")]
    return max(os.path.getmtime(f) for f in files)


def build_library(force: bool = False, verbose: bool = False, diag: bool = False) -> str:
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    lib = os.path.join(HERE, "libt2sc_diag.so") if diag else LIB
    objdir = os.path.join(OBJ, "diag") if diag else OBJ
    if not force and os.path.exists(lib) and os.path.getmtime(lib) >= _deps_mtime():
        return lib
    os.makedirs(objdir, exist_ok=True)
    extra = (["-Xptxas", "-v"] if verbose else []) + (["-DT2SC_DIAG"] if diag else [])
    extra += os.environ.get("T2SC_NVCC_FLAGS", "").split()          # experiments, e.g. -DT2SC_IDX_BATCH=2

    def cc(src):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        r = subprocess.run([NVCC, *FLAGS, *extra, "-c", src, "-o", obj], capture_output=True, text=True)
        return src, obj, r

    objs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        for src, obj, r in ex.map(cc, srcs):
            if verbose or r.returncode:
                sys.stderr.write(f"--- {os.path.basename(src)}\n{r.stdout}{r.stderr}")
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
            objs.append(obj)
    subprocess.check_call([NVCC, "-shared", "-o", lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    return lib


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv, diag="--diag" in sys.argv))
