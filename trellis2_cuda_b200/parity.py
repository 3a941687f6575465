"""`parity spconv` for this library: checks single sparse convs against dumped reference outputs.

    python -m trellis2_cuda_b200.parity spconv --ref <dir|spconv.safetensors> --ckpt <decoder.safetensors> [--strict]

Mirrors the `spconv` command of the reference's parity harness (apps/parity.cu:148-167 of trellis2-cuda): the dump
written by its tools/ref_spconv.py holds, per conv j, the keys ``conv{j}/in`` [N,Ci], ``conv{j}/out`` [N,Co],
``conv{j}/coords`` int32 [N,4] and ``conv{j}/name`` (the module name as uint8 bytes, tools/ref_spconv.py:19-20); the
checkpoint holds ``<name>.weight`` [Co,3,3,3,Ci] and ``<name>.bias`` [Co].  Every entry becomes one host-buffer call of
the operator (t2sc_subm_conv_host: copy in, neighbour map over a 4096^3 grid, conv, copy out) and one line in the
harness's `cmp` format (apps/parity.cu:10-24): elements, mismatching elements, max-abs, mean-abs, reference max, then
the shape / schedule / time line.

The reference compares bit for bit (its kernel reproduces FlexGEMM's summation order).  This library accumulates the
same products in fp32 in tap-then-channel order on tensor cores, so the default verdict is the tolerance of the path's
specification - max-abs <= 2e-2 and mean-rel <= 2e-3 - and ``--strict`` asks for zero mismatching elements.
Returns the number of failed entries (0 = PARITY OK).
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys
import time
from typing import Dict

import numpy as np
import torch

_ST_DTYPES = {"F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2), "I32": (torch.int32, 4),
              "I64": (torch.int64, 8), "U8": (torch.uint8, 1), "I8": (torch.int8, 1), "F64": (torch.float64, 8)}
_ST_NAMES = {v[0]: k for k, v in _ST_DTYPES.items()}
MAX_ABS, MEAN_REL = 2e-2, 2e-3


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """The safetensors container as the reference reads it (src/core.cu:93-150): u64 little-endian header length, a JSON
    header {name: {dtype, shape, data_offsets}}, then the raw little-endian tensor bytes.  Returns host tensors."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        blob = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt, es = _ST_DTYPES[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        n = int(np.prod(meta["shape"])) if meta["shape"] else 1
        if hi - lo != n * es:
            raise ValueError(f"{path}: tensor {name} has {hi - lo} bytes for shape {meta['shape']} {meta['dtype']}")
        t = torch.frombuffer(bytearray(blob[lo:hi]), dtype=dt) if n else torch.empty(0, dtype=dt)
        out[name] = t.reshape(meta["shape"])
    return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Writes host tensors in the same container (what tools/ref_spconv.py produces through safetensors.torch.save_file)."""
    header, chunks, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        chunks.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for c in chunks:
            f.write(c)


def cmp_line(name: str, a: torch.Tensor, ref: torch.Tensor):
    """One line in the format of the reference's `cmp` (apps/parity.cu:10-24) -> (text, mismatches, max-abs, mean-rel)."""
    if a.numel() != ref.numel():
        return f"{name:<48s} numel {a.numel()} vs ref {ref.numel()}  MISMATCH", max(a.numel(), ref.numel()), float("inf"), float("inf")
    x, y = a.float().flatten(), ref.float().flatten()
    same_dt = a.dtype == ref.dtype
    nbad = int((a.flatten().view(torch.uint8).reshape(a.numel(), -1) != ref.flatten().view(torch.uint8).reshape(ref.numel(), -1)).any(1).sum()) if same_dt \
        else int((x != y).sum())
    d = (x - y).abs()
    mx, sa, ms = float(d.max()) if d.numel() else 0.0, float(d.sum()), float(y.abs().max()) if y.numel() else 0.0
    text = (f"{name:<48s} {a.numel():10d} elems  mismatch {nbad:10d}  maxabs {mx:.3g}  meanabs {sa / max(1, a.numel()):.3g} (ref max {ms:.3g})"
            + ("" if same_dt else "  [dtype differs]"))
    return text, nbad, mx, sa / max(float(y.abs().sum()), 1e-30)


def parity_spconv(ref_path: str, ckpt_path: str, strict: bool = False, device=None, out=sys.stdout) -> int:
    import trellis2_cuda_b200 as sp
    if os.path.isdir(ref_path):
        ref_path = os.path.join(ref_path, "spconv.safetensors")
    S, W = read_safetensors(ref_path), read_safetensors(ckpt_path)
    fails, j = 0, 0
    while f"conv{j}/in" in S:
        p = f"conv{j}/"
        name = bytes(S[p + "name"].tolist()).decode()
        x, want, coords = S[p + "in"].contiguous(), S[p + "out"], S[p + "coords"].to(torch.int32).contiguous()
        w, b = W[name + ".weight"], W.get(name + ".bias")
        w = w.reshape(w.shape[0], 27, w.shape[-1]).to(x.dtype).contiguous()          # [Co,3,3,3,Ci] viewed as [Co,27,Ci] (src/sdec.cu:15-18)
        sp.subm_conv_host(coords, x, w, b, 4096, 4096, 4096, device=device)          # warm-up: the harness times a warm process
        t0 = time.perf_counter()
        y = sp.subm_conv_host(coords, x, w, b, 4096, 4096, 4096, device=device)      # synchronises before it returns
        ms = (time.perf_counter() - t0) * 1e3
        text, nbad, mx, mr = cmp_line(p + name, y, want)
        ok = nbad == 0 if strict else (mx <= MAX_ABS and mr <= MEAN_REL)
        print(text + ("" if strict else f"  meanrel {mr:.3g} {'within' if ok else 'OUTSIDE'} tolerance"), file=out)
        cfg = sp.spconv_cfg(x.shape[0], x.shape[1], w.shape[0])
        print(f"  N={x.shape[0]} Ci={x.shape[1]} Co={w.shape[0]} B1={cfg.B1} BK={cfg.BK} S={cfg.S}  {ms:.2f} ms", file=out)
        fails += 0 if ok else 1
        j += 1
    print(f"PARITY FAIL ({fails})" if fails else "PARITY OK", file=out)
    return fails


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m trellis2_cuda_b200.parity")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("spconv", help="single sparse convs against a dump of tools/ref_spconv.py")
    s.add_argument("--ref", required=True, help="spconv.safetensors or the directory that holds it")
    s.add_argument("--ckpt", required=True, help="decoder checkpoint (.safetensors) with <name>.weight / <name>.bias")
    s.add_argument("--strict", action="store_true", help="require bit equality, as the reference's harness does")
    a = ap.parse_args(argv)
    return parity_spconv(a.ref, a.ckpt, a.strict)


if __name__ == "__main__":
    sys.exit(main())
