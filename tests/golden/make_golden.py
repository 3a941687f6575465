"""Generates tests/golden/ref_small.npz by running the REFERENCE's own CUDA kernels (oracle/_ref, built by
oracle/Makefile from a checkout of suvadityamuk/trellis2-cuda) on seeded inputs.  Needs a GPU:

    make -C oracle && python tests/golden/make_golden.py [out.npz]

The CPU oracle and the CUDA library are both tested against the stored vectors, which pins them to what
the reference computes (integer maps bit for bit; fp16 features to within the tolerances in the tests).
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref  # noqa: E402
from trellis2_cuda_b200 import scenes  # noqa: E402


def random_coords(rng, n, res, batches):
    """Unique voxels in a small grid that touches its borders, several batch items, shuffled rows."""
    cells = rng.choice(batches * res ** 3, size=n, replace=False)
    b, r = np.divmod(cells, res ** 3)
    x, r = np.divmod(r, res * res)
    y, z = np.divmod(r, res)
    return np.stack([b, x, y, z], 1).astype(np.int32)


def weight(Co, Ci, seed):
    """Weights are not stored in the fixture: they are re-drawn from the seed (sha256 stored as a guard).
    Seeds: f0/f1/f2 -> 7, b0 -> 8, u0 conv1 -> 9, u0 conv2 -> 10."""
    return scenes.kaiming_uniform_weight(Co, Ci, seed).astype(np.float16)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main(out):
    rng = np.random.default_rng(2024)
    G = {}
    # --- integer maps: dense-ish random set in a 10^3 grid whose extent equals the grid (borders matter)
    c = random_coords(rng, 700, 10, 2)
    nbr, gray, srt, seg, lst = ref.build_neighbors(c, 10, 10, 10, B1=32)
    G.update(i0_coords=c, i0_nbr=nbr, i0_gray=gray, i0_sorted=srt, i0_seg=seg, i0_list=lst)
    # the decoder's calling convention: extent 4096 whatever the level
    c = random_coords(rng, 900, 14, 1)
    c[:, 1:] += 3
    nbr, gray, srt, seg, lst = ref.build_neighbors(c, 4096, 4096, 4096, B1=128)
    G.update(i1_coords=c, i1_nbr=nbr, i1_gray=gray, i1_sorted=srt, i1_seg=seg, i1_list=lst)
    # config-1 sphere shell: checksums only
    c1 = scenes.config1_sphere()
    nbr, gray, srt = ref.build_neighbors(c1)
    G.update(s1_n=np.int64(c1.shape[0]), s1_coords_sha=sha(c1), s1_nbr_sha=sha(nbr), s1_gray_sha=sha(gray), s1_sorted_sha=sha(srt),
             s1_taps=np.int64((nbr != 0xFFFFFFFF).sum()))
    # --- subdivision
    c = random_coords(rng, 300, 8, 2)
    sub = rng.standard_normal((300, 8)).astype(np.float16)
    sub[5] = 0.0            # logit exactly 0 is dropped
    sub[6] = -0.0
    cc, src = ref.c2s(c, sub)
    G.update(c2s_coords=c, c2s_sub=sub, c2s_child=cc, c2s_src=src)
    # --- convs (fp16)
    c = random_coords(rng, 640, 9, 1)
    for tag, Ci, Co, use_b in (("f0", 64, 64, True), ("f1", 64, 96, False), ("f2", 128, 256, True)):
        x = rng.standard_normal((c.shape[0], Ci)).astype(np.float16)
        w = weight(Co, Ci, 7)
        b = (0.1 * rng.standard_normal(Co)).astype(np.float16) if use_b else None
        y, _, _ = ref.subm_conv(c, x, w, b)
        G.update({f"{tag}_coords": c, f"{tag}_x": x, f"{tag}_w_sha": sha(w), f"{tag}_y": y})
        if use_b:
            G[f"{tag}_b"] = b
    # --- conv -> LN(affine) -> GELU -> + residual, and conv -> LN(no affine) -> SiLU
    Ci = Co = 64
    x = rng.standard_normal((c.shape[0], Ci)).astype(np.float16)
    w = weight(Co, Ci, 8)
    b = (0.1 * rng.standard_normal(Co)).astype(np.float16)
    g = (1.0 + 0.1 * rng.standard_normal(Co)).astype(np.float32)
    be = (0.1 * rng.standard_normal(Co)).astype(np.float32)
    y0 = ref.conv_block(c, x, w, b, ln=(g, be, 1e-6), act=3, residual=x)
    y1 = ref.conv_block(c, x, w, b, ln=(None, None, 1e-6), act=1, residual=None)
    G.update(b0_coords=c, b0_x=x, b0_w_sha=sha(w), b0_b=b, b0_g=g, b0_be=be, b0_y_ln_gelu_res=y0, b0_y_ln_silu=y1)
    # --- tail of the up block: conv1 -> c2s -> gather -> LN -> SiLU -> conv2 -> skip
    c = random_coords(rng, 400, 8, 1)
    Ci, Cc = 128, 64
    x = rng.standard_normal((c.shape[0], Ci)).astype(np.float16)
    sub = rng.standard_normal((c.shape[0], 8)).astype(np.float16)
    w1 = weight(8 * Cc, Ci, 9)
    b1 = (0.1 * rng.standard_normal(8 * Cc)).astype(np.float16)
    w2 = weight(Cc, Cc, 10)
    b2 = (0.1 * rng.standard_normal(Cc)).astype(np.float16)
    hc, o = ref.up_tail(c, x, sub, w1, b1, w2, b2)
    G.update(u0_coords=c, u0_x=x, u0_sub=sub, u0_w1_sha=sha(w1), u0_b1=b1, u0_w2_sha=sha(w2), u0_b2=b2, u0_hc=hc, u0_out=o)
    np.savez_compressed(out, **G)
    print("wrote", out, os.path.getsize(out), "bytes;", len(G), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_small.npz"))
