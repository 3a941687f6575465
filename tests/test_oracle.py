"""CPU tests of the oracle itself: against independent formulations (dense conv3d, dictionary search,
float64 per-tap matmul), against the golden vectors produced by the reference's own CUDA kernels, and of
the scene generators."""
import hashlib
import os

import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

import oracle
from trellis2_cuda_b200 import scenes


def brute_neighbors(coords, W, H, D):
    table = {}
    for i, q in enumerate(map(tuple, coords)):
        table.setdefault(q, i)
    nbr = np.full((len(coords), 27), 0xFFFFFFFF, np.uint32)
    for i, (b, x, y, z) in enumerate(coords):
        for v in range(27):
            p = (x + v // 9 - 1, y + v // 3 % 3 - 1, z + v % 3 - 1)
            if 0 <= p[0] < W and 0 <= p[1] < H and 0 <= p[2] < D and (b, *p) in table:
                nbr[i, v] = table[(b, *p)]
    return nbr


@settings(max_examples=40, deadline=None)
@given(st.integers(0, 2**31 - 1), st.integers(1, 120), st.integers(2, 6), st.integers(1, 3))
def test_neighbors_match_dictionary_search(seed, n, res, batches):
    rng = np.random.default_rng(seed)
    n = min(n, batches * res ** 3)
    cells = rng.choice(batches * res ** 3, size=n, replace=False)
    b, r = np.divmod(cells, res ** 3); x, r = np.divmod(r, res * res); y, z = np.divmod(r, res)
    c = np.stack([b, x, y, z], 1).astype(np.int32)
    nbr, gray, bin_, srt = oracle.build_neighbors(c, res, res, res)
    assert np.array_equal(nbr, brute_neighbors(c, res, res, res))
    assert np.array_equal(nbr[:, 13], np.arange(n))                      # the centre tap is the row itself
    g = ((nbr != 0xFFFFFFFF) << np.arange(27)).sum(1)
    assert np.array_equal(gray, g.astype(np.int32))
    b2 = g.copy()
    for v in range(1, 27):
        b2 ^= g >> v
    assert np.array_equal(bin_, b2.astype(np.int32))
    assert np.array_equal(srt, np.argsort(bin_, kind="stable"))
    for B1 in (4, 32):
        lst, seg = oracle.valid_taps(gray, srt, B1)
        for blk in range(len(seg) - 1):
            o = np.bitwise_or.reduce(gray[srt[blk * B1:(blk + 1) * B1]])
            assert list(lst[seg[blk]:seg[blk + 1]]) == [v for v in range(27) if o >> v & 1]


def test_duplicates_resolve_to_lowest_row():
    c = np.array([[0, 1, 1, 1], [0, 1, 1, 2], [0, 1, 1, 1]], np.int32)
    nbr = oracle.build_neighbors(c, 4, 4, 4)[0]
    assert nbr[2, 13] == 0 and nbr[1, 12] == 0


def test_full_grid_equals_dense_conv3d():
    """A submanifold conv on a fully occupied grid is the dense cross-correlation with zero padding 1 that
    the reference's conv() computes through cuDNN (src/conv.cu:30-83 of trellis2-cuda)."""
    R, Ci, Co = 6, 32, 16
    g = np.stack(np.meshgrid(*[np.arange(R)] * 3, indexing="ij"), -1).reshape(-1, 3)
    c = np.concatenate([np.zeros((len(g), 1), np.int64), g], 1).astype(np.int32)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((len(c), Ci), dtype=np.float32)
    w = scenes.kaiming_uniform_weight(Co, Ci, 1)
    b = rng.standard_normal(Co).astype(np.float32)
    y = oracle.subm_conv(x, w, b, oracle.build_neighbors(c, R, R, R)[0])
    xd = torch.from_numpy(x).reshape(1, R, R, R, Ci).permute(0, 4, 1, 2, 3)
    wd = torch.from_numpy(w).reshape(Co, 3, 3, 3, Ci).permute(0, 4, 1, 2, 3)
    yd = torch.nn.functional.conv3d(xd, wd, torch.from_numpy(b), padding=1).permute(0, 2, 3, 4, 1).reshape(-1, Co).numpy()
    assert np.abs(y - yd).max() < 1e-5


def test_conv_matches_float64_per_tap_matmul_and_indirection():
    rng = np.random.default_rng(3)
    c = scenes.config1_sphere()[:3000]
    x = rng.standard_normal((len(c), 32), dtype=np.float32)
    w = scenes.kaiming_uniform_weight(24, 32, 2)
    nbr = oracle.build_neighbors(c)[0]
    want = np.zeros((len(c), 24))
    for v in range(27):
        m = nbr[:, v] != 0xFFFFFFFF
        want[m] += x[nbr[m, v]].astype(np.float64) @ w[:, v, :].astype(np.float64).T
    assert np.abs(oracle.subm_conv(x, w, None, nbr, f64=True) - want).max() < 1e-12
    assert np.abs(oracle.subm_conv(x, w, None, nbr) - want).max() < 1e-5
    rows = np.array([5, 5, 17, 2999], np.int32)
    wsel = np.array([0, 8, 16, 8], np.int32)
    got = oracle.subm_conv(x, w, None, nbr, nrow=rows, wsel=wsel, Co=8, f64=True)
    for i, (r, s) in enumerate(zip(rows, wsel)):
        assert np.abs(got[i] - want[r, s:s + 8]).max() < 1e-12


def test_subdivide_order_and_gather_skip():
    c = np.array([[0, 1, 2, 3], [1, 0, 0, 5]], np.int32)
    keep = np.zeros((2, 8), bool); keep[0, [1, 6]] = True; keep[1, 7] = True
    cc, src = oracle.subdivide(c, keep)
    assert cc.tolist() == [[0, 3, 4, 6], [0, 2, 5, 7], [1, 1, 1, 11]] and src.tolist() == [1, 6, 15]
    x = np.arange(2 * 16, dtype=np.float32).reshape(2, 16)
    assert np.array_equal(oracle.gather_rows(x, src, 2), x.reshape(-1, 2)[src])
    h = oracle.add_skip(np.zeros((3, 4), np.float32), x, src, 2)       # Cin 16 -> Cs 2, rep 2
    assert h.tolist() == [[2, 2, 3, 3], [12, 12, 13, 13], [30, 30, 31, 31]]


def test_row_ops_match_torch():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((50, 64), dtype=np.float32) * 3 + 1
    g, b = rng.standard_normal(64).astype(np.float32), rng.standard_normal(64).astype(np.float32)
    t = torch.from_numpy(x)
    ln = torch.nn.functional.layer_norm(t, (64,), torch.from_numpy(g), torch.from_numpy(b), 1e-6).numpy()
    assert np.abs(oracle.layer_norm(x, g, b, 1e-6) - ln).max() < 1e-5
    assert np.abs(oracle.act(x, "silu") - torch.nn.functional.silu(t).numpy()).max() < 1e-6
    assert np.abs(oracle.act(x, "gelu") - torch.nn.functional.gelu(t).numpy()).max() < 1e-6
    assert np.abs(oracle.act(x, "gelu_tanh") - torch.nn.functional.gelu(t, approximate="tanh").numpy()).max() < 1e-6
    for dt, td in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        assert np.array_equal(oracle.round_to(x, dt), t.to(td).float().numpy())


def test_scene_sizes():
    c = scenes.config1_sphere()
    assert c.shape == (14534, 4) and c.dtype == np.int32
    assert int((oracle.build_neighbors(c)[0] != 0xFFFFFFFF).sum()) == 259166
    key = scenes.morton3(c[:, 1], c[:, 2], c[:, 3])
    assert (np.diff(key.astype(np.int64)) > 0).all()                     # Morton-sorted, unique
    lv = scenes.config4_levels(levels=3)
    assert [len(l[0]) for l in lv] == [3727, 16725, 57120]
    assert np.array_equal(scenes.subdivide_numpy(lv[0][0], lv[0][1])[0], lv[1][0])


# ------------------------------------------------------------------------------------------ golden vectors
GOLD = os.path.join(os.path.dirname(__file__), "golden", "ref_small.npz")
needs_gold = pytest.mark.skipif(not os.path.exists(GOLD), reason="golden vectors not generated yet")


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _w(Co, Ci, seed, want_sha):
    w = scenes.kaiming_uniform_weight(Co, Ci, seed).astype(np.float16)
    assert _sha(w) == str(want_sha)
    return w.astype(np.float32)


def _close(got, want, max_abs=2e-2, mean_rel=2e-3):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.abs(got - want).max() <= max_abs and np.abs(got - want).sum() / np.abs(want).sum() <= mean_rel


@needs_gold
def test_golden_integer_maps_bit_exact():
    G = np.load(GOLD)
    for tag, ext, B1 in (("i0", 10, 32), ("i1", 4096, 128)):
        nbr, gray, _, srt = oracle.build_neighbors(G[f"{tag}_coords"], ext, ext, ext)
        assert np.array_equal(nbr, G[f"{tag}_nbr"]) and np.array_equal(gray, G[f"{tag}_gray"]) and np.array_equal(srt, G[f"{tag}_sorted"])
        lst, seg = oracle.valid_taps(gray, srt, B1)
        assert np.array_equal(seg, G[f"{tag}_seg"]) and np.array_equal(lst, G[f"{tag}_list"])
    c1 = scenes.config1_sphere()
    assert _sha(c1) == str(G["s1_coords_sha"])
    nbr, gray, _, srt = oracle.build_neighbors(c1)
    assert (_sha(nbr), _sha(gray), _sha(srt)) == (str(G["s1_nbr_sha"]), str(G["s1_gray_sha"]), str(G["s1_sorted_sha"]))
    cc, src = oracle.subdivide(G["c2s_coords"], G["c2s_sub"].astype(np.float32) > 0)
    assert np.array_equal(cc, G["c2s_child"]) and np.array_equal(src, G["c2s_src"])


@needs_gold
def test_golden_features_within_tolerance():
    G = np.load(GOLD)
    for tag, Ci, Co in (("f0", 64, 64), ("f1", 64, 96), ("f2", 128, 256)):
        c, x = G[f"{tag}_coords"], G[f"{tag}_x"].astype(np.float32)
        w = _w(Co, Ci, 7, G[f"{tag}_w_sha"])
        b = G[f"{tag}_b"].astype(np.float32) if f"{tag}_b" in G else None
        _close(oracle.conv_block(x, w, b, oracle.build_neighbors(c)[0], "f16"), G[f"{tag}_y"])
    c, x = G["b0_coords"], G["b0_x"].astype(np.float32)
    w, b = _w(64, 64, 8, G["b0_w_sha"]), G["b0_b"].astype(np.float32)
    nbr = oracle.build_neighbors(c)[0]
    _close(oracle.conv_block(x, w, b, nbr, "f16", ln=(G["b0_g"], G["b0_be"], 1e-6), act_kind="gelu", residual=x), G["b0_y_ln_gelu_res"])
    _close(oracle.conv_block(x, w, b, nbr, "f16", ln=(None, None, 1e-6), act_kind="silu"), G["b0_y_ln_silu"])
    c, x, sub = G["u0_coords"], G["u0_x"].astype(np.float32), G["u0_sub"].astype(np.float32)
    Ci, Cc = 128, 64
    w1, w2 = _w(8 * Cc, Ci, 9, G["u0_w1_sha"]), _w(Cc, Cc, 10, G["u0_w2_sha"])
    cc, src = oracle.subdivide(c, sub > 0)
    hc = oracle.gather_rows(oracle.conv_block(x, w1, G["u0_b1"].astype(np.float32), oracle.build_neighbors(c)[0], "f16"), src, Cc)
    _close(hc, G["u0_hc"])
    h = oracle.round_to(oracle.act(oracle.round_to(oracle.layer_norm(hc, None, None, 1e-6), "f16"), "silu"), "f16")
    out = oracle.conv_block(h, w2, G["u0_b2"].astype(np.float32), oracle.build_neighbors(cc)[0], "f16", skip=(x, src, Cc // (Ci // 8)))
    _close(out, G["u0_out"])
