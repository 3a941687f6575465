"""GPU parity at the stated shapes of the five benchmark configurations: the CUDA library through its C ABI against
the CPU oracle on the same seeded scenes.  Integer maps are compared bit for bit over the whole scene; features on
sampled rows (the oracle is a scalar CPU program) within max-abs 2e-2 / mean-rel 2e-3 of an fp32-accumulated
reference, layer by layer with teacher forcing where layers are stacked (every layer is fed the library's own previous
output, the way the reference checks stage by stage on reference inputs, docs/blog.md:99-101 of trellis2-cuda)."""
import numpy as np
import pytest
import torch

import oracle
from trellis2_cuda_b200 import scenes

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_REL = 2e-2, 2e-3
TD = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
ULP = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7, "f32": 2.0 ** -23}


@pytest.fixture(scope="module")
def sp():
    import trellis2_cuda_b200 as m
    m.context()          # raises if the library or the GPU is missing
    return m


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.float().cpu().numpy() if t.is_floating_point() else t.cpu().numpy()


def check_feats(got, want, what, dt=None):
    """max-abs <= 2e-2 and mean-rel <= 2e-3; with `dt` given (outputs whose magnitude is not bounded near 1: after a
    LayerNorm, an activation or a residual) one rounding step of the storage dtype is also accepted where it exceeds
    2e-2."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    err = np.abs(got - want)
    allow = np.full_like(err, MAX_ABS)
    if dt is not None:
        allow = np.maximum(allow, ULP[dt] * 2.0 ** np.floor(np.log2(np.maximum(np.abs(want), 1e-30))))
    mr = err.sum() / max(np.abs(want).sum(), 1e-30)
    assert (err <= allow).all() and mr <= MEAN_REL, f"{what}: max-abs {err.max():.3e} mean-rel {mr:.3e}"


def gauss(n, C, seed, td):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn((n, C), generator=g, device="cuda").to(td)


def weight(Co, Ci, seed, td, scale=1.0):
    return dev(scenes.kaiming_uniform_weight(Co, Ci, seed) * scale, td)


def sample_rows(n, k, seed):
    return np.sort(np.random.default_rng(seed).choice(n, min(k, n), replace=False)).astype(np.int32)


# ------------------------------------------------------------------------------------------ configuration 3
def test_config3_full_size_fp16(sp):
    """886,752 parents at 512^3 -> 3,288,465 kept children at 1024^3, fp16: the 128 -> 64 subdivision conv over kept
    children only, then the 64 -> 64 submanifold conv on the children, default plans (the 64-channel kernel with two
    gather groups runs ~170 work items per CTA here).  Parent map, child coordinates, src and the 3.3 M-row child map
    bit for bit; both convs on sampled rows."""
    dt, td = "f16", torch.float16
    parents, flags = scenes.config3_pair()
    assert parents.shape[0] == 886752
    cc, src = oracle.subdivide(parents, flags)
    assert cc.shape[0] == 3288465
    nbr_p = oracle.build_neighbors(parents, want_sorted=False)[0]
    parent = sp.build_neighbors(dev(parents), want_sorted=False)
    assert np.array_equal(host(parent.nbr).view(np.uint32), nbr_p)
    lv = sp.subdivide(parent, dev(flags))
    assert np.array_equal(host(lv.coords), cc) and np.array_equal(host(lv.src), src)
    nbr_c, gray_c, _, _ = oracle.build_neighbors(cc, want_sorted=False)
    assert np.array_equal(host(lv.nb.nbr).view(np.uint32), nbr_c) and np.array_equal(host(lv.nb.gray), gray_c)
    del nbr_c
    Ci, Cc = 128, 64
    x = gauss(parents.shape[0], Ci, 3, td)
    w1, b1 = weight(8 * Cc, Ci, 31, td), dev(0.05 * np.random.default_rng(32).standard_normal(8 * Cc).astype(np.float32), td)
    up = sp.subdiv_conv(x, w1, b1, lv)
    rows = sample_rows(src.shape[0], 300, 1)
    want = oracle.conv_block(host(x), host(w1), host(b1), nbr_p, dt, nrow=(src[rows] >> 3).astype(np.int32),
                             wsel=((src[rows] & 7) * Cc).astype(np.int32), Co=Cc)
    check_feats(host(up[torch.from_numpy(rows).cuda().long()]), want, "config 3 subdivision conv 128 -> 64")
    del x
    # second half: 64 -> 64 on the children, fed with the library's own output of the first half
    w2 = weight(Cc, Cc, 33, td)
    y = sp.subm_conv(up, w2, None, lv.nb)
    lv.nb.ctx.device_status()
    nbr_rows = host(lv.nb.nbr)[rows].view(np.uint32)
    # the oracle needs the sampled rows' neighbours only: compact them so the 3.3 M x 64 input is not widened on the host
    need = np.unique(nbr_rows[nbr_rows != oracle.EMPTY])
    remap = np.full(src.shape[0], oracle.EMPTY, np.uint32)
    remap[need] = np.arange(need.shape[0], dtype=np.uint32)
    nbr_small = np.where(nbr_rows != oracle.EMPTY, remap[np.minimum(nbr_rows, src.shape[0] - 1)], oracle.EMPTY).astype(np.uint32)
    want2 = oracle.conv_block(host(up[torch.from_numpy(need.astype(np.int64)).cuda()]), host(w2), None, nbr_small, dt)
    check_feats(host(y[torch.from_numpy(rows).cuda().long()]), want2, "config 3 submanifold conv 64 -> 64")
    # size-independent properties at the full size: homogeneity in the weights by a power of two (exact wherever neither
    # result is an fp16 subnormal, whose rounding step does not scale), zero in -> zero out
    y2 = sp.subm_conv(up, w2 * 2, None, lv.nb).float()
    normal = y.float().abs() >= 2.0 ** -13
    assert torch.equal(y2[normal], y.float()[normal] * 2) and float((y2 - 2 * y.float()).abs().max()) <= 2.0 ** -23
    assert torch.count_nonzero(sp.subm_conv(torch.zeros_like(up), w2, None, lv.nb)) == 0


# ------------------------------------------------------------------------------------------ configuration 4
def test_config4_stack_at_its_stated_widths(sp):
    """The decoder-like stack at 1024 -> 512 -> 256 channels over the first three levels of its voxel pyramid
    (3,727 -> 16,725 -> 57,120 voxels): per level two blocks of conv -> LayerNorm -> GELU -> conv -> residual, then the
    2x subdivision conv that halves the channels (1024 -> 8 x 512, 512 -> 8 x 256).  These are the small-N / wide-C
    shapes: 16 and 8 K-chunks per tap, LayerNorm over rows wider than one accumulator (the row pass)."""
    lv = scenes.config4_levels(levels=4)
    rng = np.random.default_rng(4)
    dt, td = "bf16", torch.bfloat16
    C = 1024
    coords = lv[0][0]
    assert coords.shape[0] == 3727
    cache = sp.build_neighbors(dev(coords), want_sorted=False)
    x = gauss(coords.shape[0], C, 40, td)
    vec = lambda n, s: dev((s * rng.standard_normal(n)).astype(np.float32))
    for level in range(3):
        coords, flags = lv[level]
        nbr = oracle.build_neighbors(coords, want_sorted=False)[0]
        assert np.array_equal(host(cache.nbr).view(np.uint32), nbr)
        rows = sample_rows(coords.shape[0], 96 if C >= 512 else 200, level)
        rows_t = torch.from_numpy(rows).cuda().long()
        for blk in range(2):
            w1, w2 = weight(C, C, 100 + 10 * level + blk, td), weight(C, C, 105 + 10 * level + blk, td)
            b1 = vec(C, 0.05).to(td)
            g, be = 1 + vec(C, 0.1), vec(C, 0.1)
            h0 = sp.subm_conv(x, w1, b1, cache)
            want = oracle.conv_block(host(x), host(w1), host(b1), nbr, dt, nrow=rows)
            check_feats(host(h0[rows_t]), want, f"L{level} B{blk} conv1 {C}->{C}")
            h = sp.subm_conv(x, w1, b1, cache, ln=(g, be, 1e-6), act="gelu")
            forced = oracle.round_to(oracle.act(oracle.round_to(oracle.layer_norm(host(h0[rows_t]), host(g), host(be), 1e-6), dt), "gelu"), dt)
            check_feats(host(h[rows_t]), forced, f"L{level} B{blk} LayerNorm + GELU over {C} channels on the library's conv output", dt)
            y = sp.subm_conv(h, w2, b1, cache, residual=x)
            want = oracle.conv_block(host(h), host(w2), host(b1), nbr, dt, nrow=rows, residual=host(x[rows_t]))
            check_feats(host(y[rows_t]), want, f"L{level} B{blk} conv2 + residual", dt)
            x = y
            del w1, w2
        Cc = C // 2
        nxt = sp.subdivide(cache, dev(flags))
        assert np.array_equal(host(nxt.coords), lv[level + 1][0])
        wu, bu = weight(8 * Cc, C, 150 + level, td), vec(8 * Cc, 0.05).to(td)
        up = sp.subdiv_conv(x, wu, bu, nxt)
        src = host(nxt.src)
        r2 = sample_rows(src.shape[0], 96 if C >= 512 else 200, 10 + level)
        want = oracle.conv_block(host(x), host(wu), host(bu), nbr, dt, nrow=(src[r2] >> 3).astype(np.int32),
                                 wsel=((src[r2] & 7) * Cc).astype(np.int32), Co=Cc)
        check_feats(host(up[torch.from_numpy(r2).cuda().long()]), want, f"L{level} subdivision conv {C} -> 8 x {Cc}")
        del wu
        x, cache, C = up, nxt.nb, Cc
    cache.ctx.device_status()


# ------------------------------------------------------------------------------------------ configuration 5
def test_config5_scene_on_one_gpu(sp):
    """The 8,597,581-voxel shell of the sharded configuration (2048^3, C = 128, bf16) on one GPU with the default plan
    for that size (128-row tiles, mask sort inside runs of 65,536 rows): the whole map bit for bit, the conv on sampled
    rows, two stacked layers, and the agreement of the 128-row and 256-row schedules."""
    dt, td = "bf16", torch.bfloat16
    c = scenes.config5_shell()
    n, C = c.shape[0], 128
    assert n == 8597581
    nbr, gray, _, _ = oracle.build_neighbors(c, want_sorted=False)
    cache = sp.build_neighbors(dev(c), want_sorted=False)
    assert torch.equal(cache.gray.cpu(), torch.from_numpy(gray))
    assert torch.equal(cache.nbr.cpu(), torch.from_numpy(nbr.view(np.int32)))
    assert cache.plan_for(C, C).stats()["active_taps"] == int((nbr != oracle.EMPTY).sum())
    x = gauss(n, C, 50, td)
    rows = sample_rows(n, 300, 5)
    rows_t = torch.from_numpy(rows).cuda().long()
    nbr_rows = nbr[rows]
    del nbr

    def oracle_rows(xin, w):
        need = np.unique(nbr_rows[nbr_rows != oracle.EMPTY])
        remap = np.full(n, oracle.EMPTY, np.uint32)
        remap[need] = np.arange(need.shape[0], dtype=np.uint32)
        small = np.where(nbr_rows != oracle.EMPTY, remap[np.minimum(nbr_rows, n - 1)], oracle.EMPTY).astype(np.uint32)
        return oracle.conv_block(host(xin[torch.from_numpy(need.astype(np.int64)).cuda()]), host(w), None, small, dt)

    for layer in range(2):
        w = weight(C, C, 60 + layer, td)
        y = sp.subm_conv(x, w, None, cache)
        check_feats(host(y[rows_t]), oracle_rows(x, w), f"config 5 layer {layer}")
        x = y
    cache.ctx.device_status()
    other = sp.cache_from_map(cache.coords, cache.nbr, cache.gray, tile_rows=256)
    assert torch.equal(sp.subm_conv(x, w, None, other), sp.subm_conv(x, w, None, cache))     # same accumulation order per row
