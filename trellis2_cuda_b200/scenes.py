"""Seeded synthetic voxel shells standing in for the SC-VAE decoders' surface occupancy.

The reference measures on example images that need its 4B-parameter checkpoints; none of that is
available offline, so the benchmark configurations are analytic surfaces: the active voxels are the
integer grid points whose signed distance to a union of spheres / tori lies within a thickness
band.  Distances are float64 (torch, on the GPU when one is present) and the shapes are deterministic
for a given seed.  Coordinates come back as
int32 ``[N,4]`` = (batch, x, y, z) sorted by 3-D Morton key (x bit highest in each triple), the
row order the benchmark configurations ask for.

Large grids (1024^3, 2048^3) are never materialised: cells of 8^3 voxels are culled with the
1-Lipschitz bound of the distance function, and only surviving cells are refined.
"""
from __future__ import annotations

import dataclasses
import numpy as np


# --------------------------------------------------------------------------------------- shapes
@dataclasses.dataclass(frozen=True)
class Shape:
    kind: str            # "sphere" | "torus"
    c: tuple             # centre (voxel units)
    R: float             # sphere radius / torus major radius
    r: float = 0.0       # torus minor radius
    axis: int = 2        # torus axis

    def scaled(self, s: float) -> "Shape":
        return Shape(self.kind, tuple(s * v for v in self.c), self.R * s, self.r * s, self.axis)


def _sdf_one(sh: Shape, p):
    """p: torch float64 [...,3]."""
    import torch
    d = p - torch.tensor(sh.c, dtype=torch.float64, device=p.device)
    if sh.kind == "sphere":
        return torch.sqrt((d * d).sum(-1)) - sh.R
    a = sh.axis
    o = [i for i in range(3) if i != a]
    q = torch.sqrt(d[..., o[0]] ** 2 + d[..., o[1]] ** 2) - sh.R
    return torch.sqrt(q * q + d[..., a] ** 2) - sh.r


def _sdf_t(shapes, p):
    out = _sdf_one(shapes[0], p)
    for sh in shapes[1:]:
        out = torch_min(out, _sdf_one(sh, p))
    return out


def torch_min(a, b):
    import torch
    return torch.minimum(a, b)


def _device(device=None):
    import torch
    if device is not None:
        return torch.device(device)
    return torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")


def sdf_union(shapes, p: np.ndarray, device=None) -> np.ndarray:
    """Exact distance outside the union, a 1-Lipschitz lower bound inside; p float64 [...,3].
    Evaluated with torch float64 (on the GPU when there is one: plumbing for scene set-up only)."""
    import torch
    t = torch.as_tensor(np.ascontiguousarray(p, dtype=np.float64)).to(_device(device))
    return _sdf_t(shapes, t).cpu().numpy()


def random_shapes(n: int, res: int, rmin: float, rmax: float, seed: int):
    """n alternating spheres / tori with radii uniform in [rmin, rmax], placed to fit the grid."""
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        R = float(rng.uniform(rmin, rmax))
        if i % 2 == 0:
            ext, r, axis = R, 0.0, 2
        else:
            r = float(rng.uniform(0.2, 0.4)) * R
            axis = int(rng.integers(0, 3))
            ext = R + r
        lo, hi = ext + 2.0, res - 3.0 - ext
        if hi <= lo:
            lo = hi = res / 2.0
        c = tuple(float(v) for v in rng.uniform(lo, hi, size=3))
        out.append(Shape("sphere" if i % 2 == 0 else "torus", c, R, r, axis))
    return out


# --------------------------------------------------------------------------------------- Morton
def _part1by2(v: np.ndarray) -> np.ndarray:
    v = v.astype(np.uint64) & np.uint64(0x1FFFFF)
    v = (v | (v << np.uint64(32))) & np.uint64(0x1F00000000FFFF)
    v = (v | (v << np.uint64(16))) & np.uint64(0x1F0000FF0000FF)
    v = (v | (v << np.uint64(8))) & np.uint64(0x100F00F00F00F00F)
    v = (v | (v << np.uint64(4))) & np.uint64(0x10C30C30C30C30C3)
    v = (v | (v << np.uint64(2))) & np.uint64(0x1249249249249249)
    return v


def morton3(x, y, z) -> np.ndarray:
    """Interleave with x as the highest bit of each triple."""
    return (_part1by2(np.asarray(x)) << np.uint64(2)) | (_part1by2(np.asarray(y)) << np.uint64(1)) | _part1by2(np.asarray(z))


def morton_sort_coords(xyz: np.ndarray, batch: int = 0) -> np.ndarray:
    xyz = np.unique(np.asarray(xyz, dtype=np.int64), axis=0)
    order = np.argsort(morton3(xyz[:, 0], xyz[:, 1], xyz[:, 2]), kind="stable")
    xyz = xyz[order]
    out = np.empty((xyz.shape[0], 4), dtype=np.int32)
    out[:, 0] = batch
    out[:, 1:] = xyz
    return out


# --------------------------------------------------------------------------------------- shells
def shell_voxels(shapes, res: int, half_thickness: float, device=None) -> np.ndarray:
    """Integer points p in [0,res)^3 with |sdf_union(p)| <= half_thickness, Morton-sorted int32 [N,4].
    Cells of 64^3, 8^3 then single voxels: a cell survives while |sdf(centre)| <= half_thickness +
    its half diagonal (the distance bound is 1-Lipschitz), so no dense grid is ever built."""
    import torch
    dev = _device(device)
    top = 64 if res > 64 else 8
    n0 = (res + top - 1) // top
    g = torch.arange(n0, dtype=torch.int64, device=dev)
    cells = torch.stack(torch.meshgrid(g, g, g, indexing="ij"), -1).reshape(-1, 3)
    size = top
    while True:
        centre = cells.to(torch.float64) * size + (size - 1) / 2.0
        bound = half_thickness + (np.sqrt(3.0) * (size - 1) / 2.0 + 1e-9 if size > 1 else 0.0)
        keep = torch.zeros(cells.shape[0], dtype=torch.bool, device=dev)
        for i in range(0, cells.shape[0], 1 << 22):
            keep[i:i + (1 << 22)] = _sdf_t(shapes, centre[i:i + (1 << 22)]).abs() <= bound
        cells = cells[keep]
        if size == 1:
            break
        f = 8 if size > 8 else size
        o = torch.arange(f, dtype=torch.int64, device=dev)
        off = torch.stack(torch.meshgrid(o, o, o, indexing="ij"), -1).reshape(-1, 3)
        cells = (cells[:, None, :] * f + off[None]).reshape(-1, 3)
        size //= f
        cells = cells[(cells * size < res).all(1)]
    return morton_sort_coords(cells.cpu().numpy())


def children_in_shell(parents: np.ndarray, shapes_fine, half_thickness: float, device=None) -> np.ndarray:
    """Subdivision flags uint8 [n,8]: slot s = bit0->x, bit1->y, bit2->z child of each parent voxel,
    kept iff the child's own centre lies in the shell evaluated at the fine resolution."""
    n = parents.shape[0]
    flags = np.zeros((n, 8), dtype=np.uint8)
    base = parents[:, 1:].astype(np.float64) * 2.0
    for s in range(8):
        d = np.array([s & 1, (s >> 1) & 1, (s >> 2) & 1], dtype=np.float64)
        flags[:, s] = np.abs(sdf_union(shapes_fine, base + d, device)) <= half_thickness
    return flags


# --------------------------------------------------------------------------------------- configs
def kaiming_uniform_weight(Co: int, Ci: int, seed: int) -> np.ndarray:
    """Drawn as [27, Ci, Co] uniform(-a, a), a = 1/sqrt(27*Ci) (the bound torch's default
    kaiming_uniform_(a=sqrt(5)) gives a conv with fan-in 27*Ci), returned in the operator layout
    [Co, 27, Ci] float32."""
    rng = np.random.default_rng(seed)
    a = 1.0 / np.sqrt(27.0 * Ci)
    w = rng.uniform(-a, a, size=(27, Ci, Co)).astype(np.float32)
    return np.ascontiguousarray(w.transpose(2, 0, 1))


def features(N: int, C: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((N, C), dtype=np.float32)


def config1_sphere(seed: int = 0):
    """64^3 grid, voxels within 1.0 of the surface of the sphere r=24 centred at (32,32,32)."""
    return shell_voxels([Shape("sphere", (32.0, 32.0, 32.0), 24.0)], 64, 1.0)


def config2_shapes(seed: int = 0):
    # stream offset 3: with seed 0 the union's shell has 217,821 voxels (the configuration asks for ~200k)
    return random_shapes(6, 256, 20.0, 90.0, seed + 3)


def config2_shell(seed: int = 0):
    """256^3 grid, shell of thickness 1.5 of a union of 6 random spheres / tori."""
    return shell_voxels(config2_shapes(seed), 256, 0.75)


def config3_pair(seed: int = 0):
    """(parents at 512^3, flags [n,8]) : same six shapes scaled x2; children kept by the 1024^3 shell."""
    sh512 = [s.scaled(2.0) for s in config2_shapes(seed)]
    sh1024 = [s.scaled(4.0) for s in config2_shapes(seed)]
    parents = shell_voxels(sh512, 512, 0.75)
    return parents, children_in_shell(parents, sh1024, 0.75)


def config4_levels(seed: int = 0, levels: int = 5):
    """Shell pyramid 64^3 -> 1024^3: list of (coords_l, flags_l or None); flags_l selects the children
    that form coords_{l+1} (analytic shell at the finer level, restricted to children of level l)."""
    base = random_shapes(3, 64, 6.0, 14.0, seed + 1)   # seed 0 -> 3,727 voxels at 64^3
    coords = shell_voxels(base, 64, 0.5)
    out = []
    for l in range(levels):
        if l == levels - 1:
            out.append((coords, None))
            break
        fine = [s.scaled(2.0 ** (l + 1)) for s in base]
        flags = children_in_shell(coords, fine, 0.75)
        out.append((coords, flags))
        coords = subdivide_numpy(coords, flags)[0]
    return out


def config5_shell(seed: int = 0, res: int = 2048, n_shapes: int = 12, rmin: float = 85.0, rmax: float = 380.0):
    """2048^3 grid, thickness-1.5 shell of a union of 12 spheres / tori (about 8 M voxels)."""
    return shell_voxels(random_shapes(n_shapes, res, rmin, rmax, seed + 5), res, 0.75)


def subdivide_numpy(parents: np.ndarray, flags: np.ndarray):
    """Children in (parent, slot) ascending order: coords (b, 2x+(s&1), 2y+(s>>1&1), 2z+(s>>2&1)),
    src = parent*8 + slot.  Host helper for building scenes; the operator under test is the CUDA one."""
    p, s = np.nonzero(flags)
    c = np.empty((p.shape[0], 4), dtype=np.int32)
    c[:, 0] = parents[p, 0]
    c[:, 1] = parents[p, 1] * 2 + (s & 1)
    c[:, 2] = parents[p, 2] * 2 + ((s >> 1) & 1)
    c[:, 3] = parents[p, 3] * 2 + ((s >> 2) & 1)
    return c, (p * 8 + s).astype(np.int32)
