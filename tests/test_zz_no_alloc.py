"""The allocation-free neighbour-map entry point, t2sc_build_neighbors_static.

Some hosts of this library cannot call cudaMalloc while they are running: they have handed the whole device
to their own arena, or they forbid allocation after start-up because it can fail or stall the device.  For
them the library keeps one fixed 2 MiB hash table inside its own image.  This test calls that entry point
through the C ABI, twice in a row on different coordinate sets (the table is shared and must be cleared by
each call), and requires the same bits as the pool-backed t2sc_build_neighbors.  It lives in the last file
pytest collects so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _random_coords(seed, n, res):
    rng = np.random.default_rng(seed)
    cells = rng.choice(res ** 3, size=n, replace=False)
    x, r = np.divmod(cells, res * res)
    y, z = np.divmod(r, res)
    return np.stack([np.zeros_like(x), x, y, z], 1).astype(np.int32)


def test_static_table_matches_pool_backed_entry_point_twice():
    import trellis2_cuda_b200 as sp
    from trellis2_cuda_b200 import _lib
    ctx = sp.context()
    L = ctx.lib
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    # second set is smaller and elsewhere in the grid: stale keys of the first call would show up as ghosts
    for seed, n, res in ((1, 9000, 40), (2, 2500, 24)):
        c = torch.from_numpy(_random_coords(seed, n, res)).cuda()
        want_nbr = torch.empty((n, 27), dtype=torch.int32, device="cuda")
        want_gray = torch.empty(n, dtype=torch.int32, device="cuda")
        ctx.check(L.t2sc_build_neighbors(ctx.h, p(c), n, res, res, res, p(want_nbr), p(want_gray), None))
        nbr = torch.full((n, 27), 7, dtype=torch.int32, device="cuda")      # outputs are the caller's buffers
        gray = torch.full((n,), 7, dtype=torch.int32, device="cuda")
        ctx.check(L.t2sc_build_neighbors_static(ctx.h, p(c), n, res, res, res, p(nbr), p(gray)))
        torch.cuda.synchronize()
        assert torch.equal(nbr, want_nbr)        # integer map: bit-exact, as in the other parity tests
        assert torch.equal(gray, want_gray)
    # beyond the built-in table: refused with a message, nothing launched
    big = _lib.STATIC_MAX_ROWS + 1
    dummy = torch.zeros((big, 4), dtype=torch.int32, device="cuda")
    out = torch.empty((big, 27), dtype=torch.int32, device="cuda")
    g = torch.empty(big, dtype=torch.int32, device="cuda")
    rc = L.t2sc_build_neighbors_static(ctx.h, p(dummy), big, 4096, 4096, 4096, p(out), p(g))
    assert rc == -3 and b"exceed the built-in table" in L.t2sc_last_error(ctx.h)
