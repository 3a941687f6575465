"""Host-side logic of the Morton-range sharding (partition, halo lists, index exchange, per-layer halo exchange)
on CPU ranks with the gloo backend.  The conv itself is the CPU oracle here, so a sharded stack of layers must
reproduce the unsharded oracle exactly (same fp32 arithmetic per output row)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from trellis2_cuda_b200 import scenes, sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _scene():
    c = scenes.config1_sphere()[:6000]
    rng = np.random.default_rng(7)
    x = rng.standard_normal((len(c), 32), dtype=np.float32)
    ws = [scenes.kaiming_uniform_weight(32, 32, 20 + l) for l in range(3)]
    return c, x, ws


def _worker(rank, world, port, out_dir, drop_rank):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if drop_rank >= 0:
        return _worker_with_a_lost_peer(rank, world, out_dir, drop_rank)
    try:
        c, x, ws = _scene()
        n = len(c)
        starts = sharding.partition(n, world)
        lo, hi = starts[rank], starts[rank + 1]
        nbr_g = oracle.build_neighbors(c, want_sorted=False)[0][lo:hi].astype(np.int64)
        nbr_g[nbr_g == oracle.EMPTY] = -1
        plan = sharding.build_halo_plan(torch.from_numpy(nbr_g).to(torch.int32), rank, world, starts)
        # every halo row belongs to a peer, grouped by owner; the local map never points past the local array
        assert plan.n_own == hi - lo and sum(plan.recv_counts) == plan.n_halo and plan.recv_counts[rank] == 0
        assert ((plan.halo_global < lo) | (plan.halo_global >= hi)).all()
        assert int(plan.nbr_local.max()) < plan.n_local
        x_local = torch.zeros((plan.n_local, 32))
        x_local[:plan.n_own] = torch.from_numpy(x[lo:hi])
        pack = lambda xo, idx: xo.index_select(0, idx.long())
        nbr_l = plan.nbr_local.numpy().astype(np.int64)
        nbr_l[nbr_l < 0] = oracle.EMPTY
        for w in ws:
            sharding.exchange_halo(plan, x_local, pack)
            y = oracle.subm_conv(x_local.numpy(), w, None, nbr_l.astype(np.uint32))
            x_local[:plan.n_own] = torch.from_numpy(y)
        np.save(os.path.join(out_dir, f"y{rank}.npy"), x_local[:plan.n_own].numpy())
        np.save(os.path.join(out_dir, f"halo{rank}.npy"), np.array([plan.n_halo, plan.n_own]))
    finally:
        dist.destroy_process_group()


def _worker_with_a_lost_peer(rank, world, out_dir, drop_rank):
    """Three layers with a liveness check before each exchange; `drop_rank` leaves after the first layer without
    posting for the second.  No rank may block in a collective for a peer that is gone."""
    c, x, ws = _scene()
    starts = sharding.partition(len(c), world)
    lo, hi = starts[rank], starts[rank + 1]
    nbr_g = oracle.build_neighbors(c, want_sorted=False)[0][lo:hi].astype(np.int64)
    nbr_g[nbr_g == oracle.EMPTY] = -1
    plan = sharding.build_halo_plan(torch.from_numpy(nbr_g).to(torch.int32), rank, world, starts)
    x_local = torch.zeros((plan.n_local, 32))
    x_local[:plan.n_own] = torch.from_numpy(x[lo:hi])
    pack = lambda xo, idx: xo.index_select(0, idx.long())
    monitor = sharding.PeerMonitor(dist.distributed_c10d._get_default_store(), rank, world, timeout_s=3.0)
    done, lost = 0, None
    for layer in range(3):
        if rank == drop_rank and layer == 1:
            break                                              # between steps, nothing of this rank in flight
        try:
            monitor.step(layer)
        except sharding.PeerLost as e:
            lost = e.missing
            break
        sharding.exchange_halo(plan, x_local, pack)
        done += 1
    np.save(os.path.join(out_dir, f"lost{rank}.npy"), np.array([done, -1 if lost is None else lost[0]]))
    os._exit(0)            # no collective tear-down with a peer that is gone


@pytest.mark.parametrize("world", [2, 3])
def test_a_rank_that_never_posts_is_detected_on_the_host(tmp_path, world):
    """One rank leaves between two layers.  The others learn of it from the store before their next exchange, within the
    time limit, and stop with an error instead of waiting in a collective; every rank completed exactly one layer."""
    drop = world - 1
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), drop), nprocs=world, join=True)
    for r in range(world):
        done, lost = np.load(tmp_path / f"lost{r}.npy")
        assert done == 1
        assert lost == (-1 if r == drop else drop)


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_layers_match_unsharded(tmp_path, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), -1), nprocs=world, join=True)
    c, x, ws = _scene()
    nbr = oracle.build_neighbors(c, want_sorted=False)[0]
    want = x
    for w in ws:
        want = oracle.subm_conv(want, w, None, nbr)
    got = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(world)], 0)
    assert np.array_equal(got, want)
    halos = [np.load(tmp_path / f"halo{r}.npy") for r in range(world)]
    assert all(0 < h[0] < h[1] for h in halos)          # a real but small halo on every rank


def test_partition_is_equal_count():
    s = sharding.partition(1003, 8)
    sizes = np.diff(s)
    assert s[0] == 0 and s[-1] == 1003 and sizes.max() - sizes.min() <= 1


def test_single_rank_plan_is_identity():
    c = scenes.config1_sphere()[:500]
    nbr = oracle.build_neighbors(c, want_sorted=False)[0].astype(np.int64)
    nbr[nbr == oracle.EMPTY] = -1
    plan = sharding.build_halo_plan(torch.from_numpy(nbr).to(torch.int32), 0, 1, [0, 500])
    assert plan.n_halo == 0 and np.array_equal(plan.nbr_local.numpy(), nbr)


def test_peer_map_names_owner_and_row():
    """The map of the peer-memory conv: (owner << 28) | row inside the owner's range, absent stays all ones."""
    c = scenes.config1_sphere()[:3000]
    nbr = oracle.build_neighbors(c, want_sorted=False)[0].astype(np.int64)
    nbr[nbr == oracle.EMPTY] = -1
    for world in (3, 8):
        starts = sharding.partition(len(c), world)
        for r in range(world):
            lo, hi = starts[r], starts[r + 1]
            enc = sharding.peer_map(torch.from_numpy(nbr[lo:hi]).to(torch.int32), starts).numpy()
            u = enc.astype(np.int64) & 0xFFFFFFFF
            present = nbr[lo:hi] >= 0
            assert (u[~present] == 0xFFFFFFFF).all()
            assert (u[present] < (1 << 31)).all()            # bit 31 is left to "absent", whatever the owner (ranks 4..7 too)
            owner, row = u[present] >> sharding.PEER_SHIFT, u[present] & ((1 << sharding.PEER_SHIFT) - 1)
            assert owner.max() < world and (np.asarray(starts)[owner] + row == nbr[lo:hi][present]).all()
            assert (owner != r).any() and (owner == r).sum() > 0.8 * owner.size        # a real but small halo
    with pytest.raises(ValueError):
        sharding.peer_map(torch.zeros((1, 27), dtype=torch.int32), list(range(10)))       # more than 8 ranks
