"""Morton-range sharding of one voxel set across the GPUs of a node, with one-voxel halo exchange.

The reference is single-GPU (no collective, no `cudaSetDevice` anywhere in its tree); this is new design for
large grids.  Rows arrive Morton-sorted, so a contiguous row range is a Morton-key range.  Ranges are cut at
equal row COUNTS (equal key-space ranges are several times unbalanced on a surface shell).  A rank owns the
features and outputs of its range.  The rows of other ranks that appear in the neighbour map of an owned row
(the one-voxel halo) are appended after the owned rows, so the rank's local neighbour map indexes one local
feature array and the conv kernel is the single-GPU kernel, unchanged.  Per layer: pack the rows the peers
need (gather kernel), one all-to-all of feature rows (NCCL over NVLink; gloo in the CPU tests), conv.

Everything here is host logic on torch tensors (CPU or CUDA) and `torch.distributed`; the two device-specific
steps stay outside: the owned rows' neighbour map with GLOBAL indices (int32 [n_own,27], -1 = absent) is passed in, and
`pack(x_own, idx)` -> rows.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


def partition(n: int, world: int) -> List[int]:
    """Equal-count contiguous ranges: rank r owns rows [starts[r], starts[r+1])."""
    return [(n * r) // world for r in range(world + 1)]


@dataclasses.dataclass
class HaloPlan:
    rank: int
    world: int
    starts: List[int]
    n_own: int
    halo_global: torch.Tensor        # int64 [n_halo] sorted global rows this rank reads from its peers
    nbr_local: torch.Tensor          # int32 [n_own,27]: < n_own owned, >= n_own halo slot, -1 absent
    recv_counts: List[int]           # rows received from each peer (halo_global is grouped by owner, ascending)
    send_counts: List[int]           # rows sent to each peer
    send_idx: torch.Tensor           # int32 [sum(send_counts)] local owned rows to pack, grouped by destination

    @property
    def n_halo(self) -> int:
        return int(self.halo_global.numel())

    @property
    def n_local(self) -> int:
        return self.n_own + self.n_halo


def local_map(nbr_global: torch.Tensor, lo: int, hi: int, starts: List[int]):
    """No communication: (halo_global sorted int64, nbr_local int32, rows wanted from each owner)."""
    n_own, world, dev = hi - lo, len(starts) - 1, nbr_global.device
    g = nbr_global.to(torch.int64)
    present = g >= 0
    outside = present & ((g < lo) | (g >= hi))
    halo = torch.unique(g[outside])                                   # sorted ascending => grouped by owner
    bounds = torch.tensor(starts, dtype=torch.int64, device=dev)
    owner = torch.searchsorted(bounds, halo, right=True) - 1
    recv_counts = torch.bincount(owner, minlength=world).tolist() if halo.numel() else [0] * world
    local = torch.where(outside, n_own + torch.searchsorted(halo, g.clamp(min=0)), g - lo)
    nbr_local = torch.where(present, local, torch.full_like(local, -1)).to(torch.int32)
    return halo, nbr_local, recv_counts


PEER_SHIFT = 28        # map entries of the peer-memory conv: (owner rank << 28) | row inside the owner's array (T2SC_PEER_SHIFT)


def peer_map(nbr_global: torch.Tensor, starts: List[int]) -> torch.Tensor:
    """No communication and no halo copies: rewrites an owned-rows neighbour map with global indices into the form the
    peer-memory conv reads, (owner << 28) | (global row - first row of the owner); absent stays -1 (0xffffffff).  With
    owners below 8 and rows below 2^28 a present entry never has bit 31 set."""
    world = len(starts) - 1
    if world > 8 or max(starts[r + 1] - starts[r] for r in range(world)) > (1 << PEER_SHIFT):
        raise ValueError("peer maps hold at most 8 ranks and 2^28 rows per rank")
    g = nbr_global.to(torch.int64)
    present = g >= 0
    bounds = torch.tensor(starts, dtype=torch.int64, device=g.device)
    owner = (torch.searchsorted(bounds, g.clamp(min=0), right=True) - 1).clamp(max=world - 1)
    enc = (owner << PEER_SHIFT) | (g - bounds[owner])
    return torch.where(present, enc, torch.full_like(enc, -1)).to(torch.int32)     # present entries are below 2^31


def build_halo_plan(nbr_global: torch.Tensor, rank: int, world: int, starts: List[int], group=None) -> HaloPlan:
    """From the owned rows' neighbour map (global indices) derive the halo, the local map and, by exchanging the
    wanted-row lists, what to send to whom.  Collective over `group`."""
    lo, hi = starts[rank], starts[rank + 1]
    n_own, dev = hi - lo, nbr_global.device
    halo, nbr_local, recv_counts = local_map(nbr_global, lo, hi, starts)
    # tell every peer which of its rows are wanted here
    if world > 1:
        cnt_in = torch.tensor(recv_counts, dtype=torch.int64, device=dev)
        cnt_out = torch.empty(world, dtype=torch.int64, device=dev)
        dist.all_to_all_single(cnt_out, cnt_in, group=group)
        send_counts = cnt_out.tolist()
        want_from_me = torch.empty(sum(send_counts), dtype=torch.int64, device=dev)
        dist.all_to_all_single(want_from_me, halo, output_split_sizes=send_counts, input_split_sizes=recv_counts, group=group)
        send_idx = (want_from_me - lo).to(torch.int32)
    else:
        send_counts, send_idx = [0], torch.empty(0, dtype=torch.int32, device=dev)
    return HaloPlan(rank, world, starts, n_own, halo, nbr_local, recv_counts, send_counts, send_idx)


def exchange_halo(plan: HaloPlan, x_local: torch.Tensor, pack: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], group=None,
                  send_buf: Optional[torch.Tensor] = None) -> None:
    """Fills rows [n_own, n_local) of x_local with the peers' current features of the halo rows."""
    if plan.world == 1 or (plan.n_halo == 0 and plan.send_idx.numel() == 0):
        return
    rows = pack(x_local[:plan.n_own], plan.send_idx) if send_buf is None else pack(x_local[:plan.n_own], plan.send_idx, send_buf)
    dist.all_to_all_single(x_local[plan.n_own:], rows, output_split_sizes=plan.recv_counts, input_split_sizes=plan.send_counts, group=group)


class PeerLost(RuntimeError):
    """A peer did not report for a step within the time limit; carries the missing ranks."""

    def __init__(self, step: int, missing: List[int]):
        super().__init__(f"ranks {missing} did not report for step {step}")
        self.step, self.missing = step, missing


class PeerMonitor:
    """Host-side liveness check between steps, over a torch.distributed store (no GPU involved): every rank posts
    `step` before it launches that step's exchange and then waits, with a time limit, until all peers have posted the
    same step.  A rank that has died, hung or left never posts, so the others raise :class:`PeerLost` on the host
    BEFORE they enqueue a collective or a kernel that would wait for it on the device; they can then drop the step,
    re-partition, or shut down with their own GPUs idle and usable."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "t2sc/alive"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, step: int, rank: int) -> str:
        return f"{self.prefix}/{step}/{rank}"

    def post(self, step: int) -> None:
        self.store.set(self._key(step, self.rank), "1")

    def check(self, step: int) -> None:
        import datetime
        import time
        deadline = time.monotonic() + self.timeout_s
        missing = [r for r in range(self.world) if r != self.rank]
        while missing:
            left = deadline - time.monotonic()
            if left <= 0:
                raise PeerLost(step, missing)
            try:
                self.store.wait([self._key(step, missing[0])], datetime.timedelta(seconds=max(left, 0.01)))
                missing.pop(0)
            except Exception:            # the store's wait timed out (its exception type differs between store kinds)
                missing = [r for r in missing if not self._posted(step, r)]
                if missing:
                    raise PeerLost(step, missing)

    def _posted(self, step: int, rank: int) -> bool:
        try:
            return self.store.check([self._key(step, rank)])
        except Exception:
            return False

    def step(self, step: int) -> None:
        self.post(step)
        self.check(step)


def exchange_halo_async(plan: HaloPlan, x_local: torch.Tensor, pack: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], group=None):
    """Starts the exchange of :func:`exchange_halo` on the process group's communication stream and returns its work
    handle (None when there is nothing to exchange): the caller runs everything that does not read the halo rows, then
    ``work.wait()`` (which makes the current stream wait, not the host), then the rest."""
    if plan.world == 1 or (plan.n_halo == 0 and plan.send_idx.numel() == 0):
        return None
    rows = pack(x_local[:plan.n_own], plan.send_idx)
    return dist.all_to_all_single(x_local[plan.n_own:], rows, output_split_sizes=plan.recv_counts, input_split_sizes=plan.send_counts,
                                  group=group, async_op=True)


def halo_bytes(plan: HaloPlan, channels: int, itemsize: int) -> int:
    return plan.n_halo * channels * itemsize
