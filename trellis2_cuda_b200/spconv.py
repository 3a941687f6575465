"""Host-side mirror of the reference's sparse-conv operator API on top of the t2sc C ABI.

Same names and argument meaning as trellis2-cuda's ``src/spconv.h`` (``build_neighbors``, ``SpConvCache``,
``spconv_cfg``, ``SpConvCfg``, ``subm_conv``) and the sparse pieces of its ``SDecoder`` (``src/sdec.cu``:
``c2s`` -> :func:`subdivide`, ``k_gather_rows`` -> :func:`gather_rows`, ``k_add_skip`` -> :func:`add_skip`,
and the ops it strings after each conv, ``layer_norm`` / ``act_`` / ``add_`` of ``src/ops.h``).  Tensors are
torch CUDA tensors (device memory and streams only; every operator is a kernel of libt2sc.so).  Errors
raise :class:`T2scError` with the library's message, as the reference throws ``std::runtime_error``.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Optional

import torch

from . import _lib
from ._lib import T2scError

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.uint8: _lib.U8}
_ACT = {None: 0, "none": 0, "silu": 1, "gelu_tanh": 2, "gelu": 3, "gelu_erf": 3}
_VARIANT = {"auto": 0, "simt": 1, "umma": 2, "umma_pair": 3}

_contexts: dict = {}


class Context:
    """One t2sc context per (device, stream).  Work is enqueued on the torch stream that was current when
    the context was made (the legacy default stream is passed by its explicit handle)."""

    def __init__(self, device: int, stream_handle: int):
        self.lib = _lib.load()
        self.device = device
        h = ctypes.c_void_p()
        rc = self.lib.t2sc_ctx_create(device, ctypes.c_void_p(stream_handle or 1), ctypes.byref(h))
        if rc:
            raise T2scError(rc, self.lib.t2sc_last_error(None).decode())
        self.h = h

    def check(self, rc: int) -> None:
        if rc:
            raise T2scError(rc, self.lib.t2sc_last_error(self.h).decode())

    def launch_count(self) -> int:
        return int(self.lib.t2sc_launch_count(self.h))

    def device_status(self) -> None:
        st = ctypes.c_int(0)
        self.check(self.lib.t2sc_device_status(self.h, ctypes.byref(st)))

    def sync(self) -> None:
        self.check(self.lib.t2sc_ctx_sync(self.h))


def context(device=None) -> Context:
    if not torch.cuda.is_available():
        raise RuntimeError("trellis2_cuda_b200 needs a CUDA device: there is no CPU path")
    idx = None if device is None else torch.device(device).index
    dev = torch.cuda.current_device() if idx is None else idx
    sh = torch.cuda.current_stream(dev).cuda_stream
    key = (dev, sh)
    if key not in _contexts:
        _contexts[key] = Context(dev, sh)
    return _contexts[key]


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _chk(t: torch.Tensor, name: str, dtype=None, ndim=None):
    if not t.is_cuda or not t.is_contiguous():
        raise T2scError(-1, f"{name} must be a contiguous CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise T2scError(-1, f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise T2scError(-1, f"{name} must have {ndim} dims, got {tuple(t.shape)}")


@dataclasses.dataclass
class SpConvCfg:
    """Tile configuration, as the reference's ``SpConvCfg{B1,BK,S}`` (src/spconv.h:13)."""
    B1: int
    BK: int
    S: int


def spconv_cfg(N: int, Ci: int, Co: int) -> SpConvCfg:
    """The reference replays FlexGEMM's autotuned (B1, BK, SPLITK) per shape (src/spconv.cu:186-221); on a
    B200 its table has no entry and it runs 128/64/1.  This build has one schedule: 128-row tiles, 64-channel
    K steps, no split-K (the persistent tcgen05 kernel keeps all SMs busy without it)."""
    return SpConvCfg(128, 64, 1)


class _Plan:
    def __init__(self, ctx: Context, nbr, gray, src=None, block_rows: int = 0, tile_rows: int = 0, n_own: int = 0):
        self.ctx, self.nbr, self.gray, self.src = ctx, nbr, gray, src     # keep the borrowed tensors alive
        m = src.shape[0] if src is not None else nbr.shape[0]
        h = ctypes.c_void_p()
        if n_own:       # one rank of a partitioned scene: interior tiles first, tiles that read halo rows (entries >= n_own) last
            ctx.check(ctx.lib.t2sc_plan_create_split(ctx.h, _ptr(nbr), _ptr(gray), nbr.shape[0], n_own, block_rows, tile_rows, ctypes.byref(h)))
        else:
            ctx.check(ctx.lib.t2sc_plan_create(ctx.h, _ptr(nbr), _ptr(gray), nbr.shape[0], _ptr(src), m, block_rows, tile_rows, ctypes.byref(h)))
        self.h, self.n_out = h, m

    def parts(self):
        a, b = ctypes.c_int64(), ctypes.c_int64()
        self.ctx.check(self.ctx.lib.t2sc_plan_parts(self.ctx.h, self.h, ctypes.byref(a), ctypes.byref(b)))
        return {"interior_tiles": a.value, "boundary_tiles": b.value}

    def stats(self):
        t, c, a = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        self.ctx.check(self.ctx.lib.t2sc_plan_stats(self.ctx.h, self.h, ctypes.byref(t), ctypes.byref(c), ctypes.byref(a)))
        return {"tiles": t.value, "computed_taps": c.value, "active_taps": a.value}

    def set_input_rows(self, n_in: int) -> None:
        """The map's entries index a feature array of n_in rows (owned rows + appended halo rows)."""
        if n_in != getattr(self, "_n_in", self.nbr.shape[0]):
            self.ctx.check(self.ctx.lib.t2sc_plan_set_input_rows(self.ctx.h, self.h, n_in))
            self._n_in = n_in

    def check(self, n_in: int) -> "_Plan":
        """Runs the one-time bounds check of the plan's map copy against a feature array of n_in rows now instead of in the
        first conv."""
        self.set_input_rows(n_in)
        self.ctx.check(self.ctx.lib.t2sc_plan_check(self.ctx.h, self.h, n_in))
        return self

    def order(self) -> torch.Tensor:
        o = torch.empty(self.n_out, dtype=torch.int32, device=self.nbr.device)
        self.ctx.check(self.ctx.lib.t2sc_plan_order(self.ctx.h, self.h, _ptr(o)))
        return o

    def __del__(self):
        try:
            if self.h:
                self.ctx.lib.t2sc_plan_destroy(self.ctx.h, self.h)
        except Exception:
            pass


class SpConvCache:
    """Neighbour cache of one coordinate set (src/spconv.h:6-11): ``N``, ``nbr`` [N,27] (int32 storage of
    the uint32 map, -1 = 0xffffffff = absent), ``gray`` [N] presence mask, ``sorted`` [N] reference row
    order, ``valid(B1)`` -> (tap list, segment offsets).  ``plan`` is this build's schedule."""

    def __init__(self, ctx, coords, nbr, gray, sorted_, block_rows=0, tile_rows=0):
        self.ctx, self.coords, self.N = ctx, coords, int(coords.shape[0])
        self.nbr, self.gray, self.sorted = nbr, gray, sorted_
        self.vk: dict = {}
        self._plan = None
        self._block_rows, self._tile_rows = block_rows, tile_rows

    def valid(self, B1: int):
        if B1 not in self.vk:
            if self.sorted is None:
                raise T2scError(-1, "valid() needs the reference row order: build_neighbors(..., want_sorted=True)")
            nb = (self.N + B1 - 1) // B1
            seg = torch.zeros(nb + 1, dtype=torch.int32, device=self.nbr.device)
            lst = torch.zeros(max(27 * nb, 1), dtype=torch.int32, device=self.nbr.device)
            tot = ctypes.c_int64(0)
            self.ctx.check(self.ctx.lib.t2sc_valid_taps(self.ctx.h, _ptr(self.gray), _ptr(self.sorted), self.N, B1,
                                                        _ptr(seg), _ptr(lst), ctypes.byref(tot)))
            self.vk[B1] = (lst[:max(tot.value, 1)], seg)
        return self.vk[B1]

    @property
    def plan(self) -> _Plan:
        return self.plan_for(256)

    def _tile_rows_for(self, Co: int, Ci: int) -> int:
        """128-row tiles unless forced: every layer narrower than 256 output channels runs the form of the kernel that packs
        several (tap, chunk) units into one pipeline stage, which exists for 128-row tiles; 256-channel slabs share nothing
        between two 128-row halves that the L2 does not already give them (measured on 218 k rows: 256-row tiles are 10 %
        slower there because one union mask then covers 256 rows)."""
        return self._tile_rows or 128

    def plan_for(self, Co: int, Ci: int = 0) -> _Plan:
        """The schedule used for a conv with Ci -> Co channels."""
        tr = self._tile_rows_for(Co, Ci)
        if self._plan is None:
            self._plan = {}
        if tr not in self._plan:
            self._plan[tr] = _Plan(self.ctx, self.nbr, self.gray, None, self._block_rows, tr)
        return self._plan[tr]

    def split_plan_for(self, Co: int, Ci: int, n_own: int) -> _Plan:
        """The schedule of one rank of a partitioned scene whose map indexes owned rows (< n_own) and appended halo rows:
        same tile height as :meth:`plan_for`, interior tiles first, boundary tiles last (see :func:`subm_conv_split`)."""
        tr = self._tile_rows_for(Co, Ci)
        if self._plan is None:
            self._plan = {}
        if ("split", tr, n_own) not in self._plan:
            self._plan[("split", tr, n_own)] = _Plan(self.ctx, self.nbr, self.gray, None, self._block_rows, tr, n_own=n_own)
        return self._plan[("split", tr, n_own)]


def build_neighbors(coords: torch.Tensor, W: int = 4096, H: int = 4096, D: int = 4096, want_sorted: bool = True,
                    block_rows: int = 0, tile_rows: int = 0) -> SpConvCache:
    """coords int32 [N,4] = (b,x,y,z) -> SpConvCache (src/spconv.cu:38-54)."""
    _chk(coords, "coords", torch.int32, 2)
    if coords.shape[1] != 4:
        raise T2scError(-1, f"coords must be [N,4], got {tuple(coords.shape)}")
    ctx = context(coords.device)
    n = coords.shape[0]
    nbr = torch.empty((n, 27), dtype=torch.int32, device=coords.device)
    gray = torch.empty(n, dtype=torch.int32, device=coords.device)
    srt = torch.empty(n, dtype=torch.int32, device=coords.device) if want_sorted else None
    ctx.check(ctx.lib.t2sc_build_neighbors(ctx.h, _ptr(coords), n, W, H, D, _ptr(nbr), _ptr(gray), _ptr(srt)))
    return SpConvCache(ctx, coords, nbr, gray, srt, block_rows, tile_rows)


def build_neighbors_range(coords: torch.Tensor, row_lo: int, row_hi: int, W: int = 4096, H: int = 4096, D: int = 4096):
    """Neighbour rows (global indices) and masks of rows [row_lo, row_hi) of `coords` -> (nbr int32 [m,27], gray [m])."""
    _chk(coords, "coords", torch.int32, 2)
    ctx = context(coords.device)
    m = row_hi - row_lo
    nbr = torch.empty((m, 27), dtype=torch.int32, device=coords.device)
    gray = torch.empty(m, dtype=torch.int32, device=coords.device)
    ctx.check(ctx.lib.t2sc_build_neighbors_range(ctx.h, _ptr(coords), coords.shape[0], W, H, D, row_lo, row_hi, _ptr(nbr), _ptr(gray)))
    return nbr, gray


def voxel_lookup(coords: torch.Tensor, queries: torch.Tensor, W: int = 4096, H: int = 4096, D: int = 4096) -> torch.Tensor:
    """rows[q] = index of the row of `coords` [n,4] equal to `queries[q]` = (b,x,y,z), or -1: the lookup of the reference's
    vhash_find (src/mesh.cu:7-19) over this library's voxel hash."""
    _chk(coords, "coords", torch.int32, 2); _chk(queries, "queries", torch.int32, 2)
    if coords.shape[1] != 4 or queries.shape[1] != 4:
        raise T2scError(-1, "coords and queries must be [*,4]")
    ctx = context(coords.device)
    rows = torch.empty(queries.shape[0], dtype=torch.int32, device=coords.device)
    ctx.check(ctx.lib.t2sc_voxel_lookup(ctx.h, _ptr(coords), coords.shape[0], W, H, D, _ptr(queries), queries.shape[0], _ptr(rows)))
    return rows


def cache_from_map(coords_like: torch.Tensor, nbr: torch.Tensor, gray: torch.Tensor, block_rows: int = 0, tile_rows: int = 0) -> SpConvCache:
    """Wraps an existing neighbour map (e.g. a rank's local map whose indices point into owned + halo rows)."""
    return SpConvCache(context(nbr.device), coords_like, nbr, gray, None, block_rows, tile_rows)


def subm_conv_local(x: torch.Tensor, w: torch.Tensor, b, c: SpConvCache, **kw) -> torch.Tensor:
    """subm_conv whose input has MORE rows than the map (owned rows first, halo rows appended); output [c.N, Co]."""
    if x.shape[0] < c.N:
        raise T2scError(-1, f"spconv shapes: x has {x.shape[0]} rows, cache has {c.N}")
    plan = c.plan_for(w.shape[0], w.shape[2])
    plan.set_input_rows(x.shape[0])
    return _conv(c.ctx, plan, x, w, b, w.shape[0], kw.get("ln"), kw.get("act"), kw.get("residual"), kw.get("skip"),
                 kw.get("variant", "auto"), kw.get("out"))


def subm_conv_split(x: torch.Tensor, w: torch.Tensor, b, c: SpConvCache, plan: _Plan, part: str, *, ln=None, act=None,
                    residual=None, out=None, n_local: Optional[int] = None, ctx: Optional[Context] = None) -> torch.Tensor:
    """One part ("interior" | "boundary" | "all") of a conv over a split plan (:meth:`SpConvCache.split_plan_for`): x has
    the owned rows first and the halo rows appended; the interior part reads owned rows only, so it can run while the
    halo rows are still in flight.  Both parts write into the same `out` [c.N, Co]; the rows of the other part are left
    untouched.  `n_local` (owned + halo rows, the index space of the plan's map) may be given when x itself holds fewer rows
    - the interior part of a rank whose halo rows are never copied because its boundary tiles gather them from peer
    memory.  `ctx` runs the part on another context of the same device (another stream): the two parts write disjoint
    rows, so the boundary part may run on a side stream that waits for the halo only, beside the interior part's tail."""
    if x.shape[0] < c.N:
        raise T2scError(-1, f"spconv shapes: x has {x.shape[0]} rows, cache has {c.N}")
    if n_local is not None and part != "interior":
        raise T2scError(-1, "n_local may exceed the rows of x only for the interior part, which reads owned rows alone")
    _chk(x, "x", None, 2); _chk(w, "w", x.dtype, 3)
    Ci, Co = x.shape[1], w.shape[0]
    if w.shape[1] != 27 or w.shape[2] != Ci:
        raise T2scError(-1, f"spconv shapes: w {tuple(w.shape)} does not match x {tuple(x.shape)}")
    n_in = x.shape[0] if n_local is None else n_local
    plan.set_input_rows(n_in)
    y = out if out is not None else torch.empty((plan.n_out, Co), dtype=x.dtype, device=x.device)
    e, keep = _epilogue(Co, x.dtype, b, ln, act, residual, None)
    ctx = ctx or c.ctx
    setattr(plan, "keep_" + part, keep)
    ctx.check(ctx.lib.t2sc_subm_conv_part(ctx.h, plan.h, _ptr(x), _ptr(w), ctypes.byref(e), _ptr(y), _DT[x.dtype], n_in, Ci, Co,
                                          0, _lib.PART[part]))
    return y


def subm_conv_peers(x_ptrs, x_rows, rank: int, x_dtype, Ci: int, w: torch.Tensor, b, c: SpConvCache, *, ln=None, act=None, residual=None,
                    out=None, plan: Optional[_Plan] = None, part: str = "all", peer_nbr: Optional[torch.Tensor] = None,
                    ctx: Optional[Context] = None):
    """subm_conv for one rank of a Morton-range partition whose neighbour map holds (owner << 28) | row entries:
    the rows are gathered straight from the peers' feature arrays (`x_ptrs[r]` = device address of rank r's array
    mapped into this process, `x_rows[r]` its row count, `x_ptrs[rank]` the local one), so no halo is packed or
    exchanged.  Returns [c.N, Co].  With `plan` (a split plan over the LOCAL map), `part="boundary"` and `peer_nbr` (the
    (owner, row) form of the same map) only the boundary tiles take this path; the interior tiles go through
    :func:`subm_conv_split`."""
    _chk(w, "w", x_dtype, 3)
    Co = w.shape[0]
    plan = plan or c.plan_for(Co, Ci)
    y = out if out is not None else torch.empty((plan.n_out, Co), dtype=x_dtype, device=w.device)
    e, keep = _epilogue(Co, x_dtype, b, ln, act, residual, None)
    plan.keep_peers = keep + ([peer_nbr] if peer_nbr is not None else [])
    arr = (ctypes.c_void_p * len(x_ptrs))(*[int(p) for p in x_ptrs])
    rows = (ctypes.c_int64 * len(x_ptrs))(*[int(r) for r in x_rows])
    ctx = ctx or c.ctx
    ctx.check(ctx.lib.t2sc_subm_conv_peers_part(ctx.h, plan.h, _ptr(peer_nbr), arr, rows, len(x_ptrs), int(rank), _ptr(w), ctypes.byref(e),
                                                    _ptr(y), _DT[x_dtype], Ci, Co, _lib.PART[part]))
    return y


def peer_barrier(ctx: Context, flag_ptrs, rank: int, epoch: int, timeout_ms: int = 2000) -> None:
    """Enqueues the bounded flag barrier between the ranks of a node (t2sc_peer_barrier): `flag_ptrs[r]` is the device
    address of rank r's int32 flag array mapped into this process.  A peer that never arrives shows up as
    T2SC_ERR_DEVICE at the next :meth:`Context.device_status`, not as a hang."""
    arr = (ctypes.c_void_p * len(flag_ptrs))(*[int(p) for p in flag_ptrs])
    ctx.check(ctx.lib.t2sc_peer_barrier(ctx.h, arr, len(flag_ptrs), int(rank), int(epoch), int(timeout_ms)))


def _epilogue(Co, dtype, bias, ln, act, residual, skip):
    e = _lib.Epilogue()
    keep = []
    if bias is not None:
        bias = bias.to(dtype).contiguous()            # the reference casts an fp32 bias to fp16 (src/spconv.cu:167)
        keep.append(bias)
        e.bias = bias.data_ptr()
    if ln is not None:
        gamma, beta, eps = ln
        e.ln, e.ln_eps = 1, float(eps)
        if gamma is not None:
            gamma = gamma.float().contiguous(); keep.append(gamma); e.ln_gamma = gamma.data_ptr()
        if beta is not None:
            beta = beta.float().contiguous(); keep.append(beta); e.ln_beta = beta.data_ptr()
    e.act = _ACT[act]
    if residual is not None:
        _chk(residual, "residual", dtype, 2)
        e.residual = residual.data_ptr()
    if skip is not None:
        sx, ssrc, rep = skip
        _chk(sx, "skip x", dtype, 2); _chk(ssrc, "skip src", torch.int32, 1)
        e.skip_x, e.skip_src, e.skip_cin, e.skip_rep = sx.data_ptr(), ssrc.data_ptr(), sx.shape[1], int(rep)
    return e, keep


def _conv(ctx, plan, x, w, b, Co, ln, act, residual, skip, variant, out):
    _chk(x, "x", None, 2); _chk(w, "w", x.dtype, 3)
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise T2scError(-1, f"unsupported feature dtype {x.dtype}")
    Ci = x.shape[1]
    if w.shape[1] != 27 or w.shape[2] != Ci:
        raise T2scError(-1, f"spconv shapes: w {tuple(w.shape)} does not match x {tuple(x.shape)}")
    y = out if out is not None else torch.empty((plan.n_out, Co), dtype=x.dtype, device=x.device)
    e, keep = _epilogue(Co, x.dtype, b, ln, act, residual, skip)
    # The kernel runs on the context's stream (the torch stream that was current when the cache was built), which need
    # not be the stream torch's allocator associates with these temporaries: the plan holds them until its next conv.
    plan.keep = keep
    ctx.check(ctx.lib.t2sc_subm_conv(ctx.h, plan.h, _ptr(x), _ptr(w), ctypes.byref(e), _ptr(y), _DT[x.dtype],
                                     x.shape[0], Ci, Co, _VARIANT[variant]))
    return y


def subm_conv(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], c: SpConvCache, *, ln=None, act=None,
              residual=None, skip=None, variant: str = "auto", out=None) -> torch.Tensor:
    """y = subm_conv3d(x, w, b) (src/spconv.cu:160-175): x [N,Ci], w [Co,27,Ci], b [Co] or None -> [N,Co] in
    the caller's row order.  Keyword arguments fuse what the decoder runs right after the conv:
    ``ln=(gamma, beta, eps)`` LayerNorm over Co, ``act`` in {"silu","gelu","gelu_tanh"}, ``residual`` [N,Co]
    (``add_``), ``skip=(x_parent, src, rep)`` (``k_add_skip``)."""
    if x.shape[0] != c.N:
        raise T2scError(-1, f"spconv shapes: x has {x.shape[0]} rows, cache has {c.N}")
    return _conv(c.ctx, c.plan_for(w.shape[0], w.shape[2]), x, w, b, w.shape[0], ln, act, residual, skip, variant, out)


@dataclasses.dataclass
class Level:
    """One resolution level of the decoder (src/models.h:22): coordinates, for a subdivided level the
    ``src`` map (parent*8 + slot) and the parent's cache, and its own neighbour cache ``nb``."""
    coords: torch.Tensor
    src: Optional[torch.Tensor]
    nb: SpConvCache
    parent: Optional[SpConvCache] = None
    _up_plans: Optional[dict] = None

    def up_plan_for(self, Cc: int) -> _Plan:
        """Schedule of the subdivision conv into Cc child channels: 256-row tiles, two 128-row accumulators per weight slab
        (the 8 child slots have 8 weight sets, so a slab is reused by fewer rows than in a submanifold conv; measured on
        886,752 parents -> 3,288,465 children, 128 -> 64: 2.35 ms against 2.80 ms with 128-row tiles)."""
        tr = 256
        if self._up_plans is None:
            self._up_plans = {}
        if tr not in self._up_plans:
            self._up_plans[tr] = _Plan(self.parent.ctx, self.parent.nbr, self.parent.gray, self.src, 0, tr)
        return self._up_plans[tr]

    @property
    def up_plan(self) -> _Plan:
        """The subdivision schedule made last (for inspection)."""
        return self.up_plan_for(256) if not self._up_plans else list(self._up_plans.values())[-1]


def subdivide(parent: SpConvCache, sub: torch.Tensor, want_sorted: bool = False) -> Level:
    """SDecoder::c2s (src/sdec.cu:45-57): ``sub`` [n,8] fp16/bf16 logits (kept iff > 0) or uint8 flags ->
    child coords in (parent, slot) order, ``src``, and the children's neighbour cache."""
    _chk(sub, "sub", None, 2)
    n = parent.N
    if sub.shape != (n, 8) or sub.dtype not in (torch.float16, torch.bfloat16, torch.uint8):
        raise T2scError(-1, f"sub must be [{n},8] fp16/bf16/uint8, got {tuple(sub.shape)} {sub.dtype}")
    ctx = parent.ctx
    off = torch.empty(n + 1, dtype=torch.int32, device=sub.device)
    m = ctypes.c_int64(0)
    ctx.check(ctx.lib.t2sc_subdivide_count(ctx.h, _ptr(sub), _DT[sub.dtype], n, _ptr(off), ctypes.byref(m)))
    coords = torch.empty((m.value, 4), dtype=torch.int32, device=sub.device)
    src = torch.empty(m.value, dtype=torch.int32, device=sub.device)
    if m.value:
        ctx.check(ctx.lib.t2sc_subdivide_emit(ctx.h, _ptr(sub), _DT[sub.dtype], _ptr(parent.coords), _ptr(off), n, _ptr(coords), _ptr(src)))
    nb = build_neighbors(coords, 4096, 4096, 4096, want_sorted=want_sorted)
    return Level(coords, src, nb, parent)


def subdiv_conv(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], level: Level, *, ln=None, act=None,
                variant: str = "auto", out=None) -> torch.Tensor:
    """The conv1 -> channel-to-spatial pair of the up block (src/sdec.cu:76-80) for kept children only:
    x [n,Ci] parent features, w [8*Cc,27,Ci], b [8*Cc] -> [m,Cc] with
    y[r] = conv(x, w[slot*Cc:(slot+1)*Cc])[parent], (parent, slot) = divmod(src[r], 8)."""
    if w.shape[0] % 8:
        raise T2scError(-1, "subdivision conv needs 8*Cc weight rows")
    if x.shape[0] != level.parent.N:
        raise T2scError(-1, f"spconv shapes: x has {x.shape[0]} rows, parent cache has {level.parent.N}")
    return _conv(level.parent.ctx, level.up_plan_for(w.shape[0] // 8), x, w, b, w.shape[0] // 8, ln, act, None, None, variant, out)


def gather_rows(x: torch.Tensor, src: torch.Tensor, C: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[r] = x.view(-1, C)[src[r]] (src/sdec.cu:34-37)."""
    _chk(x, "x"); _chk(src, "src", torch.int32, 1)
    ctx = context(x.device)
    y = out[:src.shape[0]] if out is not None else torch.empty((src.shape[0], C), dtype=x.dtype, device=x.device)
    ctx.check(ctx.lib.t2sc_gather_rows(ctx.h, _ptr(x), _ptr(src), src.shape[0], C, _DT[x.dtype], _ptr(y)))
    return y


def add_skip(h: torch.Tensor, x: torch.Tensor, src: torch.Tensor, rep: int) -> torch.Tensor:
    """In place h[r,c] += x[src[r]>>3, (src[r]&7)*(Cin/8) + c/rep] (src/sdec.cu:39-43)."""
    _chk(h, "h", None, 2); _chk(x, "x", h.dtype, 2); _chk(src, "src", torch.int32, 1)
    ctx = context(h.device)
    ctx.check(ctx.lib.t2sc_add_skip(ctx.h, _ptr(h), _ptr(x), _ptr(src), h.shape[0], h.shape[1], x.shape[1], rep, _DT[h.dtype]))
    return h


def row_epilogue(x: torch.Tensor, *, ln=None, act=None, residual=None, out=None) -> torch.Tensor:
    """layer_norm -> act_ -> add_ (src/ops.cu:17-113) in one pass over [n,C]."""
    _chk(x, "x", None, 2)
    ctx = context(x.device)
    y = out if out is not None else torch.empty_like(x)
    e, keep = _epilogue(x.shape[1], x.dtype, None, ln, act, residual, None)
    ctx.check(ctx.lib.t2sc_row_epilogue(ctx.h, _ptr(x), ctypes.byref(e), _ptr(y), x.shape[0], x.shape[1], _DT[x.dtype]))
    return y


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, *, ln=None, act=None, residual=None, out=None) -> torch.Tensor:
    """y = x . w^T + b (src/gemm.cu:25-64) with what the decoder's ConvNeXt block strings around its two Linear layers fused
    (src/sdec.cu:62-65): ``act`` ("silu" after the first), ``residual`` (``add_`` after the second), ``ln``.  x [n,Ci],
    w [Co,Ci], fp16 / bf16, on the conv's tcgen05 kernel."""
    _chk(x, "x", None, 2); _chk(w, "w", x.dtype, 2)
    if w.shape[1] != x.shape[1]:
        raise T2scError(-1, f"linear shapes: w {tuple(w.shape)} does not match x {tuple(x.shape)}")
    ctx = context(x.device)
    Co = w.shape[0]
    y = out if out is not None else torch.empty((x.shape[0], Co), dtype=x.dtype, device=x.device)
    e, keep = _epilogue(Co, x.dtype, b, ln, act, residual, None)
    ctx.check(ctx.lib.t2sc_linear(ctx.h, _ptr(x), _ptr(w), ctypes.byref(e), _ptr(y), _DT[x.dtype], x.shape[0], x.shape[1], Co))
    ctx.keep = keep           # alive until this context's next linear (the kernel runs on the context's stream)
    return y


def layer_norm(x, w, b, eps):
    return row_epilogue(x, ln=(w, b, eps))


def act_(x, kind):
    return row_epilogue(x, act=kind, out=x)


def add_(x, y):
    return row_epilogue(x, residual=y, out=x)


def subm_conv_host(coords, x, w, b, W: int = 4096, H: int = 4096, D: int = 4096, device=None, out=None):
    """The whole operator on HOST tensors (pinned or pageable): copies in, neighbour map, conv, copy out,
    synchronise - what apps/parity.cu:148-167 times.  Returns a host tensor."""
    ctx = context(device)
    for t, nme in ((coords, "coords"), (x, "x"), (w, "w")):
        if t.is_cuda or not t.is_contiguous():
            raise T2scError(-1, f"{nme} must be a contiguous host tensor")
    n, Ci, Co = x.shape[0], x.shape[1], w.shape[0]
    y = out if out is not None else torch.empty((n, Co), dtype=x.dtype, pin_memory=True)
    if b is not None:
        b = b.to(x.dtype).contiguous()
    ctx.check(ctx.lib.t2sc_subm_conv_host(ctx.h, _ptr(coords), n, W, H, D, _ptr(x), _ptr(w), _ptr(b), _ptr(y),
                                          _DT[x.dtype], Ci, Co))
    return y
