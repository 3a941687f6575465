"""The sharded workload of bench.py: ONE ~8.6 M-voxel shell in a 2048^3 grid, C = 128, bf16, 4 stacked submanifold
convs, rows cut into equal-count Morton ranges over the ranks, one-voxel halo every layer.  Strong scaling: the scene
is the same at every N.

One step = the 4 layers (halo exchange + conv each).  Per layer the rank's tiles are run in two parts: the interior
tiles (no tap reads a halo row) while the halo rows are in flight, the boundary tiles after they have landed.

  * ``--halo nccl``: pack (gather kernel) -> one NCCL all-to-all of feature rows on the communication stream while the
    interior tiles run -> boundary tiles.
  * ``--halo p2p``: the feature arrays live in symmetric memory; interior tiles run the ordinary kernel, boundary tiles the
    peer-memory kernel whose gather reads halo rows straight from the owners' arrays over NVLink.  Per layer the ranks
    meet at one bounded device-side flag barrier (plain peer stores and loads) so that nobody reads an array its owner is
    still writing.

The neighbour map, halo plan and conv schedule are built once before the timed region and reported separately
(`setup_ms`, split into its parts), as a decoder level reuses one map for all of its blocks.
"""
from __future__ import annotations

import os
import time

import torch
import torch.distributed as dist


def measure(args, rank, world, local_rank, peaks, ClockSampler, visible_gpu_index, steps=None, warmup=None, halo=None,
            single_gpu_steps=0, with_e2e=True):
    """Runs the sharded scene on `world` ranks and returns the result block on rank 0 (None elsewhere).
    single_gpu_steps > 0: rank 0 afterwards runs the WHOLE scene alone for that many steps, so that the block carries the
    one-GPU time of the same scene measured in the same run."""
    import trellis2_cuda_b200 as sp
    from trellis2_cuda_b200 import scenes, sharding

    steps = steps or args.steps
    warmup = warmup if warmup is not None else args.warmup
    halo = halo or args.halo
    dev = torch.device("cuda", local_rank)
    C, layers, td = 128, args.layers, torch.bfloat16
    sync = lambda: torch.cuda.synchronize(dev)
    # rank 0 builds the scene, everyone receives the same coordinates
    t_scene = time.perf_counter()
    if rank == 0:
        coords = torch.from_numpy(scenes.config5_shell(0)).to(dev)
        n_t = torch.tensor([coords.shape[0]], dtype=torch.int64, device=dev)
    else:
        n_t = torch.zeros(1, dtype=torch.int64, device=dev)
    if world > 1:
        dist.broadcast(n_t, 0)
    N = int(n_t.item())
    if rank != 0:
        coords = torch.empty((N, 4), dtype=torch.int32, device=dev)
    if world > 1:
        dist.broadcast(coords, 0)          # also the first collective: communicator set-up lands here, not in setup_ms
        warm = torch.zeros(world, dtype=torch.int64, device=dev)
        dist.all_to_all_single(torch.empty_like(warm), warm)       # ... and the peer-to-peer connections of the first all-to-all
    sync()
    scene_ms = (time.perf_counter() - t_scene) * 1e3
    ctx = sp.context(dev)
    starts = sharding.partition(N, world)
    lo, hi = starts[rank], starts[rank + 1]
    p2p = halo == "p2p" and world > 1

    setup = {}
    t0 = time.perf_counter()
    nbr_g, gray = sp.build_neighbors_range(coords, lo, hi)
    sync(); setup["map_ms"] = (time.perf_counter() - t0) * 1e3
    t0 = time.perf_counter()
    plan = sharding.build_halo_plan(nbr_g, rank, world, starts)
    sync(); setup["halo_plan_ms"] = (time.perf_counter() - t0) * 1e3
    t0 = time.perf_counter()
    nbr_local = plan.nbr_local.contiguous()
    cache = sp.cache_from_map(coords[lo:hi], nbr_local, gray)
    split = cache.split_plan_for(C, C, plan.n_own) if world > 1 else None
    if split is not None:
        split.check(plan.n_local)        # the plan's map copy is checked against owned + halo rows now: both parts find it ready, whichever stream runs first
    peer_nbr = sharding.peer_map(nbr_g, starts).contiguous() if p2p else None
    del nbr_g
    st = (split or cache.plan_for(C, C)).stats()
    parts = split.parts() if split is not None else {"interior_tiles": st["tiles"], "boundary_tiles": 0}
    sync(); setup["schedule_ms"] = (time.perf_counter() - t0) * 1e3

    g = torch.Generator(device=dev).manual_seed(1234)
    x_full = torch.randn((N, C), generator=g, device=dev).to(td)       # the same on every rank: the one-GPU check needs the whole input
    if p2p:
        import torch.distributed._symmetric_memory as symm
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # plain peer loads only
        rows_max = max(starts[r + 1] - starts[r] for r in range(world))
        xa = symm.empty((rows_max, C), dtype=td, device=dev)
        xb = symm.empty((rows_max, C), dtype=td, device=dev)
        flags = symm.empty((64,), dtype=torch.int32, device=dev)
        flags.zero_()
        ha, hb, hf = symm.rendezvous(xa, dist.group.WORLD), symm.rendezvous(xb, dist.group.WORLD), symm.rendezvous(flags, dist.group.WORLD)
        ptrs = {xa.data_ptr(): [int(p) for p in ha.buffer_ptrs], xb.data_ptr(): [int(p) for p in hb.buffer_ptrs]}
        flag_ptrs = [int(p) for p in hf.buffer_ptrs]
        rows_of = [starts[r + 1] - starts[r] for r in range(world)]
        dist.barrier()                                  # every rank has zeroed its flags before anyone signals
        sync()
    else:
        xa = torch.zeros((plan.n_local, C), dtype=td, device=dev)
        xb = torch.zeros((plan.n_local, C), dtype=td, device=dev)
    x0 = x_full[lo:hi].clone()
    if rank != 0:
        del x_full
    ws = [torch.from_numpy(scenes.kaiming_uniform_weight(C, C, 100 + l)).to(dev).to(td) for l in range(layers)]
    send_buf = torch.empty((max(int(plan.send_idx.numel()), 1), C), dtype=td, device=dev)
    epoch = [0]
    # The boundary tiles run on a side stream that waits for the halo only: they write rows the interior tiles do not
    # touch, so they start on the first SMs the interior kernel leaves instead of behind its last tile.
    main = torch.cuda.current_stream(dev)
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        ctx_side = sp.context(dev)
    halo_ready = torch.cuda.Event()

    def step(timers=None):
        a, b = xa, xb
        a[:plan.n_own].copy_(x0)
        for l in range(layers):
            if timers:
                timers[0][l].record()
            if world == 1:
                sp.subm_conv_local(a, ws[l], None, cache, out=b[:plan.n_own])
            elif p2p:
                # every rank has written the array this layer reads (and is done reading the one it overwrites)
                epoch[0] += 1
                sp.peer_barrier(ctx, flag_ptrs, rank, epoch[0])
                if timers:
                    timers[1][l].record()
                halo_ready.record(main)
                sp.subm_conv_split(a, ws[l], None, cache, split, "interior", out=b[:plan.n_own], n_local=plan.n_local)
                with torch.cuda.stream(side):
                    side.wait_event(halo_ready)
                    sp.subm_conv_peers(ptrs[a.data_ptr()], rows_of, rank, td, C, ws[l], None, cache, out=b[:plan.n_own],
                                       plan=split, part="boundary", peer_nbr=peer_nbr, ctx=ctx_side)
                main.wait_stream(side)
            else:
                work = sharding.exchange_halo_async(plan, a, lambda xo, idx: sp.gather_rows(xo, idx, C, out=send_buf))
                if timers:
                    timers[1][l].record()
                sp.subm_conv_split(a, ws[l], None, cache, split, "interior", out=b[:plan.n_own])     # while the halo rows travel
                with torch.cuda.stream(side):
                    if work is not None:
                        work.wait()                     # the side stream waits for the all-to-all, not the host
                    else:
                        side.wait_stream(main)
                    sp.subm_conv_split(a, ws[l], None, cache, split, "boundary", out=b[:plan.n_own], ctx=ctx_side)
                main.wait_stream(side)
            a, b = b, a
        if p2p:
            epoch[0] += 1
            sp.peer_barrier(ctx, flag_ptrs, rank, epoch[0])       # nobody overwrites an array a peer may still be reading
        return a

    out = step()
    ctx.device_status()
    ctx_side.device_status()
    for _ in range(max(warmup - 1, 0)):
        step()
    sync()
    sampler = ClockSampler(visible_gpu_index(local_rank))
    if rank == 0:
        sampler.start()
        sampler.wait_first_sample()
    if world > 1:
        dist.barrier()
    sync()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    t_reg0 = time.perf_counter()
    l0, l0_side = ctx.launch_count(), ctx_side.launch_count()
    step_ms, exch_ms = [], []
    for _ in range(steps):
        tm = ([ev() for _ in range(layers)], [ev() for _ in range(layers)])
        s, e = ev(), ev()
        s.record()
        step(tm)
        e.record()
        sync()
        step_ms.append(s.elapsed_time(e))
        exch_ms.append(sum(tm[0][l].elapsed_time(tm[1][l]) for l in range(layers)) if world > 1 else 0.0)
    launches = ctx.launch_count() - l0 + ctx_side.launch_count() - l0_side
    t_reg1 = time.perf_counter()
    ctx.device_status()
    ctx_side.device_status()

    e2e = []
    if with_e2e:
        # end to end: owned features from pinned host memory each step, final features back to the host
        x_h = x0.cpu().pin_memory()
        y_h = torch.empty_like(x_h).pin_memory()
        for i in range(5):
            if world > 1:
                dist.barrier()
            sync()
            t0 = time.perf_counter()
            x0.copy_(x_h, non_blocking=True)
            out = step()
            y_h.copy_(out[:plan.n_own], non_blocking=True)
            sync()
            if i >= 2:
                e2e.append((time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop(t_reg0, t_reg1) if rank == 0 else None

    T = st["active_taps"]
    vals = torch.tensor([sum(step_ms), sum(exch_ms), (sum(e2e) / len(e2e)) if e2e else 0.0, setup["map_ms"], setup["halo_plan_ms"],
                         setup["schedule_ms"], float(parts["boundary_tiles"])], dtype=torch.float64, device=dev)
    sums = torch.tensor([float(T), float(plan.n_halo), float(st["computed_taps"]), float(parts["interior_tiles"] + parts["boundary_tiles"]),
                         float(parts["boundary_tiles"])], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)

    single, verified = None, None
    if world > 1:
        # The same scene on ONE GPU, on rank 0 in this run (the other ranks wait at the barrier below): its time, and the
        # check that the sharded result equals it bit for bit (every output row sums its taps in the same order however the
        # rows are tiled or sharded).
        rows_max = max(starts[r + 1] - starts[r] for r in range(world))
        mine = torch.zeros((rows_max, C), dtype=td, device=dev)
        mine[:plan.n_own].copy_(step()[:plan.n_own])
        parts_out = [torch.empty_like(mine) for _ in range(world)] if rank == 0 else None
        dist.gather(mine, parts_out, dst=0)
        del xa, xb, mine
        if rank == 0:
            full = sp.build_neighbors(coords, want_sorted=False)
            xa1, xb1 = x_full.clone(), torch.empty_like(x_full)
            ms1 = []
            for i in range(max(single_gpu_steps, 5) + 3):
                s, e = ev(), ev()
                s.record()
                a, b = xa1, xb1
                a.copy_(x_full)
                for l in range(layers):
                    sp.subm_conv(a, ws[l], None, full, out=b)
                    a, b = b, a
                e.record()
                sync()
                if i >= 3:
                    ms1.append(s.elapsed_time(e))
            single = sum(ms1) / len(ms1)
            ctx.device_status()
            verified = all(torch.equal(parts_out[r][:starts[r + 1] - starts[r]], a[starts[r]:starts[r + 1]]) for r in range(world))
            del full, xa1, xb1, parts_out
        dist.barrier()
    if rank != 0:
        return None
    pk, pk_src = peaks()
    ms = vals[0].item() / steps
    T_all = sums[0].item()
    flops = 2.0 * T_all * C * C * layers
    value = flops / (ms * 1e-3) / 1e12
    es = 2
    block = {
        "workload": f"cfg5: 2048^3 shell of 12 spheres/tori, {layers} stacked 128->128 submanifold convs, equal-count Morton ranges, "
                    + ("one GPU" if world == 1 else
                       ("interior tiles by the ordinary kernel, boundary tiles gather their halo rows from peer memory (P2P), one bounded flag barrier per layer"
                        if p2p else "interior tiles run while one NCCL all-to-all moves the one-voxel halo, boundary tiles after it")),
        "n_gpus": world, "halo": "none" if world == 1 else halo, "scaling": "strong", "voxels": N, "Cin": C, "Cout": C, "layers": layers,
        "active_taps": int(T_all), "computed_taps": int(sums[2].item()),
        "ms_per_step": ms, "tflops": value, "voxels_per_s": N * layers / (ms * 1e-3),
        "exchange_ms_per_step": vals[1].item() / steps,
        "exchange_note": "time from a layer's start to the launch of its interior tiles on the slowest rank (pack + enqueue of the all-to-all, or the flag barrier); the transfer itself runs beside the interior tiles",
        "halo_rows_total": int(sums[1].item()), "halo_bytes_per_layer": int(sums[1].item()) * C * es,
        "tiles_total": int(sums[3].item()), "boundary_tiles_total": int(sums[4].item()), "boundary_tiles_max_rank": int(vals[6].item()),
        "setup_ms": {"neighbour_map": vals[3].item(), "halo_plan": vals[4].item(), "schedule": vals[5].item(),
                     "scene_and_first_collective": scene_ms},
        "per_gpu_tflops": value / world, "per_gpu_frac_of_sustained_peak": value / world / pk["bf16_tflops_sustained"],
        "peak_source": f"{pk_src} cuBLAS bf16 sustained",
        "clocks": clocks, "gpu_launches": launches,
    }
    if single is not None:
        block["single_gpu_ms_per_step"] = single
        block["speedup_vs_single_gpu"] = single / ms
        block["equals_single_gpu_result_bit_for_bit"] = verified
    if e2e:
        block["e2e"] = {"value": flops / (vals[2].item() * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": N * C * es, "d2h_bytes_per_step": N * C * es,
                        "ms_per_step": vals[2].item(), "path": "owned features from pinned host memory in, 4 layers, final features to pinned host memory"}
    return block


def run(args, rank, world, local_rank, METRIC, peaks, ClockSampler, visible_gpu_index):
    """`bench.py --workload cfg5`: the sharded scene as the whole JSON line."""
    import json
    b = measure(args, rank, world, local_rank, peaks, ClockSampler, visible_gpu_index)
    if rank != 0:
        return
    pk, pk_src = peaks()
    line = {"metric": METRIC, "value": b["tflops"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": b["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": b["workload"], "voxels": b["voxels"], "Cin": 128, "Cout": 128, "active_taps": b["active_taps"],
                       "computed_taps": b["computed_taps"], "halo_rows_total": b["halo_rows_total"], "step": f"{b['layers']} x (halo exchange + conv)",
                       "l2": "inputs larger than L2 (per-rank features >= 275 MB)"},
            "voxels_per_s": b["voxels_per_s"], "exchange_ms_per_step": b["exchange_ms_per_step"], "setup_ms": b["setup_ms"],
            "halo_bytes_per_layer": b["halo_bytes_per_layer"], "boundary_tiles_total": b["boundary_tiles_total"], "tiles_total": b["tiles_total"],
            "roofline": {"bound": "tensor", "achieved": b["per_gpu_tflops"], "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": b["per_gpu_frac_of_sustained_peak"], "traffic": None,
                         "peak_source": f"{pk_src} cuBLAS bf16 sustained (kernel timed inside a multi-ms step)", "kernel": "k_conv_umma", "per": "GPU"},
            "clocks": b["clocks"], "gpu_launches": b["gpu_launches"], "e2e": b.get("e2e")}
    for k in ("single_gpu_ms_per_step", "speedup_vs_single_gpu", "equals_single_gpu_result_bit_for_bit"):
        if k in b:
            line[k] = b[k]
    print(json.dumps(line), flush=True)
