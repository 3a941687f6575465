"""The sharded workload of bench.py (``--workload cfg5``): ONE ~8.6 M-voxel shell in a 2048^3 grid, C = 128, bf16,
4 stacked submanifold convs, rows cut into equal-count Morton ranges over the ranks, one-voxel halo exchanged
with one NCCL all-to-all per layer.  Strong scaling: the scene is the same at every N.

One step = the 4 layers (halo exchange + conv each).  The neighbour map, halo plan and conv schedule are built
once before the timed region and reported separately (`setup_ms`), as a decoder level reuses one map for all of
its blocks.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist


def run(args, rank, world, local_rank, METRIC, peaks, ClockSampler, visible_gpu_index):
    import trellis2_cuda_b200 as sp
    from trellis2_cuda_b200 import scenes, sharding

    dev = torch.device("cuda", local_rank)
    C, layers, td = 128, args.layers, torch.bfloat16
    # rank 0 builds the scene, everyone receives the same coordinates
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
        dist.broadcast(coords, 0)
    ctx = sp.context(dev)
    starts = sharding.partition(N, world)
    lo, hi = starts[rank], starts[rank + 1]

    p2p = args.halo == "p2p" and world > 1
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nbr_g, gray = sp.build_neighbors_range(coords, lo, hi)
    plan = sharding.build_halo_plan(nbr_g, rank, world, starts)
    if p2p:      # the conv gathers halo rows from the peers' arrays itself: the map names (owner, row), nothing is copied
        cache = sp.cache_from_map(coords[lo:hi], sharding.peer_map(nbr_g, starts).contiguous(), gray)
    else:
        cache = sp.cache_from_map(coords[lo:hi], plan.nbr_local.contiguous(), gray)
    del nbr_g
    st = cache.plan_for(C, C).stats()
    torch.cuda.synchronize()
    setup_ms = (time.perf_counter() - t0) * 1e3

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    if p2p:
        import torch.distributed._symmetric_memory as symm
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # plain peer loads only
        rows_max = max(starts[r + 1] - starts[r] for r in range(world))
        xa = symm.empty((rows_max, C), dtype=td, device=dev)
        xb = symm.empty((rows_max, C), dtype=td, device=dev)
        ha, hb = symm.rendezvous(xa, dist.group.WORLD), symm.rendezvous(xb, dist.group.WORLD)
        ptrs = {xa.data_ptr(): [int(p) for p in ha.buffer_ptrs], xb.data_ptr(): [int(p) for p in hb.buffer_ptrs]}
        hdl = {xa.data_ptr(): ha, xb.data_ptr(): hb}
    else:
        xa = torch.zeros((plan.n_local, C), dtype=td, device=dev)
        xb = torch.zeros((plan.n_local, C), dtype=td, device=dev)
    x0 = torch.randn((plan.n_own, C), generator=g, device=dev).to(td)
    ws = [torch.from_numpy(scenes.kaiming_uniform_weight(C, C, 100 + l)).to(dev).to(td) for l in range(layers)]
    pack = lambda x_own, idx: sp.gather_rows(x_own, idx, C)

    def step(timers=None):
        a, b = xa, xb
        a[:plan.n_own].copy_(x0)
        for l in range(layers):
            if timers:
                timers[0][l].record()
            if p2p:
                hdl[a.data_ptr()].barrier(channel=l % 2)       # every rank has written the array this layer reads
            else:
                sharding.exchange_halo(plan, a, pack)
            if timers:
                timers[1][l].record()
            if p2p:
                sp.subm_conv_peers(ptrs[a.data_ptr()], rank, td, C, ws[l], None, cache, out=b[:plan.n_own])
            else:
                sp.subm_conv_local(a, ws[l], None, cache, out=b[:plan.n_own])
            a, b = b, a
        if p2p:
            hdl[a.data_ptr()].barrier(channel=0)               # nobody overwrites an array a peer may still be reading
        return a

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(visible_gpu_index(local_rank))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    t_reg0 = time.perf_counter()
    l0 = ctx.launch_count()
    step_ms, exch_ms = [], []
    for _ in range(args.steps):
        tm = ([ev() for _ in range(layers)], [ev() for _ in range(layers)])
        s, e = ev(), ev()
        s.record()
        step(tm)
        e.record()
        torch.cuda.synchronize()
        step_ms.append(s.elapsed_time(e))
        exch_ms.append(sum(tm[0][l].elapsed_time(tm[1][l]) for l in range(layers)))
    launches = ctx.launch_count() - l0
    t_reg1 = time.perf_counter()
    ctx.device_status()

    # end to end: owned features from pinned host memory each step, final features back to the host
    x_h = x0.cpu().pin_memory()
    y_h = torch.empty_like(x_h).pin_memory()
    e2e = []
    for i in range(5):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        x0.copy_(x_h, non_blocking=True)
        out = step()
        y_h.copy_(out[:plan.n_own], non_blocking=True)
        torch.cuda.synchronize()
        if i >= 2:
            e2e.append((time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop(t_reg0, t_reg1) if rank == 0 else None

    T = st["active_taps"]
    vals = torch.tensor([sum(step_ms), sum(exch_ms), sum(e2e) / len(e2e), setup_ms], dtype=torch.float64, device=dev)
    sums = torch.tensor([float(T), float(plan.n_halo), float(st["computed_taps"])], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    if rank != 0:
        return
    pk, pk_src = peaks()
    ms = vals[0].item() / args.steps
    T_all = sums[0].item()
    flops = 2.0 * T_all * C * C * layers
    value = flops / (ms * 1e-3) / 1e12
    conv_ms = (vals[0].item() - vals[1].item()) / args.steps
    es = 2
    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"cfg5: 2048^3 shell of 12 spheres/tori, {layers} stacked 128->128 submanifold convs, equal-count Morton ranges, "
                                   + ("halo rows read from peer memory by the conv kernel (P2P), one device barrier per layer" if p2p else "one-voxel halo by NCCL all-to-all per layer"), "voxels": N, "Cin": C, "Cout": C, "active_taps": int(T_all),
                       "computed_taps": int(sums[2].item()), "halo_rows_total": int(sums[1].item()), "step": f"{layers} x (halo exchange + conv)",
                       "l2": "inputs larger than L2 (per-rank features >= 275 MB)"},
            "voxels_per_s": N * layers / (ms * 1e-3), "exchange_ms_per_step": vals[1].item() / args.steps, "setup_ms": vals[3].item(),
            "halo_bytes_per_layer": int(sums[1].item()) * C * es,
            "roofline": {"bound": "tensor", "achieved": flops / world / (conv_ms * 1e-3) / 1e12, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": flops / world / (conv_ms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"], "traffic": None,
                         "peak_source": f"{pk_src} cuBLAS bf16 sustained (kernel timed inside a multi-ms step)", "kernel": "k_conv_umma", "per": "GPU"},
            "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": flops / (vals[2].item() * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": N * C * es, "d2h_bytes_per_step": N * C * es,
                    "ms_per_step": vals[2].item(), "path": "owned features from pinned host memory in, 4 layers, final features to pinned host memory"}}
    print(json.dumps(line), flush=True)
