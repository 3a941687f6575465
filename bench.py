#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg1|cfg2|cfg3|cfg4|cfg5]

One step = one pass of the operator as the reference's own harness times it (apps/parity.cu:157-160 of
trellis2-cuda): build the neighbour map of the scene, then run the submanifold conv.  The default workload (cfg2) is the
mid-decoder configuration: a ~218k-voxel shell in a 256^3 grid, Cin = Cout = 256, bf16 features and weights, fp32
accumulation, seeded synthetic data.  Other workloads:

  cfg1  14,534-voxel sphere shell, 64 -> 64, fp32 (CUDA-core kernel)
  cfg3  886,752 parents -> 3,288,465 children, fp16: maps, the 128 -> 64 subdivision conv over kept children, the 64 -> 64
        conv on the children; one table row per kernel
  cfg4  the decoder-like stack 1024 -> 512 -> 256 -> 128 -> 64 over a 64^3 ... 1024^3 pyramid; one table row per level
  cfg5  ONE 8.6M-voxel scene sharded over the ranks by Morton range, 4 stacked layers, halo exchange every layer

With N > 1 ranks (torchrun) every rank runs the default operator on the same scene (independent replicas: no data-path
collective, weak scaling) and the line carries a `sharded` block with the cfg5 measurement of that run.

Rank 0 prints one JSON line.  ``value`` is effective TFLOP/s (2 * active taps * Cin * Cout per conv; taps whose
neighbour is absent are not counted) over the whole step, all ranks together.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # peer arrays are read with plain loads; no multicast object is bound
if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":      # keeps NCCL's banner off stdout: rank 0 prints one JSON line
    os.environ["NCCL_DEBUG"] = "WARN"

import numpy as np  # noqa: E402
import torch  # noqa: E402

E2E_DEPTH = 3          # complete host-buffer calls kept in flight by the end-to-end leg
METRIC = "sparse-conv effective TFLOP/s (active taps only)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
TD = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {k: float(d.get(k, FALLBACK_PEAKS[k])) for k in FALLBACK_PEAKS}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def host_cores():
    """Threads this process may use: the smaller of the visible CPUs and the cgroup CPU quota (they can differ widely in a
    container: the reference's own environment saw 192 CPUs with a quota of 23, docs/blog.md:81-82)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    quota = None
    try:
        q, period = open("/sys/fs/cgroup/cpu.max").read().split()[:2]
        if q != "max":
            quota = float(q) / float(period)
    except (OSError, ValueError):
        pass
    use = max(1, min(n, int(quota + 0.5))) if quota else n
    return {"nproc": os.cpu_count() or 1, "affinity": n, "cgroup_quota": quota, "used": use}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def wait_first_sample(self, limit_s=5.0):
        """nvidia-smi takes a second or so to deliver its first row; a short timed region must not start before it."""
        t0 = time.perf_counter()
        while self.proc and not self.rows and time.perf_counter() - t0 < limit_s:
            time.sleep(0.02)

    def summary(self, t0=None, t1=None):
        rows = [r for t, r in self.rows if (t0 is None or t >= t0) and (t1 is None or t <= t1 + 0.05)]
        sm = [float(r[0]) for r in rows if len(r) >= 8 and r[0].replace(".", "").isdigit()]
        pw = [float(r[2]) for r in rows if len(r) >= 8 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in rows:
            if len(r) >= 8:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        smax = [float(r[1]) for r in rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w": statistics.median(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self, t0=None, t1=None):
        """Summary of the samples taken between perf_counter times t0 and t1 (the timed region)."""
        if self.proc:
            self.proc.terminate()
        return self.summary(t0, t1)


def visible_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v for v in vis.split(",") if v != ""]
        if local_rank < len(ids) and ids[local_rank].isdigit():
            return int(ids[local_rank])
    return local_rank


def alg_bytes(n_in, n_out, Ci, Co, w_rows, es):
    """Algorithmic bytes of one conv: features in and out once, weights once, 108 B of neighbour map per output row."""
    return n_in * Ci * es + n_out * Co * es + 27 * Ci * w_rows * es + n_out * 27 * 4


# ------------------------------------------------------------------------------------------ workloads (single conv)
def make_workload(name, seed):
    from trellis2_cuda_b200 import scenes
    if name == "cfg1":
        return dict(coords=scenes.config1_sphere(seed), Ci=64, Co=64, dtype="f32", desc="cfg1: 64^3 sphere shell, 64->64, fp32")
    if name in ("cfg2", "cfg5"):
        return dict(coords=scenes.config2_shell(seed), Ci=256, Co=256, dtype="bf16",
                    desc="cfg2: 256^3 shell of 6 spheres/tori, 256->256 submanifold 3x3x3, bf16 in / fp32 accumulate")
    if name == "cfg3":
        parents, flags = scenes.config3_pair(seed)
        child = scenes.subdivide_numpy(parents, flags)[0]
        return dict(coords=child, Ci=64, Co=64, dtype="f16", desc="cfg3 (second half): 1024^3 shell, 64->64 submanifold, fp16")
    if name == "cfg4":
        lv = scenes.config4_levels(seed, levels=3)
        return dict(coords=lv[2][0], Ci=256, Co=256, dtype="bf16", desc="cfg4 (level 2 of the stack): 256^3 shell, 256->256 submanifold, bf16")
    raise ValueError(name)


def cpu_sample(wl, rows, threads, reps=1):
    """Times the CPU oracle (scalar gather-GEMM-scatter) on `rows` output rows of the workload."""
    import oracle
    coords, Ci, Co = wl["coords"], wl["Ci"], wl["Co"]
    n = coords.shape[0]
    rng = np.random.default_rng(1)
    x = oracle.round_to(rng.standard_normal((n, Ci), dtype=np.float32), wl["dtype"])
    from trellis2_cuda_b200 import scenes
    w = oracle.round_to(scenes.kaiming_uniform_weight(Co, Ci, 1), wl["dtype"])
    oracle.set_threads(threads)
    t0 = time.perf_counter()
    nbr = oracle.build_neighbors(coords, want_sorted=True)[0]
    t_nbr = time.perf_counter() - t0
    sel = np.arange(min(rows, n), dtype=np.int32)
    taps = int((nbr[sel] != oracle.EMPTY).sum())
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        oracle.subm_conv(x, w, None, nbr, nrow=sel)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    # the map is built for the whole scene; charge the sample its share of it
    t = best + t_nbr * len(sel) / n
    return {"tflops": 2.0 * taps * Ci * Co / t / 1e12, "seconds": t, "conv_seconds": best, "nbr_seconds_full": t_nbr,
            "rows": int(len(sel)), "taps": taps}


def cpu_baseline_block(wl, full=True):
    """The CPU restatement on this host: all usable cores, and one thread (the "scalar" baseline)."""
    cores = host_cores()
    n, Ci = wl["coords"].shape[0], wl["Ci"]
    rows_all = 16384 if Ci >= 256 else 65536
    r = cpu_sample(wl, rows_all, cores["used"])
    out = {"value": r["tflops"], "unit": "TFLOP/s", "cores": cores["used"], "kind": "port",
           "sample": f"first {r['rows']} of {n} output rows ({r['taps']} active taps), full-scene neighbour map charged pro rata; {r['seconds']:.2f} s wall",
           "host": cores}
    if full:
        r1 = cpu_sample(wl, max(rows_all // 16, 256), 1)
        out["single_thread"] = {"value": r1["tflops"], "unit": "TFLOP/s", "cores": 1,
                                "sample": f"first {r1['rows']} output rows ({r1['taps']} active taps); {r1['seconds']:.2f} s wall"}
    return out


# ------------------------------------------------------------------------------------------ reference arm
def run_reference(args, rank, world):
    if rank != 0:
        return
    wl = make_workload(args.workload, 0)
    cores = host_cores()
    threads = cores["used"]
    # a bounded sample per step (about 0.15 s on 16 cores) so that any --steps the caller passes ends within minutes
    rows = 4096 if wl["Ci"] >= 256 else 32768
    times, res = [], None
    for i in range(args.warmup + args.steps):
        res = cpu_sample(wl, rows, threads)
        if i >= args.warmup:
            times.append(res["seconds"])
    t = sum(times) / len(times)
    v = 2.0 * res["taps"] * wl["Ci"] * wl["Co"] / t / 1e12
    sample = f"first {res['rows']} of {wl['coords'].shape[0]} output rows of the same scene ({res['taps']} active taps) per step, full-scene neighbour map charged pro rata"
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": {"workload": wl["desc"], "voxels": int(wl["coords"].shape[0]), "Cin": wl["Ci"], "Cout": wl["Co"]},
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample, "host": cores},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference has no CPU implementation of this path; this is the CPU restatement of its algorithm (oracle/oracle.c, OpenMP over output rows, scalar C)"}
    print(json.dumps(line), flush=True)


def gpu_reference_block(wl, our_conv_ms, our_map_ms):
    """The reference's own CUDA path (src/spconv.cu: build_neighbors + k_spconv, mma.sync, compiled unchanged for sm_100a
    into oracle/_ref/libt2ref.so) on the same scene with features and weights cast to fp16, timed with its own cudaEvent
    Timer the way apps/parity.cu:157-160 does.  A second GPU baseline; None when that library was not built."""
    from oracle import ref
    if not ref.available(False):
        return {"unavailable": "oracle/_ref/libt2ref.so was not built (no checkout of the reference at build time)"}
    from trellis2_cuda_b200 import scenes
    coords, Ci, Co = wl["coords"], wl["Ci"], wl["Co"]
    n = coords.shape[0]
    x = np.random.default_rng(1).standard_normal((n, Ci), dtype=np.float32).astype(np.float16)
    w = scenes.kaiming_uniform_weight(Co, Ci, 1).astype(np.float16)
    _, conv_ms, nbr_ms = ref.subm_conv(coords, x, w, None, reps=10)
    T = wl.get("active_taps")
    out = {"kernel": "k_spconv<2> (mma.sync m16n8k16, B1=128, BK=64, S=1: the reference's default on a device without an autotune section)",
           "dtype": "f16", "conv_ms": conv_ms, "build_neighbors_ms": nbr_ms, "reps": 10,
           "speedup_conv": conv_ms / our_conv_ms, "speedup_build_neighbors_vs_map_and_plan": nbr_ms / our_map_ms if our_map_ms else None}
    if T:
        out["tflops"] = 2.0 * T * Ci * Co / (conv_ms * 1e-3) / 1e12
    return out


# ------------------------------------------------------------------------------------------ our arm: one conv per step
def run_single_conv(args, rank, world, local_rank, dev):
    import torch.distributed as dist
    import trellis2_cuda_b200 as sp
    from trellis2_cuda_b200 import scenes

    wl = make_workload(args.workload, 0)               # the same scene on every rank
    if args.channels:                                  # the same geometry at another width (the narrow-layer rows of the result tables)
        wl.update(Ci=args.channels, Co=args.channels, desc=wl["desc"] + f" [geometry only: run at {args.channels}->{args.channels} channels]")
    td = TD[wl["dtype"]]
    coords_h = torch.from_numpy(wl["coords"]).pin_memory()
    n, Ci, Co = coords_h.shape[0], wl["Ci"], wl["Co"]
    g = torch.Generator().manual_seed(rank)
    x_h = torch.randn(n, Ci, generator=g).to(td).pin_memory()
    w_h = torch.from_numpy(scenes.kaiming_uniform_weight(Co, Ci, 1)).to(td).pin_memory()
    y_h = torch.empty(n, Co, dtype=td).pin_memory()
    coords, x, w = coords_h.to(dev), x_h.to(dev), w_h.to(dev)
    ctx = sp.context(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    es = x.element_size()

    def step(record=None):
        cache = sp.build_neighbors(coords, want_sorted=False)
        cache.plan_for(Co, Ci).check(n)                   # the schedule this conv will use, its map copy checked against the n feature rows
        if record:
            record[0].record()
        y = sp.subm_conv(x, w, None, cache)
        if record:
            record[1].record()
        return cache, y

    cache, y = step()
    st = cache.plan_for(Co, Ci).stats()
    T = st["active_taps"]
    wl["active_taps"] = T
    flops = 2.0 * T * Ci * Co
    ev = lambda: torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(visible_gpu_index(local_rank))
    if rank == 0:
        sampler.start()                                 # nvidia-smi needs a moment to start: launch it before the warm-up
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.wait_first_sample()
    if world > 1:
        dist.barrier()
    t_region0 = time.perf_counter()
    l0 = ctx.launch_count()
    step_ms, conv_ms = [], []
    for _ in range(args.steps):
        flush.fill_(1)                                  # evict the previous step's data from the 126 MB L2 (not timed)
        a, b, c0, c1 = ev(), ev(), ev(), ev()
        a.record()
        step((c0, c1))
        b.record()
        torch.cuda.synchronize()
        step_ms.append(a.elapsed_time(b)); conv_ms.append(c0.elapsed_time(c1))
    launches = ctx.launch_count() - l0
    t_region1 = time.perf_counter()
    ctx.device_status()
    clocks = sampler.summary(t_region0, t_region1) if rank == 0 else None

    # sustained leg: the conv back to back for >= 2 s (no flush, no map build), clocks sampled meanwhile
    sustained = None
    if not args.profile and wl["dtype"] != "f32":
        torch.cuda.synchronize()
        reps = max(50, int(2200.0 / max(min(conv_ms), 1e-3)))
        t_s0 = time.perf_counter()
        a, b = ev(), ev()
        a.record()
        for _ in range(reps):
            sp.subm_conv(x, w, None, cache, out=y)
        b.record()
        torch.cuda.synchronize()
        t_s1 = time.perf_counter()
        sus_ms = a.elapsed_time(b) / reps
        sustained = {"conv_ms": sus_ms, "reps": reps, "seconds": t_s1 - t_s0, "tflops": flops / (sus_ms * 1e-3) / 1e12,
                     "clocks": sampler.summary(t_s0 + 0.3, t_s1) if rank == 0 else None}
        ctx.device_status()

    # end to end through the host-buffer entry point: H2D of coords / features / weights, map, conv, D2H of y
    e2e_ms = []
    for i in range(0 if args.profile else max(3, min(args.steps, 10)) + 2):
        flush.fill_(1); torch.cuda.synchronize()
        t0 = time.perf_counter()
        sp.subm_conv_host(coords_h, x_h, w_h, None, device=dev, out=y_h)
        t1 = time.perf_counter()
        if i >= 2:
            e2e_ms.append((t1 - t0) * 1e3)
    # The same call from E2E_DEPTH host threads, each with its own context (stream) and output buffer: one call's copy out
    # overlaps the next call's copy in and compute, which is how a caller with a queue of objects would drive the entry
    # point.  Every call is complete (its own H2D, map, conv, D2H); the time per step is wall clock / calls.
    e2e_pipe_ms, e2e_pipe_equal = float("nan"), None
    if e2e_ms:
        import threading
        calls = max(4, min(args.steps, 10))
        gate = threading.Barrier(E2E_DEPTH + 1)
        outs = [torch.empty_like(y_h).pin_memory() for _ in range(E2E_DEPTH)]
        errs = []

        def worker(k):
            try:
                torch.cuda.set_device(dev)
                with torch.cuda.stream(torch.cuda.Stream(dev)):       # the host layer keeps one context per (device, stream)
                    sp.subm_conv_host(coords_h, x_h, w_h, None, device=dev, out=outs[k])      # warm-up: context, scratch arena
                    gate.wait()
                    for _ in range(calls):
                        sp.subm_conv_host(coords_h, x_h, w_h, None, device=dev, out=outs[k])
                    gate.wait()
            except Exception as e:      # noqa: BLE001 - reported below, the barrier must not be left waiting
                errs.append(e); gate.abort()

        th = [threading.Thread(target=worker, args=(k,)) for k in range(E2E_DEPTH)]
        for t_ in th: t_.start()
        try:
            gate.wait(); t0 = time.perf_counter(); gate.wait(); t1 = time.perf_counter()
            e2e_pipe_ms = (t1 - t0) * 1e3 / (E2E_DEPTH * calls)
        except threading.BrokenBarrierError:
            pass
        for t_ in th: t_.join()
        if errs:
            raise errs[0]
        e2e_pipe_equal = all(torch.equal(o, y_h) for o in outs)
    if rank == 0:
        sampler.stop()
    total, conv_total, e2e_total = sum(step_ms), sum(conv_ms), (sum(e2e_ms) / len(e2e_ms) if e2e_ms else float("nan"))
    conv_avg_own = conv_total / args.steps
    achieved_own = flops / (conv_avg_own * 1e-3) / 1e12          # this rank's flops over this rank's kernel time
    sus_own = sustained["tflops"] if sustained else 0.0
    if world > 1:
        t = torch.tensor([total, conv_total, e2e_total, e2e_pipe_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total, conv_total, e2e_total, e2e_pipe_ms = t[0].item(), t[1].item(), t[2].item(), t[3].item()
        r = torch.tensor([achieved_own, sus_own], dtype=torch.float64, device=dev)
        rmin = r.clone(); dist.all_reduce(rmin, op=dist.ReduceOp.MIN)
        rsum = r.clone(); dist.all_reduce(rsum, op=dist.ReduceOp.SUM)
        achieved, achieved_mean, sus_min = rmin[0].item(), rsum[0].item() / world, rmin[1].item()
    else:
        achieved, achieved_mean, sus_min = achieved_own, achieved_own, sus_own
    flops_all, vox_all = flops * world, n * world

    sharded = None
    if world > 1 and not args.profile and not args.no_sharded:
        from trellis2_cuda_b200 import sharded_bench
        del x, y, cache, flush
        torch.cuda.empty_cache()
        sharded = sharded_bench.measure(args, rank, world, local_rank, peaks, ClockSampler, visible_gpu_index, steps=10, warmup=3,
                                        halo="nccl", single_gpu_steps=3, with_e2e=False)
    if rank != 0:
        return
    pk, pk_src = peaks()
    ms = total / args.steps
    conv_avg = conv_total / args.steps
    value = flops_all / (ms * 1e-3) / 1e12
    tensor_bound = wl["dtype"] != "f32"
    ab = alg_bytes(n, n, Ci, Co, Co, es)
    traffic = None
    tp = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tp):
        traffic = json.load(open(tp)).get(f"{args.workload}_conv_dram_bytes_per_launch") if not args.channels else None
    if tensor_bound:
        roof = {"bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / pk["bf16_tflops"], "traffic": traffic,
                "peak_source": f"{pk_src} cuBLAS bf16 burst (kernel timed alone, L2 flushed between steps)", "kernel": "k_conv_umma",
                "kernel_ms": conv_avg_own, "hbm_gbs_algorithmic": ab / (conv_avg_own * 1e-3) / 1e9,
                "per": "GPU; the lowest of the ranks" if world > 1 else "GPU", "achieved_mean_over_ranks": achieved_mean}
        if sustained:
            roof["sustained"] = {"achieved": sus_min, "peak": pk["bf16_tflops_sustained"], "frac": sus_min / pk["bf16_tflops_sustained"],
                                 "peak_source": f"{pk_src} cuBLAS bf16 sustained", "conv_ms": sustained["conv_ms"], "seconds": sustained["seconds"],
                                 "clocks": sustained["clocks"]}
    else:
        gbs = ab / (conv_avg_own * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "traffic": traffic,
                "peak_source": f"{pk_src} copy", "kernel": "k_conv_simt", "kernel_ms": conv_avg_own}
    h2d = n * 16 + n * Ci * es + Co * 27 * Ci * es
    d2h = n * Co * es
    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": {"workload": wl["desc"] + (f", the same scene on each of {world} ranks (independent replicas)" if world > 1 else ""), "voxels_per_gpu": n,
                       "Cin": Ci, "Cout": Co, "active_taps": T, "computed_taps": st["computed_taps"], "tiles": st["tiles"],
                       "step": "build_neighbors + plan + subm_conv", "l2": "flushed between steps by a 256 MiB write (not timed)"},
            "voxels_per_s": vox_all / (ms * 1e-3), "conv_only_tflops": flops_all / (conv_avg * 1e-3) / 1e12, "conv_ms": conv_avg,
            "map_and_plan_ms": ms - conv_avg,
            "roofline": roof, "clocks": clocks, "gpu_launches": launches,
            "e2e": None}
    # Both ways of driving the host-buffer entry point are measured; the line's headline is the faster one on this host
    # (in multi-rank runs several calls in flight per rank have been the slower way).
    piped = e2e_pipe_ms == e2e_pipe_ms and e2e_pipe_ms <= e2e_total
    e2e_best = e2e_pipe_ms if piped else e2e_total
    line["e2e"] = {"value": flops_all / (e2e_best * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_best,
                   "calls_in_flight": E2E_DEPTH if piped else 1, "equals_single_call_result": e2e_pipe_equal,
                   "path": "t2sc_subm_conv_host: pinned host buffers in, pinned host buffer out; the faster of one call at a time and "
                           f"{E2E_DEPTH} host threads, each with its own context, keeping that many complete calls in flight (one call's copy out "
                           "overlaps the next one's copy in and compute)",
                   "one_call_at_a_time": {"value": flops_all / (e2e_total * 1e-3) / 1e12, "ms_per_step": e2e_total},
                   f"calls_in_flight_{E2E_DEPTH}": {"value": flops_all / (e2e_pipe_ms * 1e-3) / 1e12, "ms_per_step": e2e_pipe_ms}}
    if sharded is not None:
        line["sharded"] = sharded
    if world == 1 and not args.profile:
        if wl["dtype"] != "f32":
            try:
                line["gpu_reference"] = gpu_reference_block(wl, conv_avg, ms - conv_avg)
            except Exception as e:        # the baseline must never take the bench line down
                line["gpu_reference"] = {"unavailable": f"{type(e).__name__}: {e}"}
        line["cpu_baseline"] = cpu_baseline_block(wl)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ our arm: cfg3, both halves
def run_cfg3(args, rank, world, local_rank, dev):
    import trellis2_cuda_b200 as sp
    from trellis2_cuda_b200 import scenes
    if rank != 0:
        return
    td, es = torch.float16, 2
    parents_h, flags_h = scenes.config3_pair(0)
    parents, flags = torch.from_numpy(parents_h).to(dev), torch.from_numpy(flags_h).to(dev)
    n, Ci, Cc = parents.shape[0], 128, 64
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((n, Ci), generator=g, device=dev).to(td)
    w1 = torch.from_numpy(scenes.kaiming_uniform_weight(8 * Cc, Ci, 1)).to(dev).to(td)
    w2 = torch.from_numpy(scenes.kaiming_uniform_weight(Cc, Cc, 2)).to(dev).to(td)
    ctx = sp.context(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    names = ["parent map (886,752 rows)", "subdivision maps + child map (3,288,465 rows)", "plans", "subdivision conv 128->64 (kept children)",
             "submanifold conv 64->64"]

    def step(evs=None):
        mark = (lambda i: evs[i].record()) if evs else (lambda i: None)
        mark(0)
        parent = sp.build_neighbors(parents, want_sorted=False)
        mark(1)
        lv = sp.subdivide(parent, flags)
        mark(2)
        lv.up_plan_for(Cc).check(n); lv.nb.plan_for(Cc, Cc).check(lv.coords.shape[0])
        mark(3)
        up = sp.subdiv_conv(x, w1, None, lv)
        mark(4)
        y = sp.subm_conv(up, w2, None, lv.nb)
        mark(5)
        return lv, y

    lv, y = step()
    m = lv.coords.shape[0]
    st1, st2 = lv.up_plan_for(Cc).stats(), lv.nb.plan_for(Cc, Cc).stats()
    flops = [0, 0, 0, 2.0 * st1["active_taps"] * Ci * Cc, 2.0 * st2["active_taps"] * Cc * Cc]
    byts = [n * 16 + n * 27 * 4 + n * 4, n * 8 + m * 16 + m * 4 + m * 16 + m * 27 * 4 + m * 4, 0,
            alg_bytes(n, m, Ci, Cc, 8 * Cc, es), alg_bytes(m, m, Cc, Cc, Cc, es)]
    sampler = ClockSampler(visible_gpu_index(local_rank))
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler.wait_first_sample()
    t0 = time.perf_counter()
    l0 = ctx.launch_count()
    acc, total = [0.0] * 5, 0.0
    for _ in range(args.steps):
        flush.fill_(1)
        evs = [ev() for _ in range(6)]
        step(evs)
        torch.cuda.synchronize()
        for i in range(5):
            acc[i] += evs[i].elapsed_time(evs[i + 1])
        total += evs[0].elapsed_time(evs[5])
    launches = ctx.launch_count() - l0
    t1 = time.perf_counter()
    ctx.device_status()
    clocks = sampler.stop(t0, t1)
    pk, pk_src = peaks()
    ms = total / args.steps
    table = []
    for i, nm in enumerate(names):
        t = acc[i] / args.steps
        row = {"kernel": nm, "ms": t, "gb_s_algorithmic": byts[i] / (t * 1e-3) / 1e9 if byts[i] else None,
               "frac_of_hbm": byts[i] / (t * 1e-3) / 1e9 / pk["hbm_gbs"] if byts[i] else None}
        if flops[i]:
            row.update(tflops=flops[i] / (t * 1e-3) / 1e12, frac_of_tensor_burst=flops[i] / (t * 1e-3) / 1e12 / pk["bf16_tflops"])
        table.append(row)
    c64 = table[4]
    line = {"metric": METRIC, "value": (flops[3] + flops[4]) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "cfg3: 512^3 shell -> 1024^3 shell, 128->64 subdivision conv over kept children then 64->64 submanifold conv, fp16",
                       "parents": n, "children": m, "active_taps": [st1["active_taps"], st2["active_taps"]],
                       "computed_taps": [st1["computed_taps"], st2["computed_taps"]], "tiles": [st1["tiles"], st2["tiles"]],
                       "step": "parent map + subdivision + child map + plans + both convs", "l2": "flushed between steps; inputs larger than L2"},
            "voxels_per_s": m / (ms * 1e-3), "kernels": table,
            "roofline": {"bound": "hbm", "achieved": c64["gb_s_algorithmic"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": c64["frac_of_hbm"], "traffic": None,
                         "peak_source": f"{pk_src} copy", "kernel": "k_conv_umma<64> (the 64->64 conv)", "kernel_ms": c64["ms"],
                         "tensor_frac_of_burst": c64["frac_of_tensor_burst"],
                         "note": "C = 64 sits at the tensor/HBM ridge: both fractions are given; N = 64 MMAs issue at 67 % of the pipe's rate"},
            "clocks": clocks, "gpu_launches": launches, "e2e": None}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ our arm: cfg4, the stack
def run_cfg4(args, rank, world, local_rank, dev):
    import trellis2_cuda_b200 as sp
    from trellis2_cuda_b200 import scenes
    if rank != 0:
        return
    td, es = torch.bfloat16, 2
    levels = scenes.config4_levels(0, levels=5)
    chans = [1024, 512, 256, 128, 64]
    coords0 = torch.from_numpy(levels[0][0]).to(dev)
    flags = [None if f is None else torch.from_numpy(f).to(dev) for _, f in levels]
    g = torch.Generator(device=dev).manual_seed(0)

    def rand_w(Co, Ci):
        a = 1.0 / (27.0 * Ci) ** 0.5
        return ((torch.rand((Co, 27, Ci), generator=g, device=dev) * 2 - 1) * a).to(td)

    W = []
    for l, C in enumerate(chans):
        blocks = [(rand_w(C, C), rand_w(C, C), torch.ones(C, device=dev), torch.zeros(C, device=dev)) for _ in range(2)]
        up = rand_w(8 * (C // 2), C) if l < 4 else None
        W.append((blocks, up))
    x0 = torch.randn((coords0.shape[0], chans[0]), generator=g, device=dev).to(td)
    ctx = sp.context(dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    nsm = torch.cuda.get_device_properties(dev).multi_processor_count

    def step(evs=None, info=None):
        cache = sp.build_neighbors(coords0, want_sorted=False)
        x = x0
        for l, C in enumerate(chans):
            if evs:
                evs[l][0].record()
            blocks, up = W[l]
            for (w1, w2, gm, bt) in blocks:
                h = sp.subm_conv(x, w1, None, cache, ln=(gm, bt, 1e-6), act="gelu")
                x = sp.subm_conv(h, w2, None, cache, residual=x)
            if evs:
                evs[l][1].record()
            if info is not None:
                st = cache.plan_for(C, C).stats()
                info.append({"level": l, "voxels": cache.N, "C": C, "tiles": st["tiles"], "active_taps": st["active_taps"], "computed_taps": st["computed_taps"]})
            if up is None:
                if evs:
                    evs[l][2].record(); evs[l][3].record()
                break
            lv = sp.subdivide(cache, flags[l])
            if evs:
                evs[l][2].record()
            x = sp.subdiv_conv(x, up, None, lv)
            if evs:
                evs[l][3].record()
            if info is not None:
                st = lv.up_plan_for(C // 2).stats()
                info[-1].update(up_tiles=st["tiles"], up_active_taps=st["active_taps"], up_computed_taps=st["computed_taps"])
            cache = lv.nb
        return x

    info = []
    step(info=info)
    ctx.device_status()
    sampler = ClockSampler(visible_gpu_index(local_rank))
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler.wait_first_sample()
    t0 = time.perf_counter()
    l0 = ctx.launch_count()
    acc = [[0.0, 0.0, 0.0] for _ in chans]
    total = 0.0
    for _ in range(args.steps):
        evs = [[ev() for _ in range(4)] for _ in chans]
        a, b = ev(), ev()
        a.record()
        step(evs)
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
        for l in range(5):
            for k in range(3):
                acc[l][k] += evs[l][k].elapsed_time(evs[l][k + 1])
    launches = ctx.launch_count() - l0
    t1 = time.perf_counter()
    ctx.device_status()
    clocks = sampler.stop(t0, t1)
    pk, pk_src = peaks()
    ms = total / args.steps
    flops_total, table = 0.0, []
    for l, C in enumerate(chans):
        i = info[l]
        bn = max(b for b in (256, 128, 64, 32) if C % b == 0)
        items = i["tiles"] * (C // bn)
        f_blocks = 4 * 2.0 * i["active_taps"] * C * C
        t_blocks = acc[l][0] / args.steps
        row = {"level": l, "grid": 64 << l, "voxels": i["voxels"], "C": C, "tiles": i["tiles"], "work_items_per_conv": items,
               "sm_fill": items / (-(-items // nsm) * nsm), "blocks_ms": t_blocks, "blocks_tflops": f_blocks / (t_blocks * 1e-3) / 1e12,
               "blocks_frac_of_sustained": f_blocks / (t_blocks * 1e-3) / 1e12 / pk["bf16_tflops_sustained"],
               "active_over_computed_taps": i["active_taps"] / max(i["computed_taps"], 1)}
        flops_total += f_blocks
        if "up_tiles" in i:
            Cc = C // 2
            f_up = 2.0 * i["up_active_taps"] * C * Cc
            t_map, t_up = acc[l][1] / args.steps, acc[l][2] / args.steps
            bnu = max(b for b in (256, 128, 64, 32) if Cc % b == 0)
            items_up = i["up_tiles"] * (Cc // bnu)
            row.update(subdivide_and_child_map_ms=t_map, up_conv_ms=t_up, up_conv_tflops=f_up / (t_up * 1e-3) / 1e12, up_tiles=i["up_tiles"],
                       up_sm_fill=items_up / (-(-items_up // nsm) * nsm))
            flops_total += f_up
        table.append(row)
    line = {"metric": METRIC, "value": flops_total / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg4: residual-block stack 1024->512->256->128->64 over 64^3..1024^3, per level 2 x [conv -> LayerNorm -> GELU -> conv -> residual] "
                                   "then a 2x subdivision conv halving the channels, bf16",
                       "step": "level-0 map + per level: 4 convs with fused epilogues, subdivision maps, child map, subdivision conv",
                       "l2": "not flushed: a level's features are the previous conv's output, as in the decoder"},
            "levels": table,
            "roofline": {"bound": "tensor", "achieved": flops_total / (ms * 1e-3) / 1e12, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": flops_total / (ms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"], "traffic": None,
                         "peak_source": f"{pk_src} cuBLAS bf16 sustained", "kernel": "whole step (maps included)"},
            "clocks": clocks, "gpu_launches": launches, "e2e": None}
    print(json.dumps(line), flush=True)


def run_mlp(args, rank, world, local_rank, dev):
    """The MLP half of the decoder's ConvNeXt block (src/sdec.cu:62-65 of trellis2-cuda: Linear C -> 4C, SiLU, Linear 4C -> C, add_)
    on the conv kernel (t2sc_linear, fused tails), at the row counts and widths of configurations 2-4; beside it the same
    four ops through torch (cuBLAS GEMM + separate elementwise kernels), which is what the reference's gemm.cu / ops.cu do."""
    import trellis2_cuda_b200 as sp
    ctx = sp.context(dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    F = torch.nn.functional
    sampler = ClockSampler(visible_gpu_index(local_rank))
    sampler.start()
    t0 = time.perf_counter()
    l0 = ctx.launch_count()
    rows, flops_total, ms_total = [], 0.0, 0.0

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps

    sampler.wait_first_sample()
    for n, C in ((217821, 256), (201165, 128), (727949, 64)):
        g = torch.Generator(device="cpu").manual_seed(C)
        x = torch.randn(n, C, generator=g).to(torch.bfloat16).to(dev)           # 2 x n x 5C x 2 bytes per block: larger than the L2 at every size
        w1 = (torch.randn(4 * C, C, generator=g) / C ** 0.5).to(torch.bfloat16).to(dev)
        w2 = (torch.randn(C, 4 * C, generator=g) / (4 * C) ** 0.5).to(torch.bfloat16).to(dev)
        b1, b2 = torch.zeros(4 * C, dtype=torch.bfloat16, device=dev), torch.zeros(C, dtype=torch.bfloat16, device=dev)
        h, y = torch.empty(n, 4 * C, dtype=torch.bfloat16, device=dev), torch.empty(n, C, dtype=torch.bfloat16, device=dev)

        def ours():
            sp.linear(x, w1, b1, act="silu", out=h)
            sp.linear(h, w2, b2, residual=x, out=y)

        def lib():
            return F.linear(F.silu(F.linear(x, w1, b1)), w2, b2).add_(x)

        ms, ms_lib = timed(ours), timed(lib)
        fl = 2.0 * n * C * 4 * C * 2
        byt = (n * C * 2 + n * 4 * C * 2 * 2 + n * C * 2 * 2) + 2 * 4 * C * C * 2      # x, h written and read, residual, y, weights
        rows.append({"rows": n, "C": C, "ms": ms, "tflops": fl / (ms * 1e-3) / 1e12, "gb_s_algorithmic": byt / (ms * 1e-3) / 1e9,
                     "library_gemm_ms": ms_lib, "vs_library": ms_lib / ms})
        flops_total += fl; ms_total += ms
    launches = ctx.launch_count() - l0
    t1 = time.perf_counter()
    ctx.device_status()
    clocks = sampler.stop(t0, t1)
    pk, pk_src = peaks()
    line = {"metric": "dense MLP TFLOP/s", "value": flops_total / (ms_total * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "mlp: Linear C -> 4C + SiLU, Linear 4C -> C + residual (the ConvNeXt MLP of the decoder) at 217,821 x 256, 201,165 x 128, 727,949 x 64",
                       "step": "two t2sc_linear calls per size", "l2": "inputs larger than L2 (activations of one block: 0.5 - 1.1 GB)"},
            "sizes": rows,
            "roofline": {"bound": "hbm", "achieved": min(r["gb_s_algorithmic"] for r in rows), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": min(r["gb_s_algorithmic"] for r in rows) / pk["hbm_gbs"], "traffic": None, "peak_source": f"{pk_src} copy bandwidth",
                         "kernel": "k_conv_umma (dense rows), lowest of the sizes"},
            "clocks": clocks, "gpu_launches": launches, "e2e": None}
    print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.workload == "cfg5":
        from trellis2_cuda_b200 import sharded_bench
        return sharded_bench.run(args, rank, world, local_rank, METRIC, peaks, ClockSampler, visible_gpu_index)
    if args.workload == "cfg3":
        return run_cfg3(args, rank, world, local_rank, dev)
    if args.workload == "cfg4":
        return run_cfg4(args, rank, world, local_rank, dev)
    if args.workload == "mlp":
        return run_mlp(args, rank, world, local_rank, dev)
    return run_single_conv(args, rank, world, local_rank, dev)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "mlp"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--channels", type=int, default=0, help="cfg1/cfg2: run the workload's geometry at this channel width instead of its own")
    ap.add_argument("--halo", default="nccl", choices=["p2p", "nccl"], help="cfg5: halo rows by peer-memory loads inside the conv, or by NCCL all-to-all")
    ap.add_argument("--profile", action="store_true", help="timed steps only (no sustained / end-to-end leg, no baselines): for runs under ncu")
    ap.add_argument("--no-sharded", action="store_true", help="N > 1: leave out the sharded cfg5 block")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload in ("cfg3", "cfg4", "cfg5", "mlp"):
        args.steps = min(args.steps, 50)                # multi-ms steps: fifty of them time well and keep the run short
    rank, world, local_rank = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path (use --impl reference for the CPU baseline)")
    run_ours(args, rank, world, local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
