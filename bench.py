#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2|cfg5|cfg1|cfg3]

One step = one pass of the operator as the reference's own harness times it (apps/parity.cu:157-160 of
trellis2-cuda): build the neighbour map of the scene, then run the submanifold conv.  The default workload
is the mid-decoder configuration: a ~218k-voxel shell in a 256^3 grid, Cin = Cout = 256, bf16 features and
weights, fp32 accumulation, seeded synthetic data.  With N > 1 ranks (torchrun) every rank runs that
operator on its own scene (independent batch items: no data-path collective, weak scaling);
``--workload cfg5`` instead shards ONE 8.6M-voxel scene across the ranks by Morton range and exchanges
one-voxel halos every layer (strong scaling, 4 stacked layers).

Rank 0 prints one JSON line.  ``value`` is effective TFLOP/s (2 * active taps * Cin * Cout per conv; taps
whose neighbour is absent are not counted) over the whole step, all ranks together.
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

METRIC = "sparse-conv effective TFLOP/s (active taps only)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


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

    def stop(self, t0=None, t1=None):
        """Summary of the samples taken between perf_counter times t0 and t1 (the timed region)."""
        if self.proc:
            self.proc.terminate()
        rows = [r for t, r in self.rows if (t0 is None or t >= t0) and (t1 is None or t <= t1 + 0.05)]
        self.rows = rows
        sm = [float(r[0]) for r in self.rows if len(r) >= 8 and r[0].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 8:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        smax = [float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def visible_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v for v in vis.split(",") if v != ""]
        if local_rank < len(ids) and ids[local_rank].isdigit():
            return int(ids[local_rank])
    return local_rank


# ------------------------------------------------------------------------------------------ workloads
def make_workload(name, seed):
    from trellis2_cuda_b200 import scenes
    if name == "cfg1":
        return dict(coords=scenes.config1_sphere(seed), Ci=64, Co=64, dtype="f32", desc="cfg1: 64^3 sphere shell, 64->64, fp32")
    if name == "cfg2":
        return dict(coords=scenes.config2_shell(seed), Ci=256, Co=256, dtype="bf16",
                    desc="cfg2: 256^3 shell of 6 spheres/tori, 256->256 submanifold 3x3x3, bf16 in / fp32 accumulate")
    if name == "cfg3":
        parents, flags = scenes.config3_pair(seed)
        child = scenes.subdivide_numpy(parents, flags)[0]
        return dict(coords=child, Ci=64, Co=64, dtype="f16", desc="cfg3 (second half): 1024^3 shell, 64->64 submanifold, fp16")
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


# ------------------------------------------------------------------------------------------ reference arm
def run_reference(args, rank, world):
    if rank != 0:
        return
    import oracle
    wl = make_workload(args.workload if args.workload != "cfg5" else "cfg2", 0)
    threads = os.cpu_count() or 1
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
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference has no CPU implementation of this path; this is the CPU restatement of its algorithm (oracle/oracle.c, OpenMP over output rows, scalar C)"}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ our arm
def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    import trellis2_cuda_b200 as sp
    from trellis2_cuda_b200 import scenes
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.workload == "cfg5":
        from trellis2_cuda_b200 import sharded_bench
        return sharded_bench.run(args, rank, world, local_rank, METRIC, peaks, ClockSampler, visible_gpu_index)

    wl = make_workload(args.workload, rank)            # every rank its own scene (seed = rank)
    td = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[wl["dtype"]]
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
        _ = cache.plan_for(Co, Ci)                        # the schedule this conv will use (tile height depends on Co and N)
        if record:
            record[0].record()
        y = sp.subm_conv(x, w, None, cache)
        if record:
            record[1].record()
        return cache, y

    cache, y = step()
    st = cache.plan_for(Co, Ci).stats()
    T = st["active_taps"]
    flops = 2.0 * T * Ci * Co
    ev = lambda: torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(visible_gpu_index(local_rank))
    if rank == 0:
        sampler.start()                                 # nvidia-smi needs a moment to start: launch it before the warm-up
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
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
    # end to end through the host-buffer entry point: H2D of coords / features / weights, map, conv, D2H of y
    e2e_ms = []
    for i in range(0 if args.profile else max(3, min(args.steps, 10)) + 2):
        flush.fill_(1); torch.cuda.synchronize()
        t0 = time.perf_counter()
        sp.subm_conv_host(coords_h, x_h, w_h, None, device=dev, out=y_h)
        t1 = time.perf_counter()
        if i >= 2:
            e2e_ms.append((t1 - t0) * 1e3)
    clocks = sampler.stop(t_region0, t_region1) if rank == 0 else None
    total, conv_total, e2e_total = sum(step_ms), sum(conv_ms), (sum(e2e_ms) / len(e2e_ms) if e2e_ms else float("nan"))
    if world > 1:
        t = torch.tensor([total, conv_total, e2e_total, flops, n], dtype=torch.float64, device=dev)
        mx = t.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = t.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total, conv_total, e2e_total = mx[0].item(), mx[1].item(), mx[2].item()
        flops_all, vox_all = sm[3].item(), sm[4].item()
    else:
        flops_all, vox_all = flops, n
    if rank != 0:
        return
    pk, pk_src = peaks()
    ms = total / args.steps
    conv_avg = conv_total / args.steps
    value = flops_all / (ms * 1e-3) / 1e12
    achieved = flops / (conv_avg * 1e-3) / 1e12
    tensor_bound = wl["dtype"] != "f32"
    alg_bytes = n * Ci * es + n * Co * es + 27 * Ci * Co * es + n * 27 * 4
    traffic = None
    tp = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tp):
        traffic = json.load(open(tp)).get(f"{args.workload}_conv_dram_bytes_per_launch")
    roof = ({"bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / pk["bf16_tflops"], "traffic": traffic,
             "peak_source": f"{pk_src} cuBLAS bf16 burst", "kernel": "k_conv_umma", "kernel_ms": conv_avg,
             "hbm_gbs_algorithmic": alg_bytes / (conv_avg * 1e-3) / 1e9}
            if tensor_bound else
            {"bound": "hbm", "achieved": alg_bytes / (conv_avg * 1e-3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
             "frac": alg_bytes / (conv_avg * 1e-3) / 1e9 / pk["hbm_gbs"], "traffic": traffic, "peak_source": f"{pk_src} copy", "kernel": "k_conv_simt",
             "kernel_ms": conv_avg})
    h2d = n * 16 + n * Ci * es + Co * 27 * Ci * es
    d2h = n * Co * es
    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": {"workload": wl["desc"] + (f", one independent scene per rank x {world}" if world > 1 else ""), "voxels_per_gpu": n, "Cin": Ci, "Cout": Co,
                       "active_taps": T, "computed_taps": st["computed_taps"], "tiles": st["tiles"],
                       "step": "build_neighbors + plan + subm_conv", "l2": "flushed between steps by a 256 MiB write (not timed)"},
            "voxels_per_s": vox_all / (ms * 1e-3), "conv_only_tflops": flops_all / (conv_avg * 1e-3) / 1e12, "conv_ms": conv_avg,
            "map_and_plan_ms": ms - conv_avg,
            "roofline": roof, "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": flops_all / (e2e_total * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_total,
                    "path": "t2sc_subm_conv_host: pinned host buffers in, pinned host buffer out"}}
    if world == 1 and not args.profile:
        rows = 16384 if Ci >= 256 else 65536
        threads = os.cpu_count() or 1
        r = cpu_sample(wl, rows, threads)
        line["cpu_baseline"] = {"value": r["tflops"], "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": f"first {r['rows']} of {n} output rows ({r['taps']} active taps), full-scene neighbour map charged pro rata; "
                                          f"{r['seconds']:.2f} s wall"}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg1", "cfg2", "cfg3", "cfg5"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--halo", default="nccl", choices=["p2p", "nccl"], help="cfg5: halo rows by peer-memory loads inside the conv, or by NCCL all-to-all")
    ap.add_argument("--profile", action="store_true", help="timed steps only (no end-to-end leg, no CPU baseline): for runs under ncu")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
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
