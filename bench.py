#!/usr/bin/env python
"""Headline benchmark: examples/s gridded (28x48^3 fp32) forward + backward.

A step is one pass of the hot path over one batch per GPU: GridMaker.forward (per-example
rotation/translation fused in) followed by GridMaker.backward on a batch of 50 examples with
2000-4000 index-typed atoms each (30% in a 12 A ball, 70% in a 4 A blob), 28 channels, 48^3 grid
at 0.5 A, upstream gradient N(0,1).  Inputs are seeded synthetic data of those shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  `value` times device-resident inputs; `e2e` times the same step through the
public API with pinned host buffers for the atoms and the returned gradients; `roofline` is the
dominant kernel's algorithmic bytes over its CUDA-event duration against the measured HBM copy
bandwidth; `cpu_baseline` is the CPU checker (the reference's own sources when compiled, else the
C restatement) timed on the host cores on a bounded sample.  --impl reference times that CPU code
alone with all host cores.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from libmolgrid_b200 import synthetic as cases  # noqa: E402

BATCH = 50
NTYPES = 28
NMIN, NMAX = 2000, 4000
RES, DIMENSION = 0.5, 23.5
DIM = 48
GRID_BYTES = NTYPES * DIM ** 3 * 4          # 12,386,304
SEED = 1001
METRIC = "examples/s gridded (28x48^3 fp32) fwd+bwd"
WORKLOAD = ("batch 50 per GPU x [2000,4000] index-typed atoms (70% in a 4A blob), 28x48^3 @0.5A, "
            "forward with fused per-example rotation+translation, then backward with N(0,1) grid gradient")
WORKLOAD_C4A = ("one batch of 1024 x [2000,4000] index-typed atoms (70% in a 4A blob), 28x48^3 @0.5A, cut by "
                "example over the GPUs; forward with fused rotation+translation, then backward")
# dram bytes per example from the ncu captures summarised under profiles/ (batch 12, scaled per
# example: every example's grids are separate and larger than what L2 keeps, so traffic grows in
# proportion).  forward = the fill's own 12,386,304 B + the scatter kernel's 6.59 MB of read-modify-
# write on the sectors atoms touch; backward = the touched part of the grid gradient.
NCU_TRAFFIC_PER_EXAMPLE = {"forward": 12386304 + 6.59e6, "backward": 6.87e6}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle (reference sources when compiled here, else the C restatement)
# ------------------------------------------------------------------------------------------------
def _cpu_kind():
    from oracle.oracle import available
    return "reference" if available("ref") else "port"


def _cpu_worker(args):
    kind, seed, nex = args
    from oracle.oracle import CpuOracle
    o = CpuOracle("ref" if kind == "reference" else "port")
    coords, types, radii, ns, tr = cases.blob_batch(seed, nex, NMIN, NMAX, NTYPES)
    gm = o.gm(RES, DIMENSION)
    rng = np.random.default_rng(seed)
    diff = rng.standard_normal((NTYPES, DIM, DIM, DIM), dtype=np.float32)
    t0 = time.perf_counter()
    chk = 0.0
    for b in range(nex):
        n = int(ns[b])
        moved = o.transform_forward(tr[b], coords[b, :n])
        grid = o.forward_index(gm, (0, 0, 0), moved, types[b, :n], radii[b, :n], NTYPES)
        ag = o.backward_index(gm, (0, 0, 0), moved, types[b, :n], radii[b, :n], diff)
        chk += float(grid[0, 24, 24, 24]) + float(ag[0, 0])
    return time.perf_counter() - t0, chk


def cpu_examples_per_s(kind, cores, per_core, seed=SEED):
    """All `cores` workers grid `per_core` examples each, at the same time; returns examples/s."""
    import multiprocessing as mp
    ctx = mp.get_context("fork")
    with ctx.Pool(cores) as pool:
        # warm the pool (imports, library load) outside the timed region
        pool.map(_cpu_worker, [(kind, seed + 7, 1)] * cores)
        t0 = time.perf_counter()
        pool.map(_cpu_worker, [(kind, seed + 100 + i, per_core) for i in range(cores)], chunksize=1)
        wall = time.perf_counter() - t0
    return cores * per_core / wall, wall


def run_reference_arm(args, rank):
    if rank != 0:
        return
    kind = _cpu_kind()
    # the parent loads the checker library and grids one small example itself, so that the library
    # shows among the files this process has mapped; the timed work runs in forked workers
    _cpu_worker((kind, SEED + 5, 1))
    cores = os.cpu_count() or 1
    per_core = 1
    times = []
    for i in range(args.warmup + args.steps):
        rate, wall = cpu_examples_per_s(kind, cores, per_core, seed=SEED + 1000 * i)
        if i >= args.warmup:
            times.append(wall)
    total = sum(times)
    value = cores * per_core * len(times) / total
    sample = "%d examples per step (one per host core), %d timed steps" % (cores * per_core, len(times))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "examples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "host": "CPU only: the reference's CPU GridMaker"},
        "cpu_baseline": {"value": value, "unit": "examples/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "examples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Reads SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        while not self._halt.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.02)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def make_workload(args, rank, world):
    """The rank's slice of the global batch, cut by example with the sharding helper.

    headline: 50 examples per GPU (global batch 50 x world, weak scaling); c4a: ONE batch of 1024
    (strong scaling).  Every example has its own atom count; the cut balances atoms, so ranks hold
    slightly different numbers of examples."""
    from libmolgrid_b200.sharding import shard_bounds
    global_batch = 1024 if args.config == "c4a" else args.batch * world
    seed = 1004 if args.config == "c4a" else SEED
    counts = cases.blob_counts(seed, global_batch, NMIN, NMAX)
    R = cases.type_radii(seed, NTYPES)
    bounds = shard_bounds(counts, world, per_example_cost=args.example_cost)
    start, end = bounds[rank]
    return cases.blob_slice(seed, start, end, counts, R), global_batch, bounds


def run_gpu_arm(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import libmolgrid_b200 as lmg
    from libmolgrid_b200 import _cabi
    import ctypes

    # CPU baseline first (rank 0, N=1 only), before CUDA is initialised in this process
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        kind = _cpu_kind()
        cores = os.cpu_count() or 1
        per_core = 8   # about 0.1 s of CPU work per example
        rate, wall = cpu_examples_per_s(kind, cores, per_core)
        cpu = {"value": rate, "unit": "examples/s", "cores": cores, "kind": kind, "per_core": rate / cores,
               "sample": "%d examples of the same workload (%d per core, one process per core), %.1f s wall"
                         % (cores * per_core, per_core, wall)}

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # examples are independent: every rank grids its own slice of the global batch, no collective
    (coords, types, radii, ns, tr), global_batch, bounds = make_workload(args, rank, world)
    nex = coords.shape[0]
    nmax = coords.shape[1]
    g = lmg.GridMaker(RES, DIMENSION)
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + rank)

    def d(a):
        return torch.from_numpy(a).to(dev)

    dc, dt, dr, dtr, dn = d(coords), d(types), d(radii), d(tr), d(ns)
    cen = torch.zeros((nex, 3), device=dev)
    grid = torch.empty((nex,) + g.grid_dimensions(NTYPES), device=dev)
    diff = torch.randn(grid.shape, device=dev, generator=gen)
    ag = torch.empty((nex, nmax, 3), device=dev)

    def step():
        g.forward(cen, dc, dt, dr, grid, transforms=dtr, n_atoms=dn)
        g.backward(cen, dc, dt, dr, diff, ag, transforms=dtr, n_atoms=dn)

    # e2e: every step's atoms come from pinned host memory and its gradients go back to pinned host
    # memory.  As a training loop's data loader does, the copies run on a second stream one step
    # ahead of the kernels (two sets of device input buffers); the kernels of step i wait on the
    # upload of step i, the download of step i waits on its backward kernel.
    hc, ht, hr, htr = (torch.from_numpy(x).pin_memory() for x in (coords, types, radii, tr))
    hcen = torch.zeros((nex, 3)).pin_memory()
    hag = [torch.empty((nex, nmax, 3)).pin_memory() for _ in range(2)]
    host_in = (hc, ht, hr, htr, hcen)
    h2d = sum(x.numel() * x.element_size() for x in host_in)
    d2h = hag[0].numel() * hag[0].element_size()
    copy_stream = torch.cuda.Stream(device=dev)
    dev_in = [tuple(torch.empty_like(x, device=dev) for x in host_in) for _ in range(2)]
    dev_ag = [torch.empty_like(ag) for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]
    e2e_state = {"i": 0}

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])       # the kernels that read this slot are done
            for dst, src in zip(dev_in[slot], host_in):
                dst.copy_(src, non_blocking=True)
            uploaded[slot].record(copy_stream)

    def step_e2e():
        i = e2e_state["i"]
        slot = i & 1
        if i == 0:
            upload(0)
        upload(slot ^ 1)                                   # next step's atoms, one step ahead
        main = torch.cuda.current_stream(dev)
        main.wait_event(uploaded[slot])
        main.wait_event(downloaded[slot])                # this slot's previous gradients have left
        c_, t_, r_, tr_, cen_ = dev_in[slot]
        g.forward(cen_, c_, t_, r_, grid, transforms=tr_, n_atoms=dn)
        g.backward(cen_, c_, t_, r_, diff, dev_ag[slot], transforms=tr_, n_atoms=dn)
        consumed[slot].record(main)
        computed[slot].record(main)
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(computed[slot])
            hag[slot].copy_(dev_ag[slot], non_blocking=True)
            downloaded[slot].record(copy_stream)
        e2e_state["i"] = i + 1

    # The same step with the host buffers handed straight to the API: the call stages them itself
    # (host-to-device copies of the atoms, device-to-host copy of the gradients) on the calling
    # stream, nothing overlapped.
    htr_rows = htr

    def step_host_api():
        g.forward(hcen, hc, ht, hr, grid, transforms=htr_rows, n_atoms=dn)
        g.backward(hcen, hc, ht, hr, diff, hag[0], transforms=htr_rows, n_atoms=dn)

    # Every buffer on the host, the grids too: the forward call copies 12.4 MB per example out, the
    # backward call as much in.  What a caller pays who keeps nothing on the device.
    host_grid = {}

    def step_host_grids():
        if not host_grid:
            host_grid["out"] = torch.empty(tuple(grid.shape)).pin_memory()
            host_grid["diff"] = torch.empty(tuple(grid.shape)).pin_memory()
            host_grid["diff"].copy_(diff)
        g.forward(hcen, hc, ht, hr, host_grid["out"], transforms=htr_rows, n_atoms=dn)
        g.backward(hcen, hc, ht, hr, host_grid["diff"], hag[0], transforms=htr_rows, n_atoms=dn)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    per_rank = {}

    def timed(fn, steps, tag):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        h0 = time.perf_counter()
        for _ in range(steps):
            fn()
        host_ms = (time.perf_counter() - h0) * 1e3                 # time the host needed to issue the steps
        torch.cuda.current_stream(dev).wait_stream(copy_stream)   # the last download belongs to the region
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        mine = torch.tensor([ms, host_ms, float(ns.sum()), float(nex)], device=dev, dtype=torch.float64)
        if world > 1:
            every = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(every, mine)
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        else:
            every = [mine]
        per_rank[tag] = [{"device_ms": round(float(x[0]), 3), "host_issue_ms": round(float(x[1]), 3),
                          "atoms": int(x[2]), "examples": int(x[3])} for x in every]
        return ms

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    lib = _cabi.lib()
    lib.lmg_profile_enable(0)
    launches0 = lib.lmg_launch_count()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(step, args.steps, "resident")       # the headline: no timing hooks inside the library
    launches = lib.lmg_launch_count() - launches0
    extended = False
    if ms < 250.0:
        # a short timed region gives the sampler a reading or two: the same steps keep running for a
        # quarter of a second more, untimed, so that the clocks under this load are on record
        extended = True
        until = time.perf_counter() + 0.25
        while time.perf_counter() < until:
            for _ in range(10):
                step()
            torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["window"] = "timed region plus 0.25 s of the same steps" if extended else "timed region"

    # what a step costs the calling thread: short bursts into an idle GPU, so that the launch queue
    # never fills and the host is never held back by the device (the host time of the long timed
    # runs is the device's pace)
    def host_burst(fn, n=20):
        best = None
        for _ in range(3):
            torch.cuda.synchronize()
            h0 = time.perf_counter()
            for _ in range(n):
                fn()
            us = (time.perf_counter() - h0) * 1e6 / n
            best = us if best is None else min(best, us)
        torch.cuda.synchronize()
        return best
    host_issue_us = host_burst(step)
    # the same step through `import molgrid`: the compiled GridMaker (pybind11 over the C++ host layer)
    try:
        import molgrid as _mg
        gc = _mg.GridMaker(0.5, 23.5)

        def step_compiled():
            gc.forward(cen, dc, dt, dr, grid, transforms=dtr, n_atoms=dn)
            gc.backward(cen, dc, dt, dr, diff, ag, transforms=dtr, n_atoms=dn)
        step_compiled()
        host_issue_compiled_us = host_burst(step_compiled)
    except Exception as e:  # the compiled module is an extra: the benchmark runs without it
        sys.stderr.write("compiled module not measured: %r\n" % (e,))
        host_issue_compiled_us = None

    # per-kernel durations in a pass of their own (CUDA events around each launch, on its stream)
    ksteps = min(args.steps, 200)
    lib.lmg_profile_enable(4 * ksteps + 8)
    timed(step, ksteps, "kernels")
    kms = (ctypes.c_double * 3)()
    kcount = (ctypes.c_int * 3)()
    lib.lmg_profile_collect(kms, kcount)
    lib.lmg_profile_enable(0)

    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps, "e2e")
    hsteps = min(args.steps, 50)
    for _ in range(2):
        step_host_api()
    ms_host = timed(step_host_api, hsteps, "host_api")
    gsteps = min(args.steps, 5)
    step_host_grids()
    ms_hostgrid = timed(step_host_grids, gsteps, "host_grids")
    host_grid.clear()

    # sanity: the timed kernels did the work (cheap property checks, outside the timed region)
    assert torch.isfinite(ag).all() and float(grid.sum()) > 0

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    total_examples = global_batch * args.steps
    value = total_examples / (ms * 1e-3)
    peak, peak_kind = measured_peak()
    natoms = float(ns.sum())
    fwd_bytes = nex * GRID_BYTES + 20.0 * natoms           # write grid once + read atoms
    bwd_bytes = nex * GRID_BYTES + 32.0 * natoms           # read diff once + read atoms + write gradients
    kern = []
    # the forward pass is a zero fill of the grids plus the scatter kernel that adds the densities
    # into them; its algorithmic bytes (one write of every grid) are charged to the pair
    fill_ms = kms[2] / kcount[2] if kcount[2] else 0.0
    for k, name, nbytes in ((0, "forward (zero fill + k_emit + k_forward_quads)", fwd_bytes),
                            (1, "backward (k_emit + k_backward_quads)", bwd_bytes)):
        if kcount[k]:
            avg_ms = kms[k] / kcount[k] + (fill_ms if k == 0 else 0.0)
            kern.append({"kernel": name, "launches": int(kcount[k]), "avg_ms": avg_ms,
                         "achieved": nbytes / (avg_ms * 1e-3) / 1e9, "bytes_per_launch": nbytes})
    if kcount[2]:
        kern.append({"kernel": "zero fill alone", "launches": int(kcount[2]), "avg_ms": fill_ms,
                     "achieved": nex * GRID_BYTES / (fill_ms * 1e-3) / 1e9, "bytes_per_launch": nex * GRID_BYTES})
    dom = max(kern[:2], key=lambda x: x["avg_ms"] * x["launches"]) if kern else None
    roof = None
    if dom:
        traffic = NCU_TRAFFIC_PER_EXAMPLE.get(dom["kernel"].split()[0])
        roof = {"bound": "hbm", "kernel": dom["kernel"], "achieved": dom["achieved"], "peak": peak,
                "unit": "GB/s", "frac": dom["achieved"] / peak, "peak_kind": peak_kind,
                "traffic": traffic * nex if traffic else None,
                "avg_launch_ms": dom["avg_ms"], "algorithmic_bytes_per_launch": dom["bytes_per_launch"]}
    step_bytes = fwd_bytes + bwd_bytes
    strong = args.config == "c4a"
    line = {
        "metric": METRIC, "value": value, "unit": "examples/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_C4A if strong else WORKLOAD, "global_batch": global_batch,
                   "examples_per_rank": [e - s0 for s0, e in bounds],
                   "parallelism": "one global batch cut by example over %d GPU(s) with the atom-balancing "
                                  "sharding helper, no collective; every example has its own atom count" % world,
                   "l2": "inputs larger than L2: each step writes %d MB of grids and reads as much of gradients per GPU"
                         % (nex * GRID_BYTES // 1000000)},
        "roofline": roof,
        "roofline_step": {"bound": "hbm", "achieved": step_bytes / (ms / args.steps * 1e-3) / 1e9,
                          "peak": peak, "unit": "GB/s per GPU (rank 0)",
                          "frac": step_bytes / (ms / args.steps * 1e-3) / 1e9 / peak,
                          "note": "whole step (all kernels) vs 24.77 MB + 52 B/atom per example"},
        "kernels": kern,
        "cpu_baseline": cpu,
        "e2e": {"value": total_examples / (ms_e2e * 1e-3), "unit": "examples/s",
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "note": "every step uploads its atoms from pinned host memory and downloads its atom "
                        "gradients to pinned host memory; the copies run on a second stream one step ahead "
                        "of the kernels; grids and their gradients stay on the device as in a training loop"},
        "e2e_host_arrays": {"value": global_batch * hsteps / (ms_host * 1e-3), "unit": "examples/s", "steps": hsteps,
                            "note": "pinned host arrays handed to GridMaker.forward/backward themselves: the "
                                    "calls copy atoms in and gradients out on the calling stream, no overlap"},
        "e2e_host_grids": {"value": global_batch * gsteps / (ms_hostgrid * 1e-3), "unit": "examples/s", "steps": gsteps,
                           "h2d_bytes_per_step": int(h2d + nex * GRID_BYTES), "d2h_bytes_per_step": int(d2h + nex * GRID_BYTES),
                           "note": "every array in pinned host memory, the grids and their gradients too: "
                                   "bound by the host link (12.4 MB per example each way)"},
        "per_rank": per_rank,
        "host_issue_us_per_step": {"value": round(host_issue_us, 1),
                                   "compiled_module": None if host_issue_compiled_us is None else round(host_issue_compiled_us, 1),
                                   "note": "calling thread, forward + backward through the Python layer, bursts "
                                           "of 20 steps into an idle GPU (rank 0); the host_issue_ms of per_rank "
                                           "is the device's pace once the launch queue is full"},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps (default: 1000 on the GPU, 20 for --impl reference)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="examples per GPU per step (the headline workload uses 50; smaller values are for profiler captures)")
    ap.add_argument("--config", default="headline", choices=["headline", "c4a"],
                    help="headline: 50 examples per GPU; c4a: one batch of 1024 examples cut over the GPUs")
    ap.add_argument("--example-cost", type=float, default=1200.0,
                    help="cost of one example's grids in atom-equivalents, for the balanced cut")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.steps is None:
            args.steps = 20
        run_reference_arm(args, rank)
        return
    if args.steps is None:
        args.steps = 1000
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
