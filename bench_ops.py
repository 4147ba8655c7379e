"""Per-operation timings of the gridding path beside its headline benchmark (bench.py).

    python bench_ops.py [--reps 20] [--ops forward,backward,...]

One JSON line per operation: device time per call (CUDA events on the launching stream, inputs
resident on the device, 3 warm-up calls, every call's grids larger than L2), examples/s, and the
operation's algorithmic bytes against the measured HBM bandwidth.  Workloads are seeded synthetic
inputs with the shapes of the benchmark configurations:

* index types, 28x48^3 @0.5 A, batch 50 x [2000,4000] atoms in a blob (forward, binary forward,
  backward, relevance);
* vector types, 28x96^3 @0.25 A, batch 4 x 3000 atoms, Dirichlet(0.3) type vectors, type-indexed radii
  1.7 A x U[0.8,1.2] (forward, backward, backward_gradients) - compute bound: pair evaluations/s are
  reported next to the byte figure;
* one-hot type vectors with per-atom radii (what the autograd bindings pass), 28x48^3, batch 50;
* interpolation 28x48^3 -> 28x48^3, batch 48, random rotation + translation;
* provider: batches of 50 examples (receptor 2000-3900 + ligand 20-60 pre-typed records each, read
  once from .gninatypes files written to a temporary directory) assembled by
  ``ExampleProvider.next_device_batch`` (one host-to-device copy + the decode kernel) and gridded with
  random rotations: wall-clock examples/s of records -> grids, host work included.
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from libmolgrid_b200 import synthetic as cases  # noqa: E402

T = 28


def peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--ops", default="forward,forward_binary,backward,relevance,forward_vector,"
                                      "backward_vector,backward_gradients,onehot_forward,onehot_backward,onehot_gradgrad,interpolate,"
                                      "provider")
    ap.add_argument("--interp-batch", type=int, default=48)
    ap.add_argument("--onehot-batch", type=int, default=50, help="smaller for a profiler capture")
    args = ap.parse_args()
    import torch
    import libmolgrid_b200 as lmg
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pk, pk_kind = peak()
    ops = args.ops.split(",")

    def d(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.reps

    def report(op, workload, ms, batch, nbytes, extra=None):
        line = {"op": op, "workload": workload, "ms_per_call": ms, "examples_per_s": batch / (ms * 1e-3),
                "algorithmic_bytes_per_call": nbytes, "achieved_gbs": nbytes / (ms * 1e-3) / 1e9,
                "peak_gbs": pk, "peak_kind": pk_kind, "frac": nbytes / (ms * 1e-3) / 1e9 / pk}
        if extra:
            line.update(extra)
        print(json.dumps(line), flush=True)

    # ---- index types, 48^3 ----------------------------------------------------------------------
    if set(ops) & {"forward", "forward_binary", "backward", "relevance"}:
        B = 50
        coords, types, radii, ns, tr = cases.blob_batch(1001, B, 2000, 4000, T)
        g = lmg.GridMaker(0.5, 23.5)
        dc, dt, dr, dtr, dn = d(coords), d(types), d(radii), d(tr), d(ns)
        cen = torch.zeros((B, 3), device=dev)
        grid = torch.empty((B,) + g.grid_dimensions(T), device=dev)
        diff = torch.randn(grid.shape, device=dev)
        ag = torch.empty((B, coords.shape[1], 3), device=dev)
        rel = torch.empty((B, coords.shape[1]), device=dev)
        natoms = float(ns.sum())
        gb = grid.numel() * 4
        wl = "index types, 28x48^3, batch 50 x [2000,4000] atoms"
        if "forward" in ops:
            report("forward", wl, timeit(lambda: g.forward(cen, dc, dt, dr, grid, transforms=dtr, n_atoms=dn)),
                   B, gb + 20 * natoms)
        if "forward_binary" in ops:
            g.set_binary(True)
            report("forward_binary", wl,
                   timeit(lambda: g.forward(cen, dc, dt, dr, grid, transforms=dtr, n_atoms=dn)), B, gb + 20 * natoms)
            g.set_binary(False)
        g.forward(cen, dc, dt, dr, grid, transforms=dtr, n_atoms=dn)
        if "backward" in ops:
            report("backward", wl,
                   timeit(lambda: g.backward(cen, dc, dt, dr, diff, ag, transforms=dtr, n_atoms=dn)),
                   B, gb + 32 * natoms)
        if "relevance" in ops:
            report("relevance", wl,
                   timeit(lambda: g.backward_relevance(cen, dc, dt, dr, grid, diff, rel, transforms=dtr, n_atoms=dn)),
                   B, 2 * gb + 24 * natoms)
        del grid, diff

    # ---- vector types, 96^3 ---------------------------------------------------------------------
    if set(ops) & {"forward_vector", "backward_vector", "backward_gradients"}:
        B, N = 4, 3000
        rng = np.random.default_rng(1003)
        coords, tv, rad = cases.dense_vector_batch(1003, B, N, T)
        g = lmg.GridMaker(0.25, 23.75, False, True)
        dc, dtv, dr = d(coords), d(tv), d(rad)
        cen = torch.zeros((B, 3), device=dev)
        grid = torch.empty((B,) + g.grid_dimensions(T), device=dev)
        diff = torch.randn(grid.shape, device=dev)
        ag, tg = torch.empty((B, N, 3), device=dev), torch.empty((B, N, T), device=dev)
        dd, add, tdd = torch.empty_like(grid), torch.empty_like(ag), torch.empty_like(tg)
        gb = grid.numel() * 4
        # pair evaluations: per (atom, channel with weight != 0) the voxels of a sphere of 1.5 r_t
        vol = 4.0 / 3.0 * np.pi * (1.5 * rad / 0.25) ** 3              # [B][T]
        pairs_fwd = float(((tv != 0) * vol[:, None, :]).sum())
        pairs_all = float(N * vol.sum())
        wl = "vector types, 28x96^3, batch %d x %d atoms, type-indexed radii" % (B, N)
        # This configuration is bound by arithmetic, not by bytes: its roofline is the slower of the
        # special-function unit (16 results per clock per SM) and FP32 issue (128 lanes per clock per
        # SM) on the ALGORITHMIC work, i.e. the pair evaluations inside the cut-off spheres times
        # the operations one evaluation needs (forward: ~12 FP32 + 2 special-function results - a
        # square root and an exponential; backward: ~16 + 3; backward_gradients, both terms: ~80 + 3).
        prop = torch.cuda.get_device_properties(dev)
        clock_hz = float(getattr(prop, "clock_rate", 1965000)) * 1e3
        xu_peak = prop.multi_processor_count * 16 * clock_hz
        fp_peak = prop.multi_processor_count * 128 * clock_hz

        def compute_roof(pairs, fp32, mufu, ms):
            t = max(pairs * mufu / xu_peak, pairs * fp32 / fp_peak)
            return {"pair_evaluations_per_s": pairs / (ms * 1e-3),
                    "roofline_compute": {"bound": "special-function unit" if pairs * mufu / xu_peak >= pairs * fp32 / fp_peak
                                         else "fp32 issue", "sms": prop.multi_processor_count, "clock_mhz": clock_hz / 1e6,
                                         "xu_peak_per_s": xu_peak, "fp32_lane_peak_per_s": fp_peak,
                                         "pair_evaluations": pairs, "fp32_per_pair": fp32, "xu_per_pair": mufu,
                                         "roofline_ms": t * 1e3, "frac": t * 1e3 / ms}}
        if "forward_vector" in ops:
            ms = timeit(lambda: g.forward(cen, dc, dtv, dr, grid))
            report("forward_vector", wl, ms, B, gb + B * N * (12 + 4 * T), compute_roof(pairs_fwd, 12, 2, ms))
        g.forward(cen, dc, dtv, dr, grid)
        if "backward_vector" in ops:
            ms = timeit(lambda: g.backward(cen, dc, dtv, dr, diff, ag, tg))
            report("backward_vector", wl, ms, B, gb + B * N * (12 + 4 * T) * 2, compute_roof(pairs_all, 16, 3, ms))
        g.backward(cen, dc, dtv, dr, diff, ag, tg)
        if "backward_gradients" in ops:
            ms = timeit(lambda: g.backward_gradients(cen, dc, dtv, dr, diff, ag, tg, dd, add, tdd))
            report("backward_gradients", wl, ms, B, 2 * gb + B * N * (12 + 4 * T) * 3,
                   compute_roof(2 * pairs_fwd, 40, 3, ms))
        del grid, diff, dd

    # ---- vector types with per-atom radii (the autograd bindings' layout), 48^3 -------------------
    if set(ops) & {"onehot_forward", "onehot_backward", "onehot_gradgrad"}:
        B = args.onehot_batch
        coords, types, radii, ns, tr = cases.blob_batch(1001, B, 2000, 4000, T)
        tv = np.zeros(types.shape + (T,), np.float32)
        np.put_along_axis(tv, types.astype(np.int64)[..., None], 1.0, axis=2)
        g = lmg.GridMaker(0.5, 23.5)
        dc, dtv, dr, dtr, dn = d(coords), d(tv), d(radii), d(tr), d(ns)
        cen = torch.zeros((B, 3), device=dev)
        grid = torch.empty((B,) + g.grid_dimensions(T), device=dev)
        diff = torch.randn(grid.shape, device=dev)
        ag = torch.empty((B, coords.shape[1], 3), device=dev)
        tg = torch.empty((B, coords.shape[1], T), device=dev)
        natoms = float(ns.sum())
        gb = grid.numel() * 4
        wl = "one-hot type vectors, per-atom radii, 28x48^3, batch %d x [2000,4000] atoms" % B
        if "onehot_forward" in ops:
            report("onehot_forward", wl,
                   timeit(lambda: g.forward(cen, dc, dtv, dr, grid, transforms=dtr, n_atoms=dn)),
                   B, gb + natoms * (16 + 4 * T))
        if "onehot_backward" in ops:
            report("onehot_backward", wl,
                   timeit(lambda: g.backward(cen, dc, dtv, dr, diff, ag, tg, transforms=dtr, n_atoms=dn)),
                   B, gb + natoms * (28 + 8 * T))
        if "onehot_backward" in ops:
            report("onehot_backward_atoms_only", wl,
                   timeit(lambda: g.backward_arrays(cen, dc, dtv, dr, diff, ag, transforms=dtr, n_atoms=dn,
                                                    want_type_gradients=False)),
                   B, gb + natoms * (28 + 4 * T))
        if "onehot_gradgrad" in ops:
            g.backward(cen, dc, dtv, dr, diff, ag, tg, transforms=dtr, n_atoms=dn)
            dd, add, tdd = torch.empty_like(grid), torch.empty_like(ag), torch.empty_like(tg)
            report("onehot_gradgrad", wl,
                   timeit(lambda: g.backward_gradients(cen, dc, dtv, dr, diff, ag, tg, dd, add, tdd,
                                                       transforms=dtr, n_atoms=dn)),
                   B, 2 * gb + natoms * (40 + 12 * T))
            del dd
        del grid, diff

    # ---- interpolation --------------------------------------------------------------------------
    if "interpolate" in ops:
        B = args.interp_batch
        rng = np.random.default_rng(1005)
        gi = lmg.GridInterpolater(0.5, 23.5, 0.5, 23.5)
        src = torch.rand((B, T, 48, 48, 48), device=dev)
        dst = torch.empty_like(src)
        q = cases.random_quaternion(rng, B)
        trs = [lmg.Transform(lmg.Quaternion(*[float(v) for v in q[b]]), (0, 0, 0),
                             tuple(float(v) for v in rng.uniform(-2, 2, 3))) for b in range(B)]
        ms = timeit(lambda: gi.forward(src, trs, dst))
        from libmolgrid_b200 import _cabi
        # a staged box that did not arrive would have sent its block down the slower direct reads
        assert _cabi.lib().lmg_tma_timeouts() == 0, "tensor copies timed out during the interpolation"
        report("interpolate", "28x48^3 -> 28x48^3, batch %d, random rotation and translation" % B, ms, B,
               2 * src.numel() * 4)


    # ---- records -> grids -----------------------------------------------------------------------
    if "provider" in ops:
        import tempfile
        import time
        from libmolgrid_b200 import coord_cache
        rng = np.random.default_rng(1006)
        B, nex = 50, 100
        # wall-clock section: nothing of the earlier operations may still be queued, and their
        # cached device memory goes back first (a later cudaMalloc would otherwise free it mid-run)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        with tempfile.TemporaryDirectory() as tmp:
            lines = []
            for i in range(nex):
                n = int(rng.integers(2000, 3900))
                pts = cases.blob_batch(2000 + i, 1, n, n, T)[0][0]
                coord_cache.write_gninatypes(os.path.join(tmp, "r%d.gninatypes" % i), pts, rng.integers(2, 28, n))
                m = int(rng.integers(20, 60))
                coord_cache.write_gninatypes(os.path.join(tmp, "l%d.gninatypes" % i),
                                             cases.sphere(rng, m, 4.0), rng.integers(2, 21, m))
                lines.append("1 r%d.gninatypes l%d.gninatypes" % (i, i))
            with open(os.path.join(tmp, "list.types"), "w") as f:
                f.write("\n".join(lines) + "\n")
            prov = coord_cache.ExampleProvider(data_root=tmp)
            prov.populate(os.path.join(tmp, "list.types"))
            g = lmg.GridMaker(0.5, 23.5)
            grid = torch.empty((B,) + g.grid_dimensions(prov.num_types()), device=dev)
            nbytes = 0

            def one():
                batch = prov.next_device_batch(B)
                g.forward(batch, grid, 2.0, True)
                return batch

            for _ in range(4):
                one()                       # also reads every file once
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(args.reps):
                batch = one()
                nbytes += int(batch.n_atoms.numel()) * 4 + int(batch.coords.shape[0]) * 0
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) / args.reps
            h2d = float(batch.n_atoms.sum().item()) * 16
            report("provider", "records -> device batch -> forward, batch 50, wall clock incl. host assembly",
                   wall * 1e3, B, grid.numel() * 4 + h2d, {"h2d_bytes_per_call": h2d})
            # the same with the host half of the batches running ahead on worker threads
            for workers in (1, 2, 3):
                it = prov.device_batches(B, count=args.reps + 4, workers=workers)
                for _ in range(4):
                    g.forward(next(it), grid, 2.0, True)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for batch in it:
                    g.forward(batch, grid, 2.0, True)
                torch.cuda.synchronize()
                wall = (time.perf_counter() - t0) / args.reps
                report("provider_prefetch", "as provider, host assembly %d batch(es) ahead on %d worker thread(s)"
                       % (workers + 1, workers), wall * 1e3, B, grid.numel() * 4 + h2d,
                       {"h2d_bytes_per_call": h2d, "workers": workers})


if __name__ == "__main__":
    main()
