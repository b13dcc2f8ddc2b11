#!/usr/bin/env python
"""Benchmark of the fused gather-map-reduce SpMV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--grid n]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload: the multi-GPU configuration, a 7-point Laplacian on a 512^3 grid (fp64 values,
int64 row offsets, int32 columns, 937,951,232 non-zeros), rows split into nnz-balanced z-slabs, one
rank per GPU, iterated as x <- A x with a one-plane halo exchange per neighbour per iteration (NCCL).
A step is one iteration (halo exchange + one fused SpMV launch per rank).  The problem is fixed as N
grows (strong scaling).  The metric is the reference's effective bandwidth: every compulsory array
counted once per SpMV (src/flex_spmv_full_red.cu:347-359 of the reference) divided by the time.

One JSON line is printed by rank 0.  At N = 1 it also carries the per-configuration results of the
four single-GPU configurations (kernel-only, warm and with L2 flushed between launches) and the CPU
baseline: the reference's own generated CPU operator (OmpMergeSystem, compiled from the reference's
sources into oracle/_ref) timed on a bounded slab of the same matrix on the host cores.
`--impl reference` times only that CPU operator.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fused SpMV effective GB/s"
UNIT = "GB/s"
# DRAM traffic of the headline kernel: dram__bytes_read.sum + dram__bytes_write.sum of ONE ncu capture of
# flex_tile_kernel<spmv_f64, int64 offsets> on the 192^3 grid (the full-size launch holds too much memory to capture
# with more than one pass); traffic grows in proportion to the grid, so it is scaled to the benchmarked launch by the
# algorithmic bytes.  Part of y is still in L2 when that capture ends, so the write figure is a lower bound.
DRAM_CAPTURE = {"grid": 192, "read_bytes": 718.4e6, "write_bytes": 24.8e6, "algorithmic_bytes": 761_757_704}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def poisson3d_bytes(n: int) -> tuple[int, int]:
    n3 = n ** 3
    nnz = 7 * n3 - 6 * n * n
    return 12 * nnz + 8 * (n3 + 1) + 16 * n3, nnz


def workload_config(n: int) -> dict:
    """The `config` object of the JSON line: the workload only, identical for the CUDA arm and the CPU reference arm
    (what differs between the arms -- partition, halo exchange, offset width -- is reported under `run`)."""
    alg, nnz = poisson3d_bytes(n)
    return {"workload": f"config4: 3D Poisson {n}^3 7-point SpMV y = A x, fp64 values, int32 columns, {nnz} non-zeros, "
                        f"{n ** 3} rows, one SpMV per step",
            "algorithmic_bytes_per_step": alg, "l2": "inputs larger than L2 (matrix >= 1.8 GB per GPU)"}


# --------------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi in the background during the timed region (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []      # (arrival time, csv line)
        self.t_begin = self.t_end = None

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def under_load(self) -> int:
        return sum(1 for t, _ in self.lines if self.t_begin is not None and t >= self.t_begin)

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, extra_steps: int = 0) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons, power = [], [], set(), []
        in_timed = 0
        for t, ln in self.lines:
            if self.t_begin is None or t < self.t_begin:
                continue
            if self.t_end is not None and t <= self.t_end:
                in_timed += 1
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "samples_in_timed_region": in_timed,
                "trailing_untimed_steps_sampled": extra_steps, "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------------
# CPU reference arm
# --------------------------------------------------------------------------------------------------
def host_threads() -> int:
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    return min(cores, 256)      # the reference's carry arrays are [256] (codegen/merged_gen_core.py:75-77)


def time_cpu_operator(ir, prob, dtype, steps: int, warmup: int, copy_inputs: bool = True) -> dict:
    """Times the reference's generated CPU operator (oracle/_ref) on all host threads; where the AVX2 object of
    the graph exists and runs here, both objects are tried and the faster one is timed.  Falls back to the C/numpy
    restatement (kind "port", one thread) when oracle/_ref did not travel.  Returns the outputs of the last call."""
    from oracle import ref_run
    threads = host_threads()
    if ref_run.available(ir.name):
        kind, best = "reference", None
        for variant in ref_run.variants(ir.name):
            call = ref_run.PreparedCall(ir, prob, dtype, num_threads=threads, variant=variant, copy_inputs=copy_inputs)
            call.run()
            t0 = time.perf_counter()
            call.run()
            dt1 = time.perf_counter() - t0
            if best is None or dt1 < best[0]:
                best = (dt1, variant, call)
        _, variant, call = best
        run = call.run
    else:
        kind, threads, variant = "port", 1, "restatement"
        from oracle import ir_eval
        run = lambda: ir_eval.run_graph(ir, prob, dtype, num_threads=1)[0]   # noqa: E731
    for _ in range(warmup):
        run()
    times = []
    outs = None
    for _ in range(steps):
        t0 = time.perf_counter()
        outs = run()
        times.append(time.perf_counter() - t0)
    return {"seconds_median": float(np.median(times)), "seconds_mean": float(np.mean(times)), "cores": threads, "kind": kind,
            "object": {"so": "portable x86-64 object", "so_x86_64_v3": "-march=x86-64-v3 object"}.get(variant, variant),
            "outputs": outs, "steps": steps, "warmup": warmup}


def cpu_reference(grid: int, steps: int, warmup: int, planes=None) -> dict:
    """The reference's generated CPU operator (OmpMergeSystem<double,int> behind a C trampoline: no torch::zeros
    per call, which favours the reference) on the benchmark matrix, all host threads.  planes=None: the whole
    grid^3 matrix with int32 offsets (the reference's only width; 937,951,232 + 134,217,728 < 2^31 at 512^3);
    a number: that many z-planes of it (the fallback when the host cannot hold the 13 GB matrix)."""
    from flexspmv_b200 import graphs, problems
    ir = graphs.spmv_graph()
    whole = planes is None
    if whole:
        try:
            prob = problems.poisson3d_chunked(grid, offset_dtype=np.int32)
        except MemoryError:
            whole, planes = False, min(128, grid)
    if not whole:
        planes = min(planes, grid - 2) if grid > 2 else grid
        z0 = 1 if grid > 2 else 0
        prob = problems.poisson3d(grid, z_begin=z0, z_end=z0 + planes, offset_dtype=np.int32)
        shift = (z0 - 1) * grid * grid if z0 > 0 else 0
        n2 = grid * grid
        prob.indices["selector"] = (prob.indices["selector"].astype(np.int64) - shift).astype(np.int32)
        prob.values["x"] = np.ascontiguousarray(prob.values["x"][shift:shift + (planes + 2) * n2])
        prob.num_cols = prob.values["x"].shape[0]
    nnz = prob.nnz
    alg = 12 * nnz + 8 * (prob.num_rows + 1) + 8 * prob.num_cols + 8 * prob.num_rows
    r = time_cpu_operator(ir, prob, np.float64, steps, warmup, copy_inputs=False)
    dt = r["seconds_mean"]
    what = f"the whole {grid}^3 7-point Laplacian" if whole else f"{planes} of {grid} z-planes of the {grid}^3 7-point Laplacian"
    return {"value": alg / dt / 1e9, "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "whole_problem": whole,
            "sample": f"{what} ({prob.num_rows} rows, {nnz} non-zeros), {steps} calls after {warmup} warm-up, int32 offsets "
                      f"(the reference's only width), {r['object']}, called through a C trampoline (no per-call output allocation)",
            "ms_per_step": dt * 1e3, "edges_per_s": nnz / dt}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(args.warmup, 3)      # exactly the K and W of the CUDA arm (0.15 s per call)
    r = cpu_reference(args.grid, steps, warmup, planes=args.cpu_planes)
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": workload_config(args.grid),
            "run": {"arm": "the reference's generated CPU operator on the host cores, one call per step, int32 row offsets "
                           "(its only width), no halo exchange (one host)",
                    "whole_problem": r["whole_problem"]},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "edges_per_s": r["edges_per_s"]}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# single-GPU configurations 0-3 (kernel-only numbers, reported beside the headline at N = 1)
# --------------------------------------------------------------------------------------------------
def row_error(got: np.ndarray, ref: np.ndarray, abs_sums: np.ndarray) -> float:
    """max over rows and components of |got - ref| / sum_j |term_ij| (the sum of the magnitudes of the row's
    per-edge terms: rows such as 4x - sum(x) cancel, so |y_i| itself is no scale for a reordered sum)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    scale = np.maximum(np.asarray(abs_sums, np.float64).reshape(ref.shape), np.finfo(np.float64).tiny)
    finite = np.isfinite(ref)
    if not np.array_equal(np.isfinite(got), finite):
        return float("inf")
    return float((np.abs(got - ref)[finite] / scale[finite]).max()) if finite.any() else 0.0


TOLERANCE = {4: 1e-5, 8: 1e-12}      # per row, relative to the sum of term magnitudes: fp32 / fp64


def time_config(name, ir, ext, values, indices, ro, outputs, num_rows, nnz, num_cols, alg_bytes, iters, peak, flush_buf):
    import torch
    launch = ext.prepare(values, indices, ro, outputs, num_rows, nnz, num_cols).launch
    for _ in range(3):
        launch()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        launch()
    e1.record()
    torch.cuda.synchronize()
    warm_ms = e0.elapsed_time(e1) / iters
    cold = []
    for _ in range(min(iters, 20)):
        flush_buf.zero_()            # 256 MB write: evicts the inputs from L2 (not timed)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); launch(); b.record()
        torch.cuda.synchronize()
        cold.append(a.elapsed_time(b))
    cold_ms = float(np.median(cold))
    ext.check()                      # a kernel that gave up (bounded wait, unplanned workspace) fails the run here
    return {"config": name, "rows": int(num_rows), "edges": int(nnz), "algorithmic_bytes": int(alg_bytes),
            "warm": {"ms": warm_ms, "gbs": alg_bytes / warm_ms / 1e6, "frac_of_hbm_peak": alg_bytes / warm_ms / 1e6 / peak,
                     "edges_per_s": nnz / warm_ms * 1e3, "iters": iters},
            "cold_l2_flushed": {"ms": cold_ms, "gbs": alg_bytes / cold_ms / 1e6, "frac_of_hbm_peak": alg_bytes / cold_ms / 1e6 / peak,
                                "edges_per_s": nnz / cold_ms * 1e3, "iters": len(cold)}}


def cpu_beside(entry: dict, ir, prob, dtype, gpu_outputs, abs_sums=None, steps: int = 10) -> None:
    """Adds to a configuration's entry the reference's generated CPU operator timed on the same arrays (all host
    threads, median of `steps` calls after 2 warm-up calls) and the largest per-row error of the GPU result
    against that operator's result."""
    from oracle import ir_eval
    r = time_cpu_operator(ir, prob, dtype, steps, 2)
    sec = r["seconds_median"]
    alg, nnz = entry["algorithmic_bytes"], entry["edges"]
    entry["cpu_baseline"] = {"value": alg / sec / 1e9, "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "ms": sec * 1e3,
                             "edges_per_s": nnz / sec, "sample": f"the same arrays, median of {steps} calls, {r['object']}"}
    if abs_sums is None:
        _, _, abs_sums = ir_eval.run_graph(ir, prob, dtype, num_threads=host_threads(), want_abs_sums=True)
    errs = [row_error(g, c, a) for g, c, a in zip(gpu_outputs, r["outputs"], abs_sums)]
    tol = TOLERANCE[np.dtype(dtype).itemsize]
    entry["max_row_err"] = {"value": max(errs), "tol": tol, "ok": bool(max(errs) <= tol),
                            "against": "the reference's generated CPU operator on the same arrays" if r["kind"] == "reference"
                            else "the CPU restatement of the reference operator",
                            "relative_to": "sum of the magnitudes of the row's per-edge terms"}
    if not entry["max_row_err"]["ok"]:
        raise SystemExit(f"bench.py: {entry['config']}: GPU result differs from the CPU operator: {entry['max_row_err']}")


def probe_gather(log2_rows: int) -> dict:
    """The chip's rate of 4-byte gathers without locality, on the config-3 arrays (flexspmv_probe_gather): the bound of
    any kernel on that matrix, as a function of the shared memory the kernel claims per SM."""
    import ctypes
    import torch
    from flexspmv_b200 import problems
    from flexspmv_b200.binding import check, load_library
    lib = load_library()
    dev = torch.device("cuda", torch.cuda.current_device())
    ro, cols, vals, x = problems.powerlaw_device(1 << log2_rows, 3, dev)
    m = cols.numel()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    out = torch.zeros(sms * 8, device=dev)
    rows = []
    for kb_per_sm in (0, 32, 64, 132, 164, 196, 224):
        def fn():
            check(lib, lib.flexspmv_probe_gather(ctypes.c_void_p(cols.data_ptr()), ctypes.c_void_p(vals.data_ptr()),
                                                 ctypes.c_void_p(x.data_ptr()), ctypes.c_int64(m), ctypes.c_void_p(out.data_ptr()),
                                                 sms * 8, kb_per_sm * 1024 // 8, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
                  "probe_gather")
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / 10
        rows.append({"shared_kb_per_sm": kb_per_sm, "ms": ms, "giga_gathers_per_s": m / ms / 1e6})
    return {"probe": "random 4-byte gathers, power-law CSR arrays", "rows": 1 << log2_rows, "edges": int(m), "results": rows}


def single_gpu_configs(peak: float, only=None, with_cpu: bool = True, c3_log2_rows: int = 24) -> list:
    import torch
    from flexspmv_b200 import graphs, problems
    from flexspmv_b200.binding import GraphExtension
    dev = torch.device("cuda", torch.cuda.current_device())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = []

    def upload(ir, prob):
        non_gather, gathers, index_names = graphs.operator_signature(ir)
        vals = [torch.from_numpy(np.ascontiguousarray(prob.values[n])).to(dev) for n in non_gather + gathers]
        idxs = [torch.from_numpy(np.ascontiguousarray(prob.indices[n])).to(dev) for n in index_names]
        ro = torch.from_numpy(np.ascontiguousarray(prob.row_offsets)).to(dev)
        return vals, idxs, ro

    # (id for --only-config, name, graph, inputs, value bytes, iterations); id 5 is not a BASELINE config: the fused
    # `delta` graph of the reference's own shallow-water model on the config-2 mesh
    specs = [(0, "config0 2D Poisson 512^2 fp64", "spmv", lambda: problems.poisson2d(512), 8, 200),
             (1, "config1 spring-mass 1024^2 fp32", "spring_mass", lambda: problems.spring_mass(1024), 4, 200),
             (2, "config2 shallow-water Rusanov 1024^2 fp64", "rusanov", lambda: problems.shallow_water(1024), 8, 200),
             (5, "reference shallow-water model, fused delta graph, 1024^2 mesh fp64", "swe_delta",
              lambda: problems.swe_mesh(1024), 8, 200)]
    for ci, name, gname, make, vb, iters in specs:
        if only is not None and ci not in only:
            continue
        ir = graphs.ALL_GRAPHS[gname]()
        prob = make()
        vals, idxs, ro = upload(ir, prob)
        dt = vals[0].dtype
        outs = [torch.empty((prob.num_rows,) + (() if graphs.dim_of(o["shape"]) == 1 else (graphs.dim_of(o["shape"]),)),
                            dtype=dt, device=dev) for o in ir.outputs]
        alg = problems.algorithmic_bytes(ir, prob.num_rows, prob.nnz, prob.num_cols, vb, 4)
        entry = time_config(name, ir, GraphExtension(ir), vals, idxs, ro, outs, prob.num_rows, prob.nnz, prob.num_cols,
                            alg, iters, peak, flush)
        if with_cpu:
            cpu_beside(entry, ir, prob, np.float32 if vals[0].dtype == torch.float32 else np.float64, [o.cpu().numpy() for o in outs])
        out.append(entry)
        del vals, idxs, ro, outs
    # ids 6, 7 (not BASELINE configs): the aggregator / map-only flavour (flex_edge_kernel) on 2^27 edges whose
    # selector walks a 2^24-vertex tensor in order (8 edges per vertex): a per-edge product + global sum, fp32,
    # and a gather written in place through an input pointer, fp64
    E, NV = 1 << 27, 1 << 24
    for ci, name, gname, dt, vb in ((6, "aggregator graph edge_sum (per-edge product + global sum), 2^27 edges fp32", "edge_sum", torch.float32, 4),
                                    (7, "map-only graph edge_copy (gather written in place), 2^27 edges fp64", "edge_copy", torch.float64, 8)):
        if only is not None and ci not in only:
            continue
        ir = graphs.ALL_GRAPHS[gname]()
        gen = torch.Generator(device=dev)
        gen.manual_seed(60 + ci)
        edge = torch.rand(E, 2, generator=gen, device=dev, dtype=dt)
        vert = torch.rand(NV, 2, generator=gen, device=dev, dtype=dt)
        sel = (torch.arange(E, device=dev, dtype=torch.int64) // (E // NV)).to(torch.int32)
        dummy = torch.tensor([42], dtype=torch.int32, device=dev)
        outs = [torch.empty(E, 2, device=dev, dtype=dt), torch.empty(2, device=dev, dtype=dt)] if gname == "edge_sum" else []
        alg = problems.algorithmic_bytes(ir, 0, E, NV, vb, 4)
        out.append(time_config(name, ir, GraphExtension(ir), [edge, vert], [sel], dummy, outs, 0, E, NV, alg, 20, peak, flush))
        del edge, vert, sel, outs
        torch.cuda.empty_cache()
    if only is not None and 3 not in only:
        return out
    # config 3 is generated on the device (268 M non-zeros)
    ir = graphs.spmv_graph()
    ro, cols, vals, x = problems.powerlaw_device(1 << c3_log2_rows, 3, dev)
    n, m = x.numel(), cols.numel()
    y = torch.empty(n, dtype=torch.float32, device=dev)
    alg = problems.algorithmic_bytes(ir, n, m, n, 4, 4)
    entry = time_config(f"config3 power-law CSR n=2^{c3_log2_rows} fp32", ir, GraphExtension(ir), [vals, x], [cols], ro, [y], n, m, n, alg,
                        50, peak, flush)
    if with_cpu:
        # the full-size arrays go to the host once (2.2 GB) and through the reference's CPU operator; the error scale
        # (sum of |a_ij x_j| per row) is an independent torch reduction on the device
        rid = torch.repeat_interleave(torch.arange(n, device=dev, dtype=torch.int32), (ro[1:] - ro[:-1]).long())
        abs_sum = torch.zeros(n, dtype=torch.float32, device=dev).index_add_(0, rid.long(), (vals * x[cols.long()]).abs())
        del rid
        prob = problems.Problem("spmv", {"vals": vals.cpu().numpy(), "x": x.cpu().numpy()}, {"selector": cols.cpu().numpy()},
                                ro.cpu().numpy(), n, n, {"config": 3})
        cpu_beside(entry, ir, prob, np.float32, [y.cpu().numpy()], abs_sums=[abs_sum.cpu().numpy()], steps=5)
        del prob, abs_sum
    out.append(entry)
    del ro, cols, vals, x, y, flush
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------------------
# result check of the partitioned iteration (every N)
# --------------------------------------------------------------------------------------------------
def stencil_reference(x_local, plan, n: int):
    """The 7-point stencil (6 on the diagonal, -1 off it, Dirichlet) applied with torch slicing to one rank's local
    vector [halo below | owned planes | halo above]; a missing halo (first / last rank) is the zero boundary."""
    import torch
    n2 = n * n
    planes = plan.rows // n2
    X = torch.zeros((planes + 2) * n2, dtype=x_local.dtype, device=x_local.device)
    off = n2 - plan.halo_lo
    X[off:off + plan.local_len] = x_local
    X = X.view(planes + 2, n, n)
    C = X[1:-1]
    ref = 6.0 * C - X[:-2] - X[2:]
    ref[:, 1:, :] -= C[:, :-1, :]
    ref[:, :-1, :] -= C[:, 1:, :]
    ref[:, :, 1:] -= C[:, :, :-1]
    ref[:, :, :-1] -= C[:, :, 1:]
    return ref.reshape(-1)


def verify_iteration(op, plan, n: int, rank: int, world: int, use_graph: bool, steps: int = 3) -> dict:
    """After the timed region, on the same operator object: the owned vector is reset to a seeded U(-1,1) vector and
    `steps` iterations are checked, each against the stencil applied to the rank's [halo | owned | halo] vector
    (halos exchanged first).  With a captured graph, one replayed pair must also equal two eager steps bit for bit.
    The largest error over all ranks, relative to 12 max|x| (the bound of a row's sum of term magnitudes)."""
    import torch
    import torch.distributed as dist
    from flexspmv_b200 import multi_gpu
    dev = op.buf[0].device
    g = torch.Generator(device=dev)
    g.manual_seed(977 + rank)
    for b in op.buf:
        b.zero_()
    op.owned().copy_(torch.rand(plan.rows, generator=g, device=dev, dtype=torch.float64) * 2.0 - 1.0)
    worst = 0.0
    for _ in range(steps):
        x = op.buf[op.cur]
        multi_gpu.exchange_halos(x, plan, op.group)
        ref = stencil_reference(x, plan, n)
        scale = 12.0 * float(x.abs().max())
        y = op.step()
        worst = max(worst, float((y - ref).abs().max()) / max(scale, 1e-300))
        del ref
    graph_equal = None
    if use_graph:
        if op.cur != 0:
            op.step()
        start = op.owned().clone()
        op.step_pair()                       # replays the captured pair
        replayed = op.owned().clone()
        op.owned().copy_(start)
        if op.overlap:
            op.refresh_halos()               # the halos in place belong to the replayed state
        op.step()
        op.step()
        graph_equal = bool(torch.equal(op.owned(), replayed))
    t = torch.tensor([worst, 0.0 if graph_equal in (None, True) else 1.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    err, graph_bad = float(t[0].item()), bool(t[1].item() > 0)
    out = {"max_row_err": err, "tol": 1e-12, "steps": steps, "ok": bool(err <= 1e-12 and not graph_bad),
           "against": "7-point stencil applied by torch slicing to each rank's [halo | owned | halo] vector"}
    if use_graph:
        out["graph_replay_equals_eager"] = not graph_bad
    return out


# --------------------------------------------------------------------------------------------------
# the CUDA arm
# --------------------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from flexspmv_b200 import multi_gpu
    from flexspmv_b200.binding import load_builtin

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    peak, peak_kind = load_peaks()
    if args.probe_gather:                 # measurement aid: the gather bound of the chip on the config-3 arrays
        print(json.dumps(probe_gather(args.config3_log2_rows)), flush=True)
        return
    if args.only_config is not None:      # profiling aid: one single-GPU configuration, nothing else
        print(json.dumps({"configs": single_gpu_configs(peak, only=[args.only_config], with_cpu=not args.no_cpu,
                                                        c3_log2_rows=args.config3_log2_rows)}), flush=True)
        return
    n = args.grid
    n2 = n * n
    K, W = args.steps, max(args.warmup, 3)

    # ---- partition + local matrix -----------------------------------------------------------------
    bounds = multi_gpu.poisson3d_slab_bounds(n, world, dev)
    z0, z1 = bounds[rank], bounds[rank + 1]
    first_row = [b * n2 for b in bounds]
    min_col = [max(0, first_row[r] - n2) if first_row[r + 1] > first_row[r] else first_row[r] for r in range(world)]
    max_col = [min(n ** 3, first_row[r + 1] + n2) - 1 if first_row[r + 1] > first_row[r] else first_row[r] - 1 for r in range(world)]
    plan = multi_gpu.make_halo_plans(first_row, min_col, max_col)[rank]
    ro, cols, vals = multi_gpu.poisson3d_planes_device(n, z0, z1, dev, col_shift=plan.col_shift)
    g = torch.Generator(device=dev)
    g.manual_seed(4 * 1000 + rank)
    x0 = torch.rand(plan.rows, generator=g, device=dev, dtype=torch.float64) * 2.0 - 1.0
    ext = load_builtin("spmv")
    # measured on 8 B200s (512^3): 0.459 ms/step with the exchange in front of one launch, 0.432 ms with the boundary rows
    # first and the exchange behind the interior launch; at 2 GPUs the split costs more than it hides (1.633 against 1.608 ms)
    overlap = (world >= 4) if args.overlap is None else bool(args.overlap)
    op = multi_gpu.PartitionedSpmv(plan, ro, cols, vals, x0, ext=ext, overlap=overlap, overlap_spare_ctas=args.spare_ctas)
    alg_bytes, nnz_total = poisson3d_bytes(n)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def renorm(step_index: int) -> int:
        # ||A|| <= 12: rescale before the iterate can overflow fp64 (one tiny extra kernel every 200 steps)
        if step_index and step_index % 200 == 0:
            op.owned().mul_(2.0 ** -700)
            if op.overlap:
                op.refresh_halos()       # the halos were sent before the rescaling
            return 1
        return 0

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()          # nvidia-smi needs a moment to start: begin before the warm-up
    for i in range(W + (W % 2)):     # an even number of warm-up steps: the captured pair starts from buffer 0
        op.step()
    use_graph = world > 1 and not args.no_graph and K % 2 == 0 and K <= 200
    graph_error = None
    if use_graph:
        flag = torch.tensor([1 if op.capture_pair() else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)          # all ranks replay, or none does
        use_graph = bool(flag.item())
        graph_error = op.graph_error
        if not use_graph:
            op.graph = None
            if graph_error is None:
                graph_error = "capture failed on another rank"
    barrier()
    if rank == 0:
        sampler.mark_begin()
    launches0 = ext.launches
    extra = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    if use_graph:
        for i in range(K // 2):
            op.step_pair()
    else:
        for i in range(K):
            extra += renorm(W + i)
            op.step()
    e1.record()
    barrier()
    ext.check()          # raises if a kernel of the timed region gave up (bounded wait ran out, workspace not planned)
    timed_launches = (K * op.launches_per_step) if use_graph else (ext.launches - launches0 + extra)
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms = float(ms.item())
    if rank == 0:
        sampler.mark_end()
    # a timed region of a few tens of milliseconds can fall between two nvidia-smi samples: keep the same
    # workload running (untimed) until a handful of samples under load exist, and say so in the line
    extra_steps = 0
    t_wait = time.time()
    while True:
        need = torch.tensor([1 if (rank == 0 and sampler.under_load() < 4 and time.time() - t_wait < 3.0) else 0], device=dev)
        if world > 1:
            dist.broadcast(need, 0)
        if int(need.item()) == 0:
            break
        for _ in range(20):
            op.step()
        extra_steps += 20
        torch.cuda.synchronize()
    clocks = sampler.stop(extra_steps) if rank == 0 else None
    launches = torch.tensor([timed_launches], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(launches)
    ms_per_step = total_ms / K
    value = alg_bytes / ms_per_step / 1e6     # GB/s over the whole job
    ext.check()
    check = verify_iteration(op, plan, n, rank, world, use_graph)
    ext.check()

    # ---- end to end through the reference-facing operator with host buffers ---------------------------
    # Every step: pinned-host x -> device, halo exchange, merged_spmv_launch (allocates y), y -> pinned host.
    # Steps alternate between two CUDA streams with their own device and host buffers, so the y download of
    # one step overlaps the x upload of the next (PCIe is full duplex); every step still does both copies.
    E = max(2, min(K, args.e2e_steps))
    E += E % 2
    hx = torch.empty(plan.rows, dtype=torch.float64).pin_memory()
    hx.copy_(x0.cpu())
    lo = plan.halo_lo
    lanes = []
    n_lanes = args.e2e_lanes
    for i in range(n_lanes):      # every rank issues its lanes in the same order, so the NCCL exchanges pair up across ranks
        lanes.append({"stream": torch.cuda.Stream() if n_lanes > 1 else torch.cuda.current_stream(),
                      "xbuf": op.buf[i] if i < 2 else torch.zeros_like(op.buf[0]),
                      "hy": torch.empty(plan.rows, dtype=torch.float64).pin_memory()})

    def e2e_step(i):
        ln = lanes[i % len(lanes)]
        with torch.cuda.stream(ln["stream"]):
            xb = ln["xbuf"]
            xb[lo:lo + plan.rows].copy_(hx, non_blocking=True)               # host -> device: this step's input vector
            multi_gpu.exchange_halos(xb, plan)
            (y,) = ext.merged_spmv_launch(vals, xb, cols, ro, plan.rows, plan.local_len)   # the operator the reference wrapper calls
            ln["hy"].copy_(y, non_blocking=True)                             # device -> host: the step's result

    for ln in lanes:
        ln["stream"].wait_stream(torch.cuda.current_stream())
    for i in range(max(2, n_lanes)):
        e2e_step(i)
    barrier()
    a0 = torch.cuda.Event(enable_timing=True)
    a0.record()
    for ln in lanes:
        ln["stream"].wait_event(a0)
    for i in range(E):
        e2e_step(i)
    for ln in lanes:
        torch.cuda.current_stream().wait_stream(ln["stream"])
    a1 = torch.cuda.Event(enable_timing=True)
    a1.record()
    barrier()
    ems = torch.tensor([a0.elapsed_time(a1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ems, op=dist.ReduceOp.MAX)
    e2e_ms = float(ems.item()) / E
    ext.check()
    hb = torch.tensor([plan.rows * 8], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(hb)
    xbuf = lanes[0]["xbuf"]
    e2e = {"value": alg_bytes / e2e_ms / 1e6, "unit": UNIT, "h2d_bytes_per_step": int(hb.item()), "d2h_bytes_per_step": int(hb.item()),
           "ms_per_step": e2e_ms, "steps": E, "streams": len(lanes),
           "what": "per step: pinned-host x -> device, halo exchange, merged_spmv_launch (allocates y), y -> pinned host; steps "
                   "alternate between the streams so one step's download overlaps the next step's upload; "
                   "the CSR matrix is static across iterations and stays resident"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": workload_config(n),
        "run": {"arm": "hand-written sm_100a kernels behind the C ABI, int64 row offsets, iterated as x <- A x with one z-plane "
                       "halo per neighbour per iteration",
                "partition": f"{world} nnz-balanced z-slab(s), merge-path tile plan cached across iterations",
                "halo_overlap": bool(op.overlap), "launches_per_step_per_rank": op.launches_per_step,
                "cuda_graph": bool(use_graph), "cuda_graph_error": graph_error,
                "halo_bytes_per_neighbour_per_direction": n2 * 8 if world > 1 else 0},
        "edges_per_s": nnz_total / ms_per_step * 1e3,
        "frac_of_hbm_peak": value / (peak * world), "hbm_peak_gbs_per_gpu": peak, "hbm_peak_kind": peak_kind,
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches.item()), "check": check, "device_status": 0,
    }
    if world == 1:
        info = ext.symbols(torch.float64).graph_info
        line["roofline"] = {"bound": "hbm", "achieved": value, "peak": peak, "unit": UNIT, "frac": value / peak, "traffic": None,
                            "kernel": "flex_tile_kernel<spmv_f64, int64 offsets>", "peak_kind": f"of {peak_kind}",
                            "launch_ms": ms_per_step, "algorithmic_bytes_per_launch": alg_bytes,
                            "tile": {"block": info.block_threads, "items_per_thread": info.items_per_thread,
                                     "stages": info.stages, "smem_bytes": info.smem_bytes}}
        ratio = (DRAM_CAPTURE["read_bytes"] + DRAM_CAPTURE["write_bytes"]) / DRAM_CAPTURE["algorithmic_bytes"]
        line["roofline"]["traffic"] = ratio * alg_bytes
        line["roofline"]["traffic_source"] = (
            f"one ncu capture of this kernel on the {DRAM_CAPTURE['grid']}^3 grid: {DRAM_CAPTURE['read_bytes'] / 1e6:.1f} MB read + "
            f"{DRAM_CAPTURE['write_bytes'] / 1e6:.1f} MB written for {DRAM_CAPTURE['algorithmic_bytes'] / 1e6:.1f} MB of algorithmic "
            f"bytes ({ratio:.3f} x; part of y was still in L2 when the capture ended), scaled by algorithmic bytes")
        del op, ro, cols, vals, x0, xbuf
        torch.cuda.empty_cache()
        if not args.no_configs:
            line["configs"] = single_gpu_configs(peak, with_cpu=not args.no_cpu)
        if not args.no_cpu:
            r = cpu_reference(n, 5, 1, planes=args.cpu_planes)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
            line["cpu_baseline"]["edges_per_s"] = r["edges_per_s"]
    if rank == 0:
        print(json.dumps(line), flush=True)
    if not check["ok"]:
        sys.stderr.write(f"bench.py: result check failed: {check}\n")
        sys.stderr.flush()
        sys.stdout.flush()
        os._exit(1)          # no communicator teardown (see below); a failed check is a failed run
    if world > 1:
        # A captured graph holds NCCL kernels; tearing the communicator down under it has hung at exit.
        # Everything is measured and printed: drop the graph, meet once more, and leave without the
        # interpreter's teardown.
        op.graph = None
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--grid", type=int, default=512)
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--e2e-lanes", type=int, default=2, choices=[1, 2, 3, 4],
                    help="end-to-end loop: steps alternate between this many streams (one step's download overlaps the next upload)")
    ap.add_argument("--no-configs", action="store_true", help="skip the per-configuration table (N = 1)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs (N = 1)")
    ap.add_argument("--cpu-planes", type=int, default=None,
                    help="CPU arm: time this many z-planes of the matrix instead of the whole grid (hosts short of memory)")
    ap.add_argument("--only-config", type=int, default=None, choices=[0, 1, 2, 3, 5, 6, 7],
                    help="run just this single-GPU configuration (kernel-only timings) and print its entry")
    ap.add_argument("--overlap", dest="overlap", action="store_true", default=None,
                    help="N > 1: boundary rows first, halo exchange behind the interior launch (default: on from 4 GPUs)")
    ap.add_argument("--no-overlap", dest="overlap", action="store_false", help="N > 1: exchange halos in front of one launch per step")
    ap.add_argument("--spare-ctas", type=int, default=16, help="CTA slots the overlapped interior launch leaves to the communication kernel")
    ap.add_argument("--config3-log2-rows", type=int, default=24, help="rows of the power-law matrix of config 3 (profiling: 22)")
    ap.add_argument("--probe-gather", action="store_true",
                    help="print the chip's rate of random 4-byte gathers on the config-3 arrays for several shared-memory sizes")
    ap.add_argument("--no-graph", action="store_true", help="N > 1: enqueue every step from Python instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
