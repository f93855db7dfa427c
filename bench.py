#!/usr/bin/env python
"""Benchmark of the sparse-operator hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-ops]

Workload (``config.workload``): hybrid-format SpMM Y = A X on the synthetic power-law graph
(169,343 nodes, row degrees Zipf(2.1) clipped to [1, 13000], preferential-attachment columns,
values 1/deg), decomposed into ELL buckets of width 1..512.  One step is one pass over the five
feature sizes F = 32, 64, 128, 256, 512: five calls of ``sparsetir_hyb_spmm``, each on its own
X / Y buffers (1.3 GB touched per step, ten times the L2, so no call finds its operands cached).

``value`` is GFLOP/s (2 * nnz * F summed over the five F, divided by the step time) with every
operand resident in HBM.  ``e2e`` is the same work with X in pinned host memory copied in and Y
copied back to pinned host memory inside the timed region.  With N > 1 the rows are cut into
nnz-balanced contiguous shards, one per rank (strong scaling on the same graph); ``value`` times
the shard kernels (max over ranks); for ``e2e`` every rank copies its 1/N slice of X from its own
pinned host memory, the slices are all-gathered over NCCL, and the shard's output rows go back to
the rank's pinned host memory.

``--impl reference`` times the CPU restatement of the reference's lowered loop nest (the
oracle's OpenMP csrmm — what the reference's ``llvm`` target would run, parallel over rows)
on the same graph and feature sizes, on the host cores of rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FEATS = (32, 64, 128, 256, 512)
BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)
WORKLOAD = "hyb_spmm_powerlaw_169343_F32-512"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["source"] = "fallback"
    return d


def spmm_bytes(n_rows, n_cols, nnz, feat):
    """Compulsory traffic of one SpMM: indptr + (index, value) per entry + X once + Y once."""
    return 4 * (n_rows + 1) + 8 * nnz + 4 * n_cols * feat + 4 * n_rows * feat


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------
def reference_arm(args, rank, world):
    """CPU implementation of the path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    from oracle import oracle as orc
    from sparsetir_b200 import datagen as dg

    g = dg.csr_powerlaw(seed=0)
    xs = {f: dg.dense_operand(100 + f, g.n, f) for f in FEATS}
    ys = {f: np.zeros((g.m, f), np.float32) for f in FEATS}
    cores = orc.use_all_cores()
    flops = sum(2.0 * g.nnz * f for f in FEATS)

    def step():
        for f in FEATS:
            orc.csrmm(g.data, xs[f], ys[f], g.indptr, g.indices, g.m, g.n, f, omp=True)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = flops / dt / 1e9
    line = {
        "impl": "reference", "metric": "hyb_spmm_gflops", "value": val, "unit": "GFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "nnz": g.nnz, "feats": list(FEATS),
                   "note": "CPU restatement of the reference's lowered csrmm loop nest, OpenMP over rows"},
        "cpu_baseline": {"value": val, "unit": "GFLOP/s", "cores": cores, "kind": "port",
                         "sample": "whole workload: all five feature sizes on the full graph"},
        "e2e": {"value": val, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
def ours_arm(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    from sparsetir_b200 import _lib as L
    from sparsetir_b200 import datagen as dg
    from sparsetir_b200 import dist as sdist
    from sparsetir_b200 import format as fmt
    from sparsetir_b200 import ops

    L.load()  # fails loudly if the CUDA library is missing
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(device)

    # ---- workload: same seeded graph on every rank, row shard per rank
    g = dg.csr_powerlaw(seed=0)
    shard = sdist.shard_csr(g.indptr, g.indices, g.data, g.n, world, rank)
    cuts, ip, ix, vals_csr = shard.cuts, shard.indptr, shard.indices, shard.data
    m_loc, nnz_loc = shard.num_rows, shard.nnz
    parts = args.parts
    t0 = time.perf_counter()
    rows, cols, mask, vals, _ = fmt.column_part_hyb(m_loc, g.n, ip, ix, parts, BUCKETS, data=vals_csr)
    decompose_ms = (time.perf_counter() - t0) * 1e3
    # one column partition: every output row has one writer, nothing to clear between calls;
    # several: everything is added atomically into a C that the call clears first
    flags = (L.HYB_REARM | L.HYB_ALL_ATOMIC) if parts > 1 else 0
    devb = [(dev(vals[p][b]), dev(rows[p][b]), dev(cols[p][b]))
            for p in range(parts) for b in range(len(BUCKETS))]
    slots = sum(int(c[2].numel()) for c in devb)

    x_host = {f: torch.from_numpy(dg.dense_operand(100 + f, g.n, f)).pin_memory() for f in FEATS}
    x_dev = {f: x_host[f].to(device) for f in FEATS}
    y_dev = {f: torch.zeros(m_loc * f, device=device) for f in FEATS}
    calls = {f: ops.hyb_spmm.prepare(*ops.hyb_args(x_dev[f], y_dev[f], devb, f, flags)) for f in FEATS}
    launches_per_call = 1  # one kernel for all buckets (plus a driver memset with several partitions)

    def step(events=None):
        for f in FEATS:
            if events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            calls[f]()
            if events is not None:
                e1.record()
                events[f].append((e0, e1))

    # ---- device-resident timing
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    events = {f: [] for f in FEATS}
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        step(events)
    stop.record()
    barrier()
    ms_total = start.elapsed_time(stop)

    # The same K steps replayed from a CUDA graph (the calls neither allocate nor synchronise,
    # so a step can be captured): takes the per-launch host work out of the measurement.
    graph_ms = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg):
            step()
        for _ in range(3):
            cg.replay()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps):
            cg.replay()
        g1.record()
        barrier()
        graph_ms = g0.elapsed_time(g1) / args.steps
    except Exception as exc:  # capture is an extra; the eager number stands on its own
        log(f"bench.py: graph replay skipped: {exc!r}")
    if args.kernels_only:  # short run for profilers: no clock sampling tail, e2e, CPU or ops legs
        if rank == 0:
            sampler.stop()
            print(json.dumps({"kernels_only": True, "ms_per_step": ms_total / args.steps,
                              "graph_replay_ms_per_step": graph_ms,
                              "per_feat_ms": {str(f): statistics.mean(a.elapsed_time(b) for a, b in events[f])
                                              for f in FEATS}}), flush=True)
        return
    # keep the GPU busy a little longer so the clock sampler sees the loaded state
    t_end = time.perf_counter() + (1.0 if rank == 0 else 0.0)
    extra = 0
    while time.perf_counter() < t_end:
        step()
        extra += 1
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    per_f_ms = {f: statistics.mean(a.elapsed_time(b) for a, b in events[f]) for f in FEATS}
    ms_step = ms_total / args.steps
    if world > 1:
        t = torch.tensor([ms_step], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item())
        tf = torch.tensor([per_f_ms[f] for f in FEATS], device=device)
        dist.all_reduce(tf, op=dist.ReduceOp.MAX)
        per_f_ms = {f: float(v) for f, v in zip(FEATS, tf.tolist())}
    total_flops = sum(2.0 * g.nnz * f for f in FEATS)
    # `value` is taken from the graph replay of the same K steps when the capture worked (max over
    # ranks like the eager figure): it times the kernels of the step without the Python call
    # overhead between launches; the eager figure is kept beside it.
    eager_ms_step = ms_step
    launch_mode = "eager"
    if world > 1:  # every rank takes part, whether or not its own capture worked
        t = torch.tensor([graph_ms if graph_ms is not None else -1.0], device=device)
        t_max, t_min = t.clone(), t.clone()
        dist.all_reduce(t_max, op=dist.ReduceOp.MAX)
        dist.all_reduce(t_min, op=dist.ReduceOp.MIN)
        graph_ms = float(t_max.item()) if float(t_min.item()) >= 0 else None
    if graph_ms is not None:
        ms_step, launch_mode = graph_ms, "cuda_graph_replay"
    value = total_flops / (ms_step * 1e-3) / 1e9

    # ---- end to end: X from pinned host memory, Y back to pinned host memory.
    # One GPU: the whole X in, the whole Y out.  N GPUs: every rank owns an equal slice of the
    # rows of X in ITS pinned host memory and the rows of Y of its shard; per step it copies its
    # slice in over its own PCIe link, the slices are all-gathered over NVLink (NCCL), the shard
    # kernels run, and the shard's output rows go back to the rank's pinned host memory.  The
    # bytes per step are the same as with one GPU; they are spread over N links.
    xcuts = [(g.n * k) // world for k in range(world + 1)]
    xr0, xr1 = xcuts[rank], xcuts[rank + 1]
    x_host_loc = ({f: x_host[f].reshape(-1)[xr0 * f:xr1 * f].clone().pin_memory() for f in FEATS}
                  if world > 1 else x_host)
    y_host = {f: torch.empty(m_loc * f, dtype=torch.float32).pin_memory() for f in FEATS}

    # Three streams so that the PCIe link runs in both directions while kernels execute: the
    # copy-in of feature size k+1 and the copy-out of k-1 overlap the kernels of k.  Events order
    # every buffer's copy-in -> kernel -> copy-out, and the reuse of the buffers by the next step.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = {f: torch.cuda.Event() for f in FEATS}
    ev_done = {f: torch.cuda.Event() for f in FEATS}
    ev_out = {f: torch.cuda.Event() for f in FEATS}
    for f in FEATS:
        ev_done[f].record(main)
        ev_out[f].record(main)

    def e2e_step():
        for f in FEATS:
            s_in.wait_event(ev_done[f])       # previous step's kernels have read x_dev[f]
            with torch.cuda.stream(s_in):
                if world == 1:
                    x_dev[f].copy_(x_host[f], non_blocking=True)
                else:
                    piece = x_dev[f].view(-1)[xr0 * f:xr1 * f]
                    piece.copy_(x_host_loc[f], non_blocking=True)
                    sdist.all_gather_blocks(piece, [(xcuts[k + 1] - xcuts[k]) * f for k in range(world)],
                                            out=x_dev[f].view(-1))
                ev_in[f].record(s_in)
        for f in FEATS:
            main.wait_event(ev_in[f])
            main.wait_event(ev_out[f])        # previous step's copy-out has read y_dev[f]
            calls[f]()
            ev_done[f].record(main)
            s_out.wait_event(ev_done[f])
            with torch.cuda.stream(s_out):
                y_host[f].copy_(y_dev[f], non_blocking=True)
                ev_out[f].record(s_out)
        main.wait_event(ev_out[FEATS[-1]])    # the step ends when its last result is on the host

    for _ in range(2):
        e2e_step()
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_steps = max(3, min(args.steps, 10))
    e_start.record()
    for _ in range(e_steps):
        e2e_step()
    e_stop.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_stop) / e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    h2d = sum(4 * g.n * f for f in FEATS)
    d2h = sum(4 * g.m * f for f in FEATS)

    # ---- N > 1: the shard kernels followed by the all-gather of the output rows (device-resident X)
    gather_ms = None
    if world > 1:
        shard_rows = [int(cuts[k + 1] - cuts[k]) for k in range(world)]
        y_all = {f: torch.empty(g.m * f, device=device) for f in FEATS}

        def gather_step():
            for f in FEATS:
                calls[f]()
                sdist.all_gather_rows(y_dev[f], shard_rows, f, out=y_all[f])

        for _ in range(2):
            gather_step()
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(e_steps):
            gather_step()
        a1.record()
        barrier()
        t = torch.tensor([a0.elapsed_time(a1) / e_steps], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gather_ms = float(t.item())
        del y_all

    # ---- the largest graph of the benchmark set (SDDMM, 1.2e8 positions) sharded the same way:
    # collective, so every rank runs it; rank 0 reports it
    ops_sharded = None
    if world > 1 and args.ops:
        try:
            from sparsetir_b200 import opbench
            ops_sharded = {"sddmm": opbench.bench_sddmm_sharded(device, peaks, rank, world)}
        except Exception as e:  # the headline line must still be printed
            ops_sharded = {"error": repr(e)}

    if rank != 0:
        return

    # ---- sanity: the timed result is the right one (device result vs CPU oracle, one F)
    from oracle import oracle as orc
    f_chk = 64 if 64 in FEATS else FEATS[0]
    want = np.zeros((g.m, f_chk), np.float32)
    orc.csrmm(g.data, x_host[f_chk].numpy(), want, g.indptr, g.indices, g.m, g.n, f_chk, omp=True)
    got = y_host[f_chk].numpy().reshape(m_loc, f_chk)  # rank 0 holds the rows of its shard
    np.testing.assert_allclose(got, want[int(cuts[0]):int(cuts[1])], rtol=1e-4, atol=1e-5)

    # ---- roofline of the dominant launch (F = 512)
    f_dom = FEATS[-1]
    alg_bytes = spmm_bytes(m_loc, g.n, nnz_loc, f_dom)
    achieved = alg_bytes / (per_f_ms[f_dom] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"],
                # dram__bytes_read.sum + dram__bytes_write.sum of this launch from the committed ncu
                # capture of the same workload (the F = 512 summary in the profiles folder), one GPU
                "traffic": 703.8e6 if (world == 1 and FEATS[-1] == 512) else None,
                "peak_source": peaks["source"],
                "kernel": "hyb_spmm_lean_kernel<32> (+ hyb_rearm_kernel), F=512 call",
                "algorithmic_bytes": alg_bytes, "launch_ms": per_f_ms[f_dom]}
    per_f = {}
    for f in FEATS:
        byts = spmm_bytes(m_loc, g.n, nnz_loc, f)
        per_f[str(f)] = {"ms": per_f_ms[f], "gflops": 2.0 * g.nnz * f / (per_f_ms[f] * 1e-3) / 1e9,
                         "alg_gbs": byts / (per_f_ms[f] * 1e-3) / 1e9,
                         "hbm_frac": byts / (per_f_ms[f] * 1e-3) / 1e9 / peaks["hbm_gbs"]}

    # ---- CPU baseline on the host cores (bounded sample)
    cpu = None
    if world == 1 or True:
        cores = orc.use_all_cores()
        ys = {f: np.zeros((g.m, f), np.float32) for f in FEATS}
        xs = {f: x_host[f].numpy() for f in FEATS}

        def cpu_step():
            for f in FEATS:
                orc.csrmm(g.data, xs[f], ys[f], g.indptr, g.indices, g.m, g.n, f, omp=True)

        cpu_step()
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or (time.perf_counter() - t0 < 5.0 and reps < 50):
            cpu_step()
            reps += 1
        cdt = (time.perf_counter() - t0) / reps
        cpu = {"value": total_flops / cdt / 1e9, "unit": "GFLOP/s", "cores": cores, "kind": "port",
               "sample": f"whole workload ({reps} passes over all five feature sizes, OpenMP csrmm)"}

    line = {
        "metric": "hyb_spmm_gflops", "value": value, "unit": "GFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "nodes": g.m, "nnz": g.nnz, "feats": list(FEATS),
                   "col_parts": parts, "buckets": list(BUCKETS), "ell_slots_rank0": slots,
                   "launch": launch_mode,
                   "l2": "inputs larger than L2: each step touches 1.3 GB over five X/Y pairs",
                   "sharding": "nnz-balanced contiguous row shards, one per GPU",
                   "host_decompose_ms_rank0": decompose_ms},
        "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e9, "unit": "GFLOP/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "includes": "H2D of X, kernels, D2H of Y" + (
                    "; every rank copies its 1/N slice of X from its own pinned host memory, NCCL "
                    "all-gather of the slices, shard kernels, D2H of the shard's output rows to the "
                    "rank's pinned host memory" if world > 1 else "")},
        "gpu_launches": launches_per_call * len(FEATS) * args.steps,
        "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks, "per_feat": per_f,
        "graph_replay_ms_per_step": graph_ms, "eager_ms_per_step": eager_ms_step,
        "ms_per_step_with_allgather_of_y": gather_ms,
        "alg_gbs": sum(spmm_bytes(m_loc, g.n, nnz_loc, f) for f in FEATS) / (ms_step * 1e-3) / 1e9,
    }
    if ops_sharded is not None:
        line["ops_sharded"] = ops_sharded
    if args.ops and world == 1:
        try:
            from sparsetir_b200 import opbench
            line["ops"] = opbench.run_all(device, peaks, log)
        except Exception as e:  # the headline line must still be printed
            line["ops"] = {"error": repr(e)}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--parts", type=int, default=1, help="column partitions of the hyb format")
    ap.add_argument("--no-ops", dest="ops", action="store_false",
                    help="skip the per-operator table (CSR SpMM, SDDMM, BSR, RGMS)")
    ap.add_argument("--feats", default=None,
                    help="comma-separated feature sizes (default: the workload's 32,64,128,256,512)")
    ap.add_argument("--kernels-only", action="store_true",
                    help="time the device-resident steps and stop (for profiler captures)")
    ap.add_argument("--only-op", default=None, choices=["csrmm", "bsrmm", "rgms", "rgms_ell3d", "rgms_f16", "tcspmm", "sddmm"],
                    help="measure one of the other operators alone and stop (for profiler captures)")
    args = ap.parse_args()
    if args.feats:
        global FEATS
        FEATS = tuple(int(x) for x in args.feats.split(","))
    if args.only_op:
        import torch
        from sparsetir_b200 import opbench
        dev = torch.device("cuda", 0)
        peaks = load_peaks()
        if args.only_op == "sddmm":
            feats = FEATS if args.feats else (32,)
            print(json.dumps(opbench.bench_sddmm(dev, peaks, feats=feats)), flush=True)
        else:
            flush = torch.empty(2 * opbench.L2_BYTES, dtype=torch.uint8, device=dev)
            fn = getattr(opbench, "bench_" + args.only_op)
            print(json.dumps(fn(dev, peaks, flush)), flush=True)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        try:
            ours_arm(args, rank, world, local_rank)
        finally:
            dist.barrier()
            dist.destroy_process_group()
    else:
        if args.gpus > 1:
            log("bench.py: --gpus > 1 needs torchrun; running on one GPU")
        ours_arm(args, rank, 1, local_rank)


if __name__ == "__main__":
    main()
