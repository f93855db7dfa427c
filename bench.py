#!/usr/bin/env python
"""Benchmark of the sparse-operator hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-ops]

Workload (``config.workload``): hybrid-format SpMM Y = A X on the synthetic power-law graph
(169,343 nodes, row degrees Zipf(2.1) clipped to [1, 13000], preferential-attachment columns,
values 1/deg), decomposed into ELL buckets of width 1..512.  One step is one pass over the five
feature sizes F = 32, 64, 128, 256, 512: five calls of ``sparsetir_hyb_spmm``, each on its own
X / Y buffers (1.3 GB touched per step, ten times the L2, so no call finds its operands cached).

One GPU: ``value`` is GFLOP/s (2 * nnz * F summed over the five F, divided by the step time) with
every operand resident in HBM, the step replayed from a CUDA graph.  ``e2e`` is the same work with
X in pinned host memory copied in and Y copied back to pinned host memory inside the timed region.

N GPUs (strong scaling on the same graph): the rows are cut into nnz-balanced contiguous shards,
one per rank; X is replicated.  ``value`` times the step that ENDS WITH Y ALL-GATHERED on every
rank (shard kernels on one stream, the NCCL all-gather of each feature size queued behind its
kernel on another, largest feature size first so that its gather overlaps the other kernels);
the shard kernels alone are reported beside it (``kernel_only``).  For ``e2e`` every rank copies
its equal block of the rows of X from its own pinned host memory, the blocks are all-gathered over
NCCL, the shard kernels run, and the shard's output rows go back to the rank's pinned host memory.

``--impl reference`` times the CPU restatement of the reference's lowered loop nest (the
oracle's OpenMP csrmm — what the reference's ``llvm`` target would run, parallel over rows)
on the same graph and feature sizes, on the host cores of rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import re
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
NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool


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


def spmm_bytes(n_rows, x_rows, nnz, feat):
    """Compulsory traffic of one SpMM: indptr + (index, value) per entry + the x_rows rows of X
    the matrix references once + Y once."""
    return 4 * (n_rows + 1) + 8 * nnz + 4 * x_rows * feat + 4 * n_rows * feat


def common_config(g, parts):
    """The workload description both arms print (identical dictionaries)."""
    return {"workload": WORKLOAD, "nodes": g.m, "nnz": g.nnz, "feats": list(FEATS), "col_parts": parts,
            "buckets": list(BUCKETS),
            "l2": "inputs larger than L2: each step touches 1.3 GB over five X/Y pairs"}


def profiled_traffic(kernel: str, feat: int, nnz: int):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if that
    summary describes the same kernel instantiation, feature size and matrix; else None."""
    path = os.path.join(ROOT, "profiles", "hyb_spmm_lean_kernel_F512.md")
    try:
        with open(path) as f:
            text = f.read()
    except OSError:
        return None, None
    m = re.search(r"bench-traffic:\s*kernel=(\S+)\s+feat=(\d+)\s+nnz=(\d+)\s+dram_bytes_per_launch=(\d+)", text)
    if not m or m.group(1) != kernel or int(m.group(2)) != feat or int(m.group(3)) != nnz:
        return None, None
    return int(m.group(4)), "profiles/hyb_spmm_lean_kernel_F512.md"


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


def cpu_legs(g, xs, total_flops, seconds=5.0):
    """The oracle's csrmm on the host cores: OpenMP over rows on every core of the process, and
    the serial loop nest on one core (what the reference's unscheduled llvm lowering runs)."""
    from oracle import oracle as orc
    cores = orc.use_all_cores()
    ys = {f: np.zeros((g.m, f), np.float32) for f in FEATS}

    def step(omp):
        for f in FEATS:
            orc.csrmm(g.data, xs[f], ys[f], g.indptr, g.indices, g.m, g.n, f, omp=omp)

    step(True)
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < seconds and reps < 50):
        step(True)
        reps += 1
    par = (time.perf_counter() - t0) / reps
    step(False)
    sreps, t0 = 0, time.perf_counter()
    while sreps < 2 or (time.perf_counter() - t0 < seconds and sreps < 20):
        step(False)
        sreps += 1
    ser = (time.perf_counter() - t0) / sreps
    return {"value": total_flops / par / 1e9, "unit": "GFLOP/s", "cores": cores, "kind": "port",
            "sample": f"whole workload ({reps} passes over all five feature sizes, OpenMP csrmm over rows)",
            "serial_gflops": total_flops / ser / 1e9,
            "serial_sample": f"whole workload ({sreps} passes), the same loop nest on 1 core"}


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
        "data": "synthetic", "config": common_config(g, args.parts),
        "note": "CPU restatement of the reference's lowered csrmm loop nest, OpenMP over rows",
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
    from sparsetir_b200 import sharded

    lib = L.load()  # fails loudly if the CUDA library is missing
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def over_ranks(values, op):
        """Element-wise max / min over ranks of a list of floats."""
        if world == 1:
            return list(values)
        t = torch.tensor(list(values), device=device, dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return [float(v) for v in t.tolist()]

    MAX, MIN = dist.ReduceOp.MAX, dist.ReduceOp.MIN

    def timed(fn, steps, warm=2):
        """Mean ms per call of fn over `steps` calls between two events, max over ranks."""
        for _ in range(warm):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return over_ranks([e0.elapsed_time(e1) / steps], MAX)[0]

    # ---- workload: same seeded graph on every rank, row shard per rank
    g = dg.csr_powerlaw(seed=0)
    parts = args.parts
    t0 = time.perf_counter()
    op = sharded.ShardedHybSpmm(g.indptr, g.indices, g.data, g.n, BUCKETS, parts=parts, device=device)
    setup_ms = (time.perf_counter() - t0) * 1e3
    shard = op.shard
    m_loc, nnz_loc = shard.num_rows, shard.nnz
    slots = sum(int(c[2].numel()) for c in op.buckets)

    # X lives in a buffer padded to `world` equal row blocks (the layout replicate_rows gathers into)
    blk = sharded.row_block(g.n, world)
    x_host = {f: torch.from_numpy(dg.dense_operand(100 + f, g.n, f)).pin_memory() for f in FEATS}
    x_dev = {}
    for f in FEATS:
        x_dev[f] = torch.zeros(world * blk * f, device=device)
        x_dev[f][:g.n * f].copy_(x_host[f].reshape(-1))
    y_dev = {f: torch.zeros(m_loc * f, device=device) for f in FEATS}
    calls = {f: op.prepare(x_dev[f], y_dev[f], f) for f in FEATS}

    def step(events=None, order=FEATS):
        for f in order:
            if events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            calls[f]()
            if events is not None:
                e1.record()
                events[f].append((e0, e1))

    # ---- device-resident timing of the shard kernels
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
    eager_ms = start.elapsed_time(stop) / args.steps

    # The same K steps replayed from a CUDA graph (the calls neither allocate nor synchronise once
    # the stream's scratch exists): takes the per-launch host work out of the measurement.
    graph_ms = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg, stream=side):  # the stream whose scratch the warm-up step set up
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
    per_f_ms = {f: statistics.mean(a.elapsed_time(b) for a, b in events[f]) for f in FEATS}
    if args.kernels_only:  # short run for profilers: no clock sampling tail, e2e, CPU or ops legs
        if rank == 0:
            sampler.stop()
            print(json.dumps({"kernels_only": True, "ms_per_step": eager_ms,
                              "graph_replay_ms_per_step": graph_ms,
                              "per_feat_ms": {str(f): per_f_ms[f] for f in FEATS}}), flush=True)
        return
    # keep the GPU busy a little longer so the clock sampler sees the loaded state
    t_end = time.perf_counter() + (1.0 if rank == 0 else 0.0)
    while time.perf_counter() < t_end:
        step()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    eager_ms = over_ranks([eager_ms], MAX)[0]
    per_f_max = over_ranks([per_f_ms[f] for f in FEATS], MAX)
    per_f_min = over_ranks([per_f_ms[f] for f in FEATS], MIN)
    per_f_ms = dict(zip(FEATS, per_f_max))
    if world > 1:  # every rank takes part, whether or not its own capture worked
        hi = over_ranks([graph_ms if graph_ms is not None else -1.0], MAX)[0]
        lo = over_ranks([graph_ms if graph_ms is not None else -1.0], MIN)[0]
        graph_ms = hi if lo >= 0 else None
    kernel_ms = graph_ms if graph_ms is not None else eager_ms
    kernel_mode = "cuda_graph_replay" if graph_ms is not None else "eager"
    total_flops = sum(2.0 * g.nnz * f for f in FEATS)

    # ---- N > 1: the step that ends with Y all-gathered on every rank.  Largest feature size first:
    # its gather (half of all bytes) overlaps the kernels of the others.
    gather_ms = nvlink = y_all = None
    if world > 1:
        y_all = {f: sharded.peer_empty(g.m * f, torch.float32, device) for f in FEATS}
        order = tuple(sorted(FEATS, reverse=True))

        gathered = {f: op.prepare_gathered(x_dev[f], y_all[f], f) for f in FEATS}
        # The five calls are independent: they alternate between two streams, so that the first
        # rows of one call reach the links while the last blocks of the previous one drain.
        lanes = [torch.cuda.Stream(), torch.cuda.Stream()]

        def gather_step():
            cur = torch.cuda.current_stream()
            for s in lanes:
                s.wait_stream(cur)
            for i, f in enumerate(order):
                with torch.cuda.stream(lanes[i % 2]):
                    gathered[f]()
            for s in lanes:
                cur.wait_stream(s)
            op.wait()

        gather_ms = timed(gather_step, max(3, min(args.steps, 20)))
        recv = sum(4 * f * (g.m - m_loc) for f in FEATS)  # bytes this GPU receives per step
        recv_max = over_ranks([float(recv)], MAX)[0]
        nvlink = {"bound": "nvlink", "achieved": recv_max / (gather_ms * 1e-3) / 1e9, "peak": NVLINK_GBS,
                  "unit": "GB/s", "frac": recv_max / (gather_ms * 1e-3) / 1e9 / NVLINK_GBS,
                  "bytes_received_per_gpu_per_step": recv_max,
                  "transport": (sharded.peer_transport_note()
                                if isinstance(y_all[FEATS[0]], sharded.PeerOutput) else "NCCL all-gather"),
                  "note": "every GPU must receive the other shards' rows of Y: these bytes over the "
                          "measured 770 GB/s per direction are the floor of this step"}
    value_ms = gather_ms if world > 1 else kernel_ms
    value = total_flops / (value_ms * 1e-3) / 1e9

    # ---- end to end: X from pinned host memory, Y back to pinned host memory.
    # One GPU: the whole X in, the whole Y out.  N GPUs: every rank owns an equal block of the rows
    # of X in ITS pinned host memory and the rows of Y of its shard; per step it copies its block in
    # over its own PCIe link, the blocks are all-gathered over NVLink (NCCL), the shard kernels run,
    # and the shard's output rows go back to the rank's pinned host memory.  The bytes per step are
    # the same as with one GPU; they are spread over N links.
    xr0, xr1 = min(g.n, rank * blk), min(g.n, (rank + 1) * blk)
    x_host_loc = {}
    if world > 1:
        for f in FEATS:
            buf = torch.zeros(blk * f, dtype=torch.float32).pin_memory()
            buf[:(xr1 - xr0) * f].copy_(x_host[f].reshape(-1)[xr0 * f:xr1 * f])
            x_host_loc[f] = buf
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

    def my_block(f):
        return x_dev[f][rank * blk * f:(rank + 1) * blk * f]

    def copy_in(f):
        if world == 1:
            x_dev[f][:g.n * f].copy_(x_host[f].reshape(-1), non_blocking=True)
        else:
            my_block(f).copy_(x_host_loc[f], non_blocking=True)

    def e2e_step():
        for f in FEATS:
            s_in.wait_event(ev_done[f])       # previous step's kernels have read x_dev[f]
            with torch.cuda.stream(s_in):
                copy_in(f)
                if world > 1:
                    sharded.replicate_rows(my_block(f), x_dev[f])
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

    e_steps = max(3, min(args.steps, 10))
    e2e_ms = timed(e2e_step, e_steps)
    h2d = sum(4 * g.n * f for f in FEATS)
    d2h = sum(4 * g.m * f for f in FEATS)

    # the same step phase by phase, one after the other on one stream (no overlap), so that the sum
    # can be read against the overlapped figure: where does an end-to-end step spend its time
    phases = {"h2d_ms": timed(lambda: [copy_in(f) for f in FEATS], 3, warm=1)}
    if world > 1:
        phases["x_allgather_ms"] = timed(lambda: [sharded.replicate_rows(my_block(f), x_dev[f]) for f in FEATS], 3, warm=1)
    phases["kernels_ms"] = timed(step, 3, warm=1)
    phases["d2h_ms"] = timed(lambda: [y_host[f].copy_(y_dev[f], non_blocking=True) for f in FEATS], 3, warm=1)
    phases["h2d_gbs_per_gpu"] = (h2d / world) / (phases["h2d_ms"] * 1e-3) / 1e9
    phases["d2h_gbs_per_gpu"] = sum(4 * m_loc * f for f in FEATS) / (phases["d2h_ms"] * 1e-3) / 1e9

    # ---- the other operators sharded the same way (collective: every rank runs them)
    ops_sharded = None
    if world > 1 and args.ops:
        try:
            from sparsetir_b200 import opbench
            ops_sharded = opbench.run_sharded(device, peaks, rank, world, log)
        except Exception as e:  # the headline line must still be printed
            ops_sharded = {"error": repr(e)}

    # ---- every rank checks ITS rows of the timed result against the CPU oracle (one F), and with
    # N > 1 the gathered copy of everybody's rows too; the verdicts are and-reduced
    from oracle import oracle as orc
    orc.use_all_cores()
    f_chk = 64 if 64 in FEATS else FEATS[0]
    want = np.zeros((g.m, f_chk), np.float32)
    orc.csrmm(g.data, x_host[f_chk].numpy(), want, g.indptr, g.indices, g.m, g.n, f_chk, omp=True)
    ok = True
    try:
        got = y_host[f_chk].numpy().reshape(m_loc, f_chk)
        np.testing.assert_allclose(got, want[shard.row0:shard.row1], rtol=1e-4, atol=1e-5)
        if world > 1:
            np.testing.assert_allclose(sharded.local_tensor(y_all[f_chk]).cpu().numpy().reshape(g.m, f_chk), want,
                                       rtol=1e-4, atol=1e-5)
    except AssertionError as e:
        ok = False
        log(f"bench.py: rank {rank}: result differs from the oracle: {str(e)[:400]}")
    all_ok = over_ranks([1.0 if ok else 0.0], MIN)[0] == 1.0
    if rank != 0:
        return
    assert all_ok, "a rank's result differs from the CPU oracle"

    # ---- roofline of the dominant launch (F = 512): the rows of X this shard references, once
    f_dom = FEATS[-1]
    lanes, lane_w = ctypes.c_int(0), ctypes.c_int(0)
    lib.sparsetir_hyb_spmm_tile(g.n, f_dom, ctypes.byref(lanes), ctypes.byref(lane_w))
    kernel = f"hyb_spmm_lean_kernel<{lanes.value},{lane_w.value}>"
    x_rows = g.n if world == 1 else op.referenced_cols
    alg_bytes = spmm_bytes(m_loc, x_rows, nnz_loc, f_dom)
    achieved = alg_bytes / (per_f_ms[f_dom] * 1e-3) / 1e9
    traffic, traffic_source = profiled_traffic(kernel, f_dom, g.nnz) if world == 1 else (None, None)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "traffic_source": traffic_source,
                "peak_source": peaks["source"], "kernel": f"{kernel}, F={f_dom} call (one launch)",
                "algorithmic_bytes": alg_bytes, "launch_ms": per_f_ms[f_dom],
                "x_rows_counted": x_rows,
                "x_rows_note": ("all rows of X, the formula of the workload; this graph references "
                                f"{op.referenced_cols} of {g.n}" if world == 1 else
                                "the rows of X this shard's column indices name (rank 0)")}
    per_f = {}
    for f, lo in zip(FEATS, per_f_min):
        byts = spmm_bytes(m_loc, x_rows, nnz_loc, f)
        per_f[str(f)] = {"ms": per_f_ms[f], "ms_min_over_ranks": lo,
                         "gflops": 2.0 * g.nnz * f / (per_f_ms[f] * 1e-3) / 1e9,
                         "alg_gbs": byts / (per_f_ms[f] * 1e-3) / 1e9,
                         "hbm_frac": byts / (per_f_ms[f] * 1e-3) / 1e9 / peaks["hbm_gbs"]}

    # ---- CPU baseline on the host cores (bounded sample), OpenMP and serial: one-GPU runs only
    # (with N ranks on the box the other processes' threads would share the cores it is timed on)
    cpu = cpu_legs(g, {f: x_host[f].numpy() for f in FEATS}, total_flops) if world == 1 else None

    # ---- the same step with 2 and 4 column partitions (every contribution added atomically into
    # a C that the call clears first), one GPU only
    parts_sweep = None
    if world == 1 and args.ops:
        parts_sweep = {}
        for p in (2, 4):
            try:
                op_p = sharded.ShardedHybSpmm(g.indptr, g.indices, g.data, g.n, BUCKETS, parts=p, device=device)
                calls_p = {f: op_p.prepare(x_dev[f], y_dev[f], f) for f in FEATS}
                ms_p = timed(lambda: [calls_p[f]() for f in FEATS], max(3, min(args.steps, 20)))
                parts_sweep[str(p)] = {"ms_per_step": ms_p, "gflops": total_flops / (ms_p * 1e-3) / 1e9,
                                       "launch": "eager", "ell_slots": sum(int(c[2].numel()) for c in op_p.buckets)}
                del op_p, calls_p
            except Exception as e:
                parts_sweep[str(p)] = {"error": repr(e)}

    line = {
        "metric": "hyb_spmm_gflops", "value": value, "unit": "GFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": value_ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": common_config(g, parts),
        "run": {"value_is": ("shard kernels + all-gather of Y on every rank (eager, two streams)" if world > 1
                             else f"the five kernels of a step, {kernel_mode}"),
                "ell_slots_rank0": slots, "sharding": "nnz-balanced contiguous row shards, one per GPU",
                "host_setup_ms_rank0": setup_ms, "rows_rank0": m_loc, "nnz_rank0": nnz_loc},
        "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e9, "unit": "GFLOP/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "phases_unoverlapped": phases,
                "includes": "H2D of X, kernels, D2H of Y" + (
                    "; every rank copies its equal block of the rows of X from its own pinned host "
                    "memory, one NCCL all-gather per feature size, shard kernels, D2H of the shard's "
                    "output rows to the rank's pinned host memory" if world > 1 else "")},
        "gpu_launches": len(FEATS) * args.steps,
        "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks, "per_feat": per_f,
        "kernel_only": {"ms_per_step": kernel_ms, "gflops": total_flops / (kernel_ms * 1e-3) / 1e9,
                        "launch": kernel_mode, "eager_ms_per_step": eager_ms,
                        "alg_gbs": sum(spmm_bytes(m_loc, x_rows, nnz_loc, f) for f in FEATS) / (kernel_ms * 1e-3) / 1e9},
        "verified": "every rank's rows (and the gathered result) against the CPU oracle at F=%d" % f_chk,
    }
    if nvlink is not None:
        line["nvlink"] = nvlink
    if parts_sweep is not None:
        line["col_parts_sweep"] = parts_sweep
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
