"""Per-operator measurements of the other benchmark configurations (CSR SpMM, SDDMM, BSR SpMM,
RGMS) on one GPU, reported beside the headline hyb-SpMM line by ``bench.py``.

Protocol: the reference's time_evaluator (one untimed call, ``number`` back-to-back calls between
two device events, src/runtime/profiling.cc:742-795), preceded by extra warm-up calls; for the
microsecond-scale operators an L2 flush (a write of a buffer larger than the L2) separates the
repeats and both the cold and the back-to-back (warm) figures are given.
"""
from __future__ import annotations

import math
import statistics
from typing import Callable, Dict

import numpy as np
import torch

from . import datagen as dg
from . import ops

L2_BYTES = 126 * 1024 * 1024
FP32_GFLOPS_NOMINAL = 148 * 128 * 2 * 1.965     # fp32 FMA rate at the maximum SM clock
L2_GATHER_GBS_MEASURED = 17800.0                 # random 128-byte row gathers from an L2-resident array


def _time(fn: Callable[[], None], number: int, repeat: int = 3, warmup: int = 3) -> float:
    """Mean milliseconds per call over ``number`` back-to-back calls, median of ``repeat``."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(repeat):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(number):
            fn()
        e1.record()
        e1.synchronize()
        out.append(e0.elapsed_time(e1) / number)
    return statistics.median(out)


def _time_graph(fn: Callable[[], None], number: int, repeat: int = 5) -> float:
    """Mean milliseconds per call with ``number`` calls captured in one CUDA graph and replayed:
    the device-side cost of back-to-back launches without per-call host work."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):  # the stream whose scratch the warm-up call set up
        for _ in range(number):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    out = []
    for _ in range(repeat):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        e1.synchronize()
        out.append(e0.elapsed_time(e1) / number)
    return statistics.median(out)


def _time_cold(fn: Callable[[], None], flush: torch.Tensor, repeat: int = 10) -> float:
    """Milliseconds of single calls, each after an L2 flush; median."""
    out = []
    for _ in range(repeat):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        out.append(e0.elapsed_time(e1))
    return statistics.median(out)


def _entry(ms: float, flops: float, byts: float, peaks: dict, **extra) -> dict:
    d = {"ms": ms, "gflops": flops / (ms * 1e-3) / 1e9, "alg_gbs": byts / (ms * 1e-3) / 1e9,
         "hbm_frac": byts / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    d.update(extra)
    return d


def bench_csrmm(device, peaks, flush) -> dict:
    c = dg.csr_poisson(seed=0)
    feat = 64
    dv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)  # noqa: E731
    x = dv(dg.dense_operand(0, c.n, feat).reshape(-1))
    y = torch.zeros(c.m * feat, device=device)
    args = (dv(c.data), x, y, dv(c.indptr), dv(c.indices))
    fn = ops.csrmm.prepare(*args)
    flops = 2.0 * c.nnz * feat
    byts = 4 * (c.m + 1) + 8 * c.nnz + 4 * c.n * feat + 4 * c.m * feat
    warm = _time(fn, number=1000)
    cold = _time_cold(fn, flush)
    graph = _time_graph(fn, number=200)
    out = {"workload": "csr_spmm_4096_poisson10_F64", "nnz": c.nnz,
           "warm": _entry(warm, flops, byts, peaks), "cold_l2": _entry(cold, flops, byts, peaks),
           "graph_replay": _entry(graph, flops, byts, peaks),
           "bound": "launch latency (ideal 0.4 us at the HBM peak)"}
    # the same kernel on the graph of the headline workload (no format decomposition): what the
    # hyb format buys can be read off against the per-F times of the main bench line
    g = dg.csr_powerlaw(seed=0)
    gd = (dv(g.data), dv(g.indptr), dv(g.indices))
    out["powerlaw_169343"] = {"nnz": g.nnz, "per_feat": {}}
    for f in (32, 128, 512):
        xg = dv(dg.dense_operand(100 + f, g.n, f).reshape(-1))
        yg = torch.zeros(g.m * f, device=device)
        fn = ops.csrmm.prepare(gd[0], xg, yg, gd[1], gd[2])
        ms = _time_cold(fn, flush, repeat=10)
        out["powerlaw_169343"]["per_feat"][str(f)] = _entry(
            ms, 2.0 * g.nnz * f, 4 * (g.m + 1) + 8 * g.nnz + 4 * g.n * f + 4 * g.m * f, peaks)
        del xg, yg
    return out


def sddmm_graph_on_device(device, n=232_965, mu=5.5, sigma=1.2, max_deg=21_000, seed=0):
    """Config-3 graph built on the GPU: same distributions as datagen.csr_lognormal (degrees
    from the same numpy stream; column draws from a torch generator, because 1.2e8 draws and a
    segmented sort take a minute on the host)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    deg_np = np.clip(np.rint(rng.lognormal(mu, sigma, size=n)), 1, min(max_deg, n)).astype(np.int64)
    deg = torch.from_numpy(deg_np).to(device)
    indptr = torch.zeros(n + 1, dtype=torch.int64, device=device)
    indptr[1:] = torch.cumsum(deg, 0)
    nnz = int(indptr[-1].item())
    assert nnz < 2**31
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    rows = torch.repeat_interleave(torch.arange(n, device=device), deg)
    span = (n - deg + 1)[rows]
    draw = (torch.rand(nnz, device=device, generator=gen, dtype=torch.float64) * span).long()
    draw = torch.minimum(draw, span - 1)
    del span
    key = rows * (n + 1) + draw
    del draw
    key, _ = torch.sort(key)
    draw = key - rows * (n + 1)
    del key
    rank = torch.arange(nnz, device=device) - indptr[:-1][rows]
    indices = (draw + rank).int()
    del draw, rank, rows
    scale = torch.rand(nnz, device=device, generator=gen)
    return indptr.int(), indices, scale, nnz


def bench_sddmm(device, peaks, feats=(32, 64, 128, 256)) -> dict:
    n = 232_965
    indptr, indices, scale, nnz = sddmm_graph_on_device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(1)
    out = {"workload": "sddmm_lognormal_232965", "nnz": nnz,
           "graph": "built on the GPU with a torch generator: the twin of datagen.csr_lognormal(seed=0) "
                    "(same degree sequence, other column draws)",
           "per_feat": {}}
    c = torch.empty(nnz, device=device)
    for f in feats:
        a = torch.rand(n * f, device=device, generator=gen) * 2 - 1
        b = torch.rand(n * f, device=device, generator=gen) * 2 - 1
        fn = ops.sddmm.prepare(a, b, c, indptr, indices, scale)
        ms = _time(fn, number=3, repeat=3, warmup=2)
        flops = 2.0 * nnz * f + nnz
        byts = 4 * (n + 1) + 12 * nnz + 8 * n * f
        ent = _entry(ms, flops, byts, peaks, gather_gbs=(4.0 * nnz * f) / (ms * 1e-3) / 1e9)
        # the three roofs side by side: HBM by the compulsory bytes, the fp32 FMA pipes (nominal
        # 148 SMs x 128 lanes x 2 x 1.965 GHz), and the L2-to-SM path that carries one B row per
        # position (17.8 TB/s is the rate this kernel reached at F = 32 with the path 77-79 % busy)
        ent["fma_frac"] = ent["gflops"] / FP32_GFLOPS_NOMINAL
        ent["l2_gather_frac"] = ent["gather_gbs"] / L2_GATHER_GBS_MEASURED
        ent["binding_roof"] = max((ent["hbm_frac"], "hbm"), (ent["fma_frac"], "fp32 fma"),
                                  (ent["l2_gather_frac"], "l2-to-sm gather"))[1]
        out["per_feat"][str(f)] = ent
        del a, b
    # spot check of the full-size result against a float64 recomputation of 4096 random edges
    f = feats[0]
    gen.manual_seed(1)
    a = torch.rand(n * f, device=device, generator=gen) * 2 - 1
    b = torch.rand(n * f, device=device, generator=gen) * 2 - 1
    ops.sddmm(a, b, c, indptr, indices, scale)
    e = torch.randint(0, nnz, (4096,), device=device)
    row = torch.searchsorted(indptr.long(), e, right=True) - 1
    want = (a.view(n, f)[row].double() * b.view(n, f)[indices[e].long()].double()).sum(1) * scale[e].double()
    err = (c[e].double() - want).abs().max().item()
    out["spot_check_max_abs_err"] = err
    assert err < 1e-4, err
    # the row-wise operators that follow SDDMM in attention-style pipelines, on the same graph:
    # row sums and the reference's sparse softmax of the per-position values (streaming, HBM-bound)
    del a, b
    rs = torch.empty(n, device=device)
    fn = ops.csr_reduce.prepare(scale, rs, indptr, indices)
    ms = _time(fn, number=5, repeat=3, warmup=2)
    byts = 4 * nnz + 4 * (n + 1) + 4 * n
    out["csr_reduce"] = _entry(ms, float(nnz), byts, peaks)
    fn = ops.sparse_softmax.prepare(scale, c, indptr, indices)
    ms = _time(fn, number=5, repeat=3, warmup=2)
    byts = 8 * nnz + 4 * (n + 1)
    out["sparse_softmax"] = _entry(ms, 4.0 * nnz, byts, peaks)
    # sparse attention in one pass (fusedmm) against the same three operators one after the other
    f = 64
    gen.manual_seed(2)
    qf = (torch.rand(n * f, device=device, generator=gen) * 2 - 1) * (2.0 / math.sqrt(f))
    kf = torch.rand(n * f, device=device, generator=gen) * 2 - 1
    vf = torch.rand(n * f, device=device, generator=gen) * 2 - 1
    of = torch.empty(n * f, device=device)
    fn = ops.fusedmm.prepare(qf, kf, vf, of, indptr, indices)
    ms = _time(fn, number=3, repeat=3, warmup=2)
    flops = 4.0 * nnz * f
    byts = 4 * (n + 1) + 4 * nnz + 16 * n * f
    out["fusedmm_F64"] = _entry(ms, flops, byts, peaks, gather_gbs=(8.0 * nnz * f) / (ms * 1e-3) / 1e9)
    prob = torch.empty(nnz, device=device)
    o2 = torch.empty(n * f, device=device)
    s1 = ops.sddmm.prepare(qf, kf, c, indptr, indices)
    s2 = ops.sparse_softmax.prepare(c, prob, indptr, indices)
    s3 = ops.csrmm.prepare(prob, vf, o2, indptr, indices)

    def three():
        s1(); s2(); s3()

    out["fusedmm_F64"]["ms_three_operators"] = _time(three, number=3, repeat=3, warmup=2)
    out["fusedmm_F64"]["max_abs_diff_vs_three_operators"] = (of - o2).abs().max().item()
    return out


def _max_over_ranks(ms: float, device) -> float:
    import torch.distributed as dist
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _all_ranks_ok(ok: bool, device) -> bool:
    import torch.distributed as dist
    t = torch.tensor([1.0 if ok else 0.0], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item() == 1.0)


def bench_sddmm_sharded(device, peaks, rank: int, world: int, feats=(32, 128)) -> dict:
    """Config 3 cut into nnz-balanced row blocks, one per rank (every rank builds the same seeded
    graph and keeps its block), each block in four row chunks whose all-gathers overlap the next
    chunk's kernels.  Per feature size: the shard kernels alone (max and min over ranks), the step
    that ends with the per-position outputs all-gathered on every rank, and the whole graph on
    rank 0 alone in the same run, so that the parallel efficiency is a ratio of two numbers of one
    run.  Every rank checks its own positions against the CPU oracle.  Collective."""
    import torch.distributed as dist

    from oracle import oracle as orc
    from . import sharded

    n = 232_965
    indptr, indices, scale, nnz = sddmm_graph_on_device(device)
    op = sharded.ShardedSddmm(indptr, indices, scale, n, chunks=4, device=device)
    c_out = sharded.peer_empty(nnz, torch.float32, device)
    c_full = sharded.local_tensor(c_out)
    gen = torch.Generator(device=device)
    gen.manual_seed(1)
    out = {"workload": "sddmm_lognormal_232965", "nnz": nnz,
           "graph": "built on the GPU with a torch generator: the twin of datagen.csr_lognormal(seed=0) "
                    "(same degree sequence, other column draws)",
           "transport": sharded.peer_transport_note("sddmm") if isinstance(c_out, sharded.PeerOutput) else "NCCL",
           "rows_per_rank": [int(op.cuts[k + 1] - op.cuts[k]) for k in range(world)],
           "nnz_per_rank": [sum(op.chunk_sizes[c][k] for c in range(op.chunks)) for k in range(world)],
           "chunks": op.chunks, "per_feat": {}}
    ok = True
    for f in feats:
        a = torch.rand(n * f, device=device, generator=gen) * 2 - 1
        b = torch.rand(n * f, device=device, generator=gen) * 2 - 1
        # kernels alone: the shard's calls writing this GPU's buffer only; with the gather: the
        # calls prepared on the peer-mapped output (which may store into the peers themselves)
        local_calls = op.prepare(a, b, sharded.local_tensor(c_out), f)
        calls = op.prepare(a, b, c_out, f)
        dist.barrier()
        mine = _time(lambda: op.run(local_calls), number=3, repeat=3, warmup=2)
        ms = _max_over_ranks(mine, device)
        ms_min = -_max_over_ranks(-mine, device)

        def with_gather():
            op.run(calls, c_out)
            op.wait()

        dist.barrier()
        ms_g = _max_over_ranks(_time(with_gather, number=3, repeat=3, warmup=2), device)
        # the whole graph on rank 0 alone (the other ranks wait at the barrier)
        single = 0.0
        if rank == 0:
            fn1 = ops.sddmm.prepare(a, b, torch.empty(nnz, device=device), indptr, indices, scale)
            single = _time(fn1, number=3, repeat=3, warmup=2)
            del fn1
        dist.barrier()
        single = _max_over_ranks(single, device)
        flops = 2.0 * nnz * f + nnz
        recv = 4.0 * (nnz - out["nnz_per_rank"][rank])
        out["per_feat"][str(f)] = {
            "ms": ms, "ms_min_over_ranks": ms_min, "gflops": flops / (ms * 1e-3) / 1e9,
            "gather_gbs": (4.0 * nnz * f) / (ms * 1e-3) / 1e9,
            "ms_with_allgather": ms_g, "gflops_with_allgather": flops / (ms_g * 1e-3) / 1e9,
            "allgather_recv_gbs_per_gpu": recv / (ms_g * 1e-3) / 1e9,
            "ms_one_gpu_same_run": single,
            "parallel_efficiency_kernels": single / (world * ms),
            "parallel_efficiency_with_allgather": single / (world * ms_g)}
        if f == feats[0]:
            # this rank's positions (taken from the gathered result on this GPU) against the oracle's
            # loop nest on the host, and a few thousand positions of the other ranks in float64
            with_gather()
            torch.cuda.synchronize()
            r0, r1 = op.row0, op.row1
            ip_host = indptr[r0:r1 + 1].cpu().numpy()
            p0, p1 = int(ip_host[0]), int(ip_host[-1])
            orc.use_all_cores()
            want = orc.sddmm(a.view(n, f)[r0:r1].cpu().numpy(), b.view(n, f).cpu().numpy(),
                             (ip_host - p0).astype(np.int32), indices[p0:p1].cpu().numpy(), r1 - r0, n, f,
                             scale=scale[p0:p1].cpu().numpy(), omp=True)
            got = c_full[p0:p1].cpu().numpy()
            ok = bool(np.allclose(got, want, rtol=1e-4, atol=1e-5))
            e = torch.randint(0, nnz, (4096,), device=device)
            row = torch.searchsorted(indptr.long(), e, right=True) - 1
            ref = (a.view(n, f)[row].double() * b.view(n, f)[indices[e].long()].double()).sum(1) * scale[e].double()
            err = (c_full[e].double() - ref).abs().max().item()
            ok = ok and err < 1e-4
            out["spot_check_max_abs_err"] = err
        del a, b, calls
    out["every_rank_matches_oracle"] = _all_ranks_ok(ok, device)
    assert out["every_rank_matches_oracle"], "a rank's SDDMM positions differ from the oracle"
    return out


def bench_bsrmm_sharded(device, peaks, rank: int, world: int) -> dict:
    """Config 4 cut into block rows balanced by stored blocks; every rank checks its block rows
    against the oracle.  A call of a few microseconds: the figures show the latency floor."""
    import torch.distributed as dist

    from oracle import oracle as orc
    from . import sharded

    bs = dg.bsr_mask(seed=0)
    feat = 512
    op = sharded.ShardedBsrmm(bs.indptr, bs.indices, bs.data, bs.nb, bs.blk, device=device)
    b_host = dg.dense_operand_normal(1, bs.nb * bs.blk, feat)
    b = torch.from_numpy(b_host.astype(np.float16).reshape(-1)).to(device)
    c_loc = torch.zeros(op.block_rows * bs.blk * feat, device=device)
    c_out = sharded.peer_empty(bs.mb * bs.blk * feat, torch.float32, device)
    c_all = sharded.local_tensor(c_out)
    call = op.prepare(b, c_loc, feat)
    run = (lambda: call()) if call is not None else (lambda: None)
    dist.barrier()
    ms = _max_over_ranks(_time(run, number=100), device)

    def with_gather():
        run()
        op.gather(c_loc, feat, c_out)
        op.wait()

    dist.barrier()
    ms_g = _max_over_ranks(_time(with_gather, number=20), device)
    torch.cuda.synchronize()
    s = op.shard
    ok = True
    if op.block_rows > 0:
        want = orc.bsrmm_f16(s.data, b_host, s.indptr, s.indices, op.block_rows, bs.nb, bs.blk, feat, omp=True)
        ok = bool(np.allclose(c_loc.cpu().numpy().reshape(want.shape), want, rtol=1e-2, atol=1e-2))
        lo = s.row0 * bs.blk * feat
        ok = ok and bool(torch.equal(c_all[lo:lo + c_loc.numel()], c_loc))
    flops = 2.0 * bs.nnzb * bs.blk * bs.blk * feat
    res = {"workload": "bsr_spmm_4096_blk32_10pct_F512_f16", "block_rows_per_rank": [r // bs.blk for r in op.rows_per_rank],
           "ms": ms, "gflops": flops / (ms * 1e-3) / 1e9, "ms_with_allgather": ms_g,
           "transport": sharded.peer_transport_note("bsrmm"),
           "every_rank_matches_oracle": _all_ranks_ok(ok, device)}
    assert res["every_rank_matches_oracle"], "a rank's BSR block rows differ from the oracle"
    return res


def bench_rgms_sharded(device, peaks, rank: int, world: int) -> dict:
    """Config 5 cut by destination rows balanced by edges (one writer per output row); every rank
    checks its rows against the oracle."""
    import torch.distributed as dist

    from oracle import oracle as orc
    from . import sharded

    cf = dg.csf_relational(seed=0)
    feat = 64
    op = sharded.ShardedRgms(cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j, cf.data, cf.m, cf.n, device=device)
    x_host = dg.dense_operand(1, cf.n, feat)
    w_host = dg.relation_weights(2, cf.num_rels, feat)
    x = torch.from_numpy(x_host.reshape(-1)).to(device)
    w = torch.from_numpy(w_host.reshape(-1)).to(device)
    s = op.shard
    y_loc = torch.zeros(s.num_rows * feat, device=device)
    y_out = sharded.peer_empty(cf.m * feat, torch.float32, device)
    y_all = sharded.local_tensor(y_out)
    call = op.prepare(w, x, y_loc)

    def run():
        y_loc.zero_()  # the operator accumulates: clearing Y is part of every call
        if call is not None:
            call()

    dist.barrier()
    ms = _max_over_ranks(_time(run, number=20), device)

    def with_gather():
        run()
        op.gather(y_loc, feat, y_out)
        op.wait()

    dist.barrier()
    ms_g = _max_over_ranks(_time(with_gather, number=10), device)
    torch.cuda.synchronize()
    ok = True
    if s.num_rows > 0:
        orc.use_all_cores()
        want = orc.rgms(s.data, w_host, x_host, np.zeros((s.num_rows, feat), np.float32), s.indptr_i, s.indices_i,
                        s.indptr_j, s.indices_j, s.num_rows, cf.n, cf.num_rels, feat, omp=True)
        # the oracle's sequential fp32 sums are themselves up to 1e-5 off the float64 result
        ok = bool(np.allclose(y_loc.cpu().numpy().reshape(want.shape), want, rtol=1e-4, atol=3e-5))
        ok = ok and bool(torch.equal(y_all[s.row0 * feat:s.row1 * feat], y_loc))
    flops_ref = 2.0 * cf.nnz_j * feat * feat + 2.0 * cf.nnz_j * feat
    res = {"workload": "rgms_100k_46rel_1.5M_F64", "rows_per_rank": op.rows_per_rank,
           "edges_rank0": int(len(s.indices_j)), "ms": ms, "gflops": flops_ref / (ms * 1e-3) / 1e9,
           "ms_with_allgather": ms_g, "transport": sharded.peer_transport_note("rgms"),
           "every_rank_matches_oracle": _all_ranks_ok(ok, device)}
    assert res["every_rank_matches_oracle"], "a rank's RGMS rows differ from the oracle"
    return res


def run_sharded(device, peaks, rank: int, world: int, log=print) -> Dict[str, dict]:
    """The other operators of the set on row shards, one per rank (collective)."""
    out = {}
    for name, fn in (("sddmm", lambda: bench_sddmm_sharded(device, peaks, rank, world)),
                     ("bsrmm", lambda: bench_bsrmm_sharded(device, peaks, rank, world)),
                     ("rgms", lambda: bench_rgms_sharded(device, peaks, rank, world))):
        try:
            out[name] = fn()
        except Exception as e:  # keep the other operators' numbers (every rank fails or none does)
            out[name] = {"error": repr(e)}
        if rank == 0:
            log(f"[opbench sharded] {name}: {out[name]}")
        torch.cuda.empty_cache()
    return out


def bench_bsrmm(device, peaks, flush) -> dict:
    bs = dg.bsr_mask(seed=0)
    feat = 512
    dv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)  # noqa: E731
    b = dv(dg.dense_operand_normal(1, bs.nb * bs.blk, feat).reshape(-1))
    c = torch.zeros(bs.mb * bs.blk * feat, device=device)
    args = (dv(bs.data.reshape(-1)), b, c, dv(bs.indptr), dv(bs.indices), bs.mb, bs.nb, bs.nnzb,
            bs.blk, feat)
    fn = ops.bsrmm.prepare(*args)
    flops = 2.0 * bs.nnzb * bs.blk * bs.blk * feat
    byts = (2 * bs.nnzb * bs.blk * bs.blk + 4 * bs.nnzb + 4 * (bs.mb + 1)
            + 2 * bs.nb * bs.blk * feat + 4 * bs.mb * bs.blk * feat)
    warm = _time(fn, number=200)
    cold = _time_cold(fn, flush)
    graph = _time_graph(fn, number=100)
    tc_peak = peaks["bf16_tflops"] * 1e3  # GFLOP/s; fp16 taken equal to bf16
    return {"workload": "bsr_spmm_4096_blk32_10pct_F512_f16", "nnzb": bs.nnzb,
            "graph_replay": _entry(graph, flops, byts, peaks, tensor_frac=flops / (graph * 1e-3) / 1e9 / tc_peak),
            "warm": _entry(warm, flops, byts, peaks, tensor_frac=flops / (warm * 1e-3) / 1e9 / tc_peak),
            "cold_l2": _entry(cold, flops, byts, peaks, tensor_frac=flops / (cold * 1e-3) / 1e9 / tc_peak),
            "bound": "HBM / launch latency (arithmetic intensity 114 flop/B is below the ridge)"}


def bench_rgms(device, peaks, flush) -> dict:
    cf = dg.csf_relational(seed=0)
    feat = 64
    dv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)  # noqa: E731
    x = dv(dg.dense_operand(1, cf.n, feat).reshape(-1))
    w = dv(dg.relation_weights(2, cf.num_rels, feat).reshape(-1))
    y = torch.zeros(cf.m * feat, device=device)
    args = (dv(cf.data), w, x, y, dv(cf.indptr_i), dv(cf.indices_i), dv(cf.indptr_j), dv(cf.indices_j))

    call = ops.rgms.prepare(*args)

    def fn():
        y.zero_()  # the operator accumulates: clearing Y is part of every call
        call()

    flops_ref = 2.0 * cf.nnz_j * feat * feat + 2.0 * cf.nnz_j * feat   # per-edge formulation
    flops_done = 2.0 * cf.nnz_j * feat + 2.0 * cf.nnz_i * feat * feat  # aggregate, then transform
    byts = 12 * cf.nnz_j + 4 * cf.num_rels * feat * feat + 8 * cf.n * feat
    warm = _time(fn, number=20)
    cold = _time_cold(fn, flush)
    return {"workload": "rgms_100k_46rel_1.5M_F64", "nnz_i": cf.nnz_i, "nnz_j": cf.nnz_j,
            "warm": _entry(warm, flops_ref, byts, peaks, gflops_executed=flops_done / (warm * 1e-3) / 1e9),
            "cold_l2": _entry(cold, flops_ref, byts, peaks, gflops_executed=flops_done / (cold * 1e-3) / 1e9),
            "note": "gflops counts the reference's per-edge formulation; the kernel aggregates first"}


def ell3d_values(cf, cols_bkt, masks) -> list:
    """The CSF values scattered into the ELL3D slots.  Inside a bucket the stored slots follow
    the CSF order of the rows that fall into the bucket (relation-major, rows ascending, entries
    in order), so the values of those rows, in order, fill the slots whose mask is 1."""
    deg = np.diff(cf.indptr_j)
    cb = np.asarray(cols_bkt)
    bucket_of_row = np.minimum(np.searchsorted(cb, deg, side="left"), len(cb) - 1)
    entry_bucket = np.repeat(bucket_of_row, deg)
    out = []
    for b, m in enumerate(masks):
        v = np.zeros(m.shape, np.float32)
        v[m == 1] = cf.data[entry_bucket == b]
        out.append(v)
    return out


def bench_rgms_ell3d(device, peaks, flush) -> dict:
    """Config 5 in the decomposed ELL3D form (buckets of 1..32 columns, 32 slots per group)."""
    from . import format as fmt
    cf = dg.csf_relational(seed=0)
    feat = 64
    cols_bkt = [1, 2, 4, 8, 16, 32]
    rows_bkt = [32 // c for c in cols_bkt]
    ip, rows, cols, mask = fmt.csf_to_ell3d(cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j,
                                            rows_bkt, cols_bkt)
    vals = ell3d_values(cf, cols_bkt, mask)
    dv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)  # noqa: E731
    buckets = []
    for b in range(len(cols_bkt)):
        mid = np.repeat(np.arange(cf.num_rels, dtype=np.int32), np.diff(ip[b]))
        buckets.append((dv(vals[b]), dv(rows[b]), dv(cols[b]), dv(mid)))
    x = dv(dg.dense_operand(1, cf.n, feat).reshape(-1))
    w = dv(dg.relation_weights(2, cf.num_rels, feat).reshape(-1))
    y = torch.zeros(cf.m * feat, device=device)
    call = ops.rgms_ell3d.prepare(*ops.rgms_ell3d_args(w, x, y, buckets, feat))

    def fn():
        y.zero_()
        call()

    # same answer as the CSF form on the same graph
    fn()
    y_csf = torch.zeros_like(y)
    ops.rgms(dv(cf.data), w, x, y_csf, dv(cf.indptr_i), dv(cf.indices_i), dv(cf.indptr_j), dv(cf.indices_j))
    err = (y - y_csf).abs().max().item()
    assert err < 1e-3, err
    slots = int(sum(m.size for m in mask))
    ell_rows = int(sum(r.size for r in rows))
    flops_ref = 2.0 * cf.nnz_j * feat * feat + 2.0 * cf.nnz_j * feat
    byts = 12 * cf.nnz_j + 4 * cf.num_rels * feat * feat + 8 * cf.n * feat
    warm = _time(fn, number=20)
    cold = _time_cold(fn, flush)
    return {"workload": "rgms_ell3d_100k_46rel_1.5M_F64", "buckets": cols_bkt, "ell_rows": ell_rows,
            "slots": slots, "padding": 1.0 - cf.nnz_j / slots, "max_abs_diff_vs_csf": err,
            "warm": _entry(warm, flops_ref, byts, peaks), "cold_l2": _entry(cold, flops_ref, byts, peaks)}


def bench_rgms_f16(device, peaks, flush) -> dict:
    """fp16 RGMS with rectangular weights on ELL3D buckets: (a) config 5's graph in buckets of
    1..32 columns, 64 -> 64; (b) the shape the sparse convolution driver builds — 27 relations
    (kernel offsets), every (input, output) pair its own ELL row (buckets = [1]), unit values —
    at 64 -> 128, 64 -> 256 and 128 -> 128 channels on 100,000 points with 1.6 M pairs."""
    from . import format as fmt
    dv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)  # noqa: E731
    out = {"workload": "rgms_ell3d_f16", "cases": {}}

    def one(name, cf, cols_bkt, group, feat_in, feat_out, number, out_dtype=torch.float32):
        rows_bkt = [max(1, group // c) for c in cols_bkt]
        ip, rows, cols, mask = fmt.csf_to_ell3d(cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j,
                                                rows_bkt, cols_bkt)
        buckets = []
        for b in range(len(cols_bkt)):
            mid = np.repeat(np.arange(cf.num_rels, dtype=np.int32), np.diff(ip[b]))
            buckets.append((dv(mask[b].astype(np.float16)), dv(rows[b]), dv(cols[b]), dv(mid)))
        x = dv(dg.dense_operand(1, cf.n, feat_in).astype(np.float16).reshape(-1))
        w = dv((np.random.default_rng(2).standard_normal((cf.num_rels, feat_in, feat_out)) /
                np.sqrt(feat_in)).astype(np.float16).reshape(-1))
        y = torch.zeros(cf.m * feat_out, device=device, dtype=out_dtype)
        call = ops.rgms_ell3d_f16.prepare(*ops.rgms_ell3d_f16_args(w, x, y, buckets, feat_in, feat_out))

        def fn():
            y.zero_()
            call()

        ell_rows = int(sum(r.size for r in rows))
        slots = int(sum(m.size for m in mask))
        flops = 2.0 * ell_rows * feat_in * feat_out + 2.0 * slots * feat_in   # executed: transform + gather
        byts = (6 * slots + 8 * ell_rows + 2 * cf.num_rels * feat_in * feat_out + 2 * cf.n * feat_in
                + y.element_size() * cf.m * feat_out)
        warm = _time(fn, number=number)
        cold = _time_cold(fn, flush)
        out["cases"][name] = {"ell_rows": ell_rows, "slots": slots, "feat_in": feat_in, "feat_out": feat_out,
                              "warm": _entry(warm, flops, byts, peaks), "cold_l2": _entry(cold, flops, byts, peaks)}

    cf = dg.csf_relational(seed=0)
    one("config5_graph_buckets_1_32_64x64", cf, [1, 2, 4, 8, 16, 32], 32, 64, 64, 20)
    conv = dg.sparse_conv_pairs(seed=1)  # 100,000 points, 27 offsets, about 1.6 M pairs, none repeated
    one("sparse_conv_27_offsets_64x128", conv, [1], 1, 64, 128, 20)
    one("sparse_conv_27_offsets_64x256", conv, [1], 1, 64, 256, 20)
    one("sparse_conv_27_offsets_128x128", conv, [1], 1, 128, 128, 20)
    one("sparse_conv_27_offsets_128x128_f16_out", conv, [1], 1, 128, 128, 20, torch.float16)
    return out


def bench_tcspmm(device, peaks, flush, feats=(128, 512), t: int = 16, g: int = 16) -> dict:
    """The power-law graph of the headline workload, condensed (ConDense, t x g = 16 x 16) and
    multiplied in fp16 with fp32 accumulation and fp16 output, as the reference example does."""
    from . import format as fmt
    gr = dg.csr_powerlaw(seed=0)
    gi, ti, mk = fmt.condense(gr.indptr, gr.indices, t, g)
    mb, nb, nnzb = len(gi) - 1, -(-gr.n // g), len(ti)
    dv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)  # noqa: E731
    a16, gi_d, ti_d = dv(mk.astype(np.float16).reshape(-1)), dv(gi), dv(ti.reshape(-1))
    out = {"workload": "tcspmm_powerlaw_169343_t16_g16_f16", "nnz": gr.nnz, "groups": nnzb,
           "condensed_density": float(mk.mean()), "per_feat": {}}
    for f in feats:
        xb = torch.zeros(nb * g * f, dtype=torch.float16, device=device)
        xb[:gr.n * f] = dv(dg.dense_operand(100 + f, gr.n, f).astype(np.float16).reshape(-1))
        c = torch.empty(mb * t * f, dtype=torch.float16, device=device)
        fn = ops.tcspmm.prepare(a16, xb, c, gi_d, ti_d, mb, nb, nnzb, f, t, g)
        warm = _time(fn, number=50)
        cold = _time_cold(fn, flush)
        flops = 2.0 * gr.nnz * f                                   # useful products only
        byts = 2 * nnzb * t * g + 4 * nnzb * g + 4 * (mb + 1) + 2 * gr.n * f + 2 * gr.m * f
        out["per_feat"][str(f)] = {"warm": _entry(warm, flops, byts, peaks), "cold_l2": _entry(cold, flops, byts, peaks),
                                   "gflops_executed": 2.0 * nnzb * t * g * f / (warm * 1e-3) / 1e9}
    return out


def run_all(device, peaks, log=print) -> Dict[str, dict]:
    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device)
    out = {}
    for name, fn in (("csrmm", lambda: bench_csrmm(device, peaks, flush)),
                     ("bsrmm", lambda: bench_bsrmm(device, peaks, flush)),
                     ("rgms", lambda: bench_rgms(device, peaks, flush)),
                     ("rgms_ell3d", lambda: bench_rgms_ell3d(device, peaks, flush)),
                     ("rgms_f16", lambda: bench_rgms_f16(device, peaks, flush)),
                     ("tcspmm", lambda: bench_tcspmm(device, peaks, flush)),
                     ("sddmm", lambda: bench_sddmm(device, peaks))):
        try:
            out[name] = fn()
        except Exception as e:  # keep the other operators' numbers
            out[name] = {"error": repr(e)}
        log(f"[opbench] {name}: {out[name]}")
        torch.cuda.empty_cache()
    return out
