"""The sharded-operator layer (sparsetir_b200/sharded.py) as gloo ranks on the CPU: chunked
all-gathers land every rank's pieces in place, equal-block replication of the dense operand, and
a collective whose peer never joins surfaces as ShardError within the process group's time-out.
The per-shard arithmetic is the CPU oracle's here (the CUDA entry points need a GPU)."""
import datetime
import os
import socket
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as orc
from sparsetir_b200 import datagen as dg
from sparsetir_b200 import sharded

CPU = torch.device("cpu")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))


def _pipeline_worker(rank, world, port, out_dir):
    _init(rank, world, port)
    try:
        # ---- SDDMM: per-position outputs, rows cut into 3 chunks per rank
        g = dg.csr_lognormal(n=900, mu=2.5, sigma=1.0, max_deg=300, seed=4)
        feat = 16
        a = dg.dense_operand(1, g.m, feat)
        b = dg.dense_operand(2, g.n, feat)
        op = sharded.ShardedSddmm(g.indptr, g.indices, g.data, g.n, chunks=3, device=CPU)
        assert op.chunks == 3 and op.chunk_rows[0] == op.row0 and op.chunk_rows[-1] == op.row1
        out = torch.full((g.nnz,), -5.0)
        for c in range(op.chunks):
            r0, r1 = op.chunk_rows[c], op.chunk_rows[c + 1]
            off, size = op.chunk_offsets[c][rank], op.chunk_sizes[c][rank]
            assert off == g.indptr[r0] and size == g.indptr[r1] - g.indptr[r0]
            ip = op._ip[c].numpy()
            part = orc.sddmm(a[r0:r1], b, ip, op._ix[c].numpy(), r1 - r0, g.n, feat, scale=op._scale[c].numpy())
            out[off:off + size] = torch.from_numpy(part)
        op.run([None] * op.chunks, out)
        op.wait()
        # ---- hyb SpMM: output row blocks of unequal length
        gp = dg.csr_powerlaw(n=2500, max_deg=1500, seed=6)
        x = dg.dense_operand(3, gp.n, feat)
        hy = sharded.ShardedHybSpmm(gp.indptr, gp.indices, gp.data, gp.n, [1, 2, 4, 8], parts=2, device=CPU)
        y_loc = np.zeros((hy.shard.num_rows, feat), np.float32)
        for w, rows, cols in hy.buckets:
            orc.ell_spmm(w.numpy(), rows.numpy(), cols.numpy(), x, y_loc, feat)
        y = torch.zeros(gp.m * feat)
        hy.gather(torch.from_numpy(y_loc).reshape(-1), feat, y)
        hy.wait()
        # ---- replication of a dense operand from equal row blocks (padded at the end)
        blk = sharded.row_block(gp.n, world)
        xp = np.zeros((world * blk, feat), np.float32)
        xp[:gp.n] = x
        full = torch.zeros(world * blk * feat)
        sharded.replicate_rows(torch.from_numpy(xp[rank * blk:(rank + 1) * blk].reshape(-1).copy()), full)
        assert torch.equal(full.view(-1, feat)[:gp.n], torch.from_numpy(x))
        if rank == 0:
            np.save(os.path.join(out_dir, "sddmm.npy"), out.numpy())
            np.save(os.path.join(out_dir, "y.npy"), y.numpy())
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_two_rank_sharded_operators_match_single_process(tmp_path):
    mp.spawn(_pipeline_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    g = dg.csr_lognormal(n=900, mu=2.5, sigma=1.0, max_deg=300, seed=4)
    a, b = dg.dense_operand(1, g.m, 16), dg.dense_operand(2, g.n, 16)
    want = orc.sddmm(a, b, g.indptr, g.indices, g.m, g.n, 16, scale=g.data)
    assert np.array_equal(np.load(os.path.join(tmp_path, "sddmm.npy")), want)
    gp = dg.csr_powerlaw(n=2500, max_deg=1500, seed=6)
    x = dg.dense_operand(3, gp.n, 16)
    want_y = np.zeros((gp.m, 16), np.float32)
    orc.csrmm(gp.data, x, want_y, gp.indptr, gp.indices, gp.m, gp.n, 16)
    np.testing.assert_allclose(np.load(os.path.join(tmp_path, "y.npy")).reshape(gp.m, 16), want_y,
                               rtol=1e-4, atol=1e-5)


def _failure_worker(rank, world, port, out_dir):
    _init(rank, world, port, timeout_s=3)
    if rank == 1:
        # this rank never reaches the collective (it is busy elsewhere, then leaves between steps
        # with nothing of its own in flight): the others must not wait for it for ever
        time.sleep(12)
        os._exit(0)
    gp = dg.csr_powerlaw(n=600, max_deg=300, seed=8)
    hy = sharded.ShardedHybSpmm(gp.indptr, gp.indices, gp.data, gp.n, [1, 2, 4], device=CPU)
    y = torch.zeros(gp.m * 4)
    t0 = time.perf_counter()
    try:
        hy.gather(torch.zeros(hy.shard.num_rows * 4), 4, y)
        hy.wait()
        outcome = "no error"
    except sharded.ShardError as e:
        outcome = f"ShardError after {time.perf_counter() - t0:.1f} s: {e}"
    with open(os.path.join(out_dir, "outcome.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)  # the process group cannot be torn down collectively any more


def test_missing_peer_surfaces_as_shard_error(tmp_path):
    ctx = mp.spawn(_failure_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=False)
    deadline = time.time() + 90
    while not ctx.join(timeout=1) and time.time() < deadline:
        pass
    with open(os.path.join(tmp_path, "outcome.txt")) as f:
        outcome = f.read()
    assert outcome.startswith("ShardError after"), outcome
    assert float(outcome.split()[2]) < 60


def test_single_process_layer_is_identity():
    g = dg.csr_powerlaw(n=500, max_deg=200, seed=2)
    hy = sharded.ShardedHybSpmm(g.indptr, g.indices, g.data, g.n, [1, 2, 4], device=CPU)
    assert hy.world == 1 and hy.rows_per_rank == [g.m] and hy.referenced_cols == np.unique(g.indices).size
    y_loc = torch.arange(g.m * 2, dtype=torch.float32)
    out = torch.zeros(g.m * 2)
    hy.gather(y_loc, 2, out)
    hy.wait()
    assert torch.equal(out, y_loc)
    sd = sharded.ShardedSddmm(g.indptr, g.indices, None, g.n, chunks=4, device=CPU)
    assert sd.chunks == 1 and sd.chunk_sizes == [[g.nnz]] and sd.chunk_offsets == [[0]]
    assert sharded.row_block(10, 4) == 3


def test_transport_selection(monkeypatch):
    # per-operator defaults, the environment override, operators without a fused form
    from sparsetir_b200 import sharded
    monkeypatch.delenv("SPARSETIR_PEER_TRANSPORT", raising=False)
    assert sharded._peer_transport("hyb_spmm") == "fused"
    assert sharded._peer_transport("sddmm") == "copy"
    assert sharded._peer_transport("bsrmm") == "scatter" and sharded._peer_transport("rgms") == "scatter"
    monkeypatch.setenv("SPARSETIR_PEER_TRANSPORT", "fused")
    assert sharded._peer_transport("sddmm") == "fused"
    assert sharded._peer_transport("rgms") == "scatter"  # no kernel of RGMS finishes a row alone
    monkeypatch.setenv("SPARSETIR_PEER_TRANSPORT", "COPY")
    assert sharded._peer_transport("hyb_spmm") == "copy"
    monkeypatch.setenv("SPARSETIR_PEER_TRANSPORT", "carrier-pigeon")
    with pytest.raises(ValueError, match="SPARSETIR_PEER_TRANSPORT"):
        sharded._peer_transport("hyb_spmm")
    for op in ("hyb_spmm", "sddmm", "bsrmm", "rgms"):
        monkeypatch.setenv("SPARSETIR_PEER_TRANSPORT", "scatter")
        assert "stores it to every peer" in sharded.peer_transport_note(op)
