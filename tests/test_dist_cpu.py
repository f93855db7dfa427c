"""Host-side logic of the multi-GPU layer, run as two gloo ranks on the CPU: nnz-balanced row
shards, per-shard format decomposition, broadcast of the dense operand, all-gather of unequal
output blocks.  The per-shard arithmetic is done by the CPU oracle here (the CUDA kernels need a
GPU); what is under test is that the sharded pipeline reproduces the single-process result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as orc
from sparsetir_b200 import datagen as dg
from sparsetir_b200 import dist as sdist
from sparsetir_b200 import format as fmt


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = dg.csr_powerlaw(n=3000, max_deg=2000, seed=5)
        feat = 24
        buckets = [1, 2, 4, 8, 16]
        # dense operand exists on rank 0 only and is broadcast
        x = torch.from_numpy(dg.dense_operand(6, g.n, feat)) if rank == 0 else torch.zeros(g.n, feat)
        sdist.broadcast_dense(x, src=0)
        shard = sdist.shard_csr(g.indptr, g.indices, g.data, g.n, world, rank)
        assert shard.cuts[0] == 0 and shard.cuts[-1] == g.m
        # hyb SpMM of the shard (decomposition by the library's host C++, arithmetic by the oracle)
        rows, cols, mask, vals, _ = fmt.column_part_hyb(shard.num_rows, g.n, shard.indptr, shard.indices,
                                                       2, buckets, data=shard.data)
        y_loc = np.zeros((shard.num_rows, feat), np.float32)
        for p in range(2):
            for b in range(len(buckets)):
                orc.ell_spmm(vals[p][b], rows[p][b], cols[p][b], x.numpy(), y_loc, feat)
        y = sdist.all_gather_rows(torch.from_numpy(y_loc).reshape(-1), shard.rows_per_rank(), feat)
        # SDDMM of the shard: edge-indexed output blocks of unequal length
        a = dg.dense_operand(7, g.m, feat)
        e_loc = orc.sddmm(a[shard.row0:shard.row1], x.numpy(), shard.indptr, shard.indices,
                          shard.num_rows, g.n, feat)
        e = sdist.all_gather_blocks(torch.from_numpy(e_loc), sdist.shard_edges(shard, g.indptr))
        if rank == 0:
            np.save(os.path.join(out_dir, "y.npy"), y.numpy())
            np.save(os.path.join(out_dir, "e.npy"), e.numpy())
        # a block of the wrong length must be refused, not silently mis-placed
        with pytest.raises(ValueError):
            sdist.all_gather_blocks(torch.zeros(3), [5, 7])
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_two_rank_sharded_pipeline_matches_single_process(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g = dg.csr_powerlaw(n=3000, max_deg=2000, seed=5)
    feat = 24
    x = dg.dense_operand(6, g.n, feat)
    want = np.zeros((g.m, feat), np.float32)
    orc.csrmm(g.data, x, want, g.indptr, g.indices, g.m, g.n, feat)
    got = np.load(os.path.join(tmp_path, "y.npy")).reshape(g.m, feat)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)
    a = dg.dense_operand(7, g.m, feat)
    want_e = orc.sddmm(a, x, g.indptr, g.indices, g.m, g.n, feat)
    assert np.array_equal(np.load(os.path.join(tmp_path, "e.npy")), want_e)


def test_shards_cover_the_matrix_and_balance():
    g = dg.csr_powerlaw(n=20000, seed=9)
    for world in (1, 2, 4, 8):
        shards = [sdist.shard_csr(g.indptr, g.indices, g.data, g.n, world, r) for r in range(world)]
        assert sum(s.num_rows for s in shards) == g.m and sum(s.nnz for s in shards) == g.nnz
        assert max(s.nnz for s in shards) <= g.nnz / world + np.diff(g.indptr).max()
        cat = np.concatenate([s.indices for s in shards])
        assert np.array_equal(cat, g.indices)
        for s in shards:
            assert s.indptr[0] == 0 and s.indptr[-1] == s.nnz
            assert np.array_equal(s.data, g.data[g.indptr[s.row0]:g.indptr[s.row1]])


def test_single_process_collectives_are_identity():
    t = torch.arange(12, dtype=torch.float32)
    assert torch.equal(sdist.all_gather_rows(t, [3], 4), t)
    assert sdist.broadcast_dense(t) is t


def test_bsr_block_row_shards_reproduce_the_whole_product():
    bs = dg.bsr_mask(size=512, blk=32, density=0.15, seed=3)
    feat = 64
    b = dg.dense_operand_normal(1, bs.nb * bs.blk, feat).astype(np.float16)
    want = orc.bsrmm_f16(bs.data, b, bs.indptr, bs.indices, bs.mb, bs.nb, bs.blk, feat).reshape(-1, feat)
    for world in (1, 2, 3, 8):
        shards = [sdist.shard_bsr(bs.indptr, bs.indices, bs.data, world, r) for r in range(world)]
        assert shards[0].row0 == 0 and shards[-1].row1 == bs.mb
        assert sum(len(s.indices) for s in shards) == bs.nnzb
        parts = [orc.bsrmm_f16(s.data, b, s.indptr, s.indices, s.row1 - s.row0, bs.nb, bs.blk, feat)
                 for s in shards if s.row1 > s.row0]
        got = np.concatenate(parts).reshape(-1, feat)
        assert np.array_equal(got, want)  # same blocks, same order inside a block row: bit-exact


def test_rgms_destination_row_shards_reproduce_the_whole_result():
    c = dg.csf_relational(n=3000, num_rels=7, num_edges=40000, seed=2)
    feat = 16
    x = dg.dense_operand(4, c.n, feat)
    w = dg.relation_weights(5, c.num_rels, feat)
    want = np.zeros((c.m, feat), np.float32)
    orc.rgms(c.data, w, x, want, c.indptr_i, c.indices_i, c.indptr_j, c.indices_j, c.m, c.n, c.num_rels, feat)
    for world in (1, 2, 4):
        got = np.zeros_like(want)
        edges = []
        for r in range(world):
            s = sdist.shard_rgms(c.indptr_i, c.indices_i, c.indptr_j, c.indices_j, c.data, c.m, world, r)
            assert s.indptr_i[-1] == len(s.indices_i) and s.indptr_j[-1] == len(s.indices_j)
            assert np.all(s.indices_i >= 0) and np.all(s.indices_i < max(1, s.num_rows))
            edges.append(len(s.indices_j))
            y = np.zeros((s.num_rows, feat), np.float32)
            if s.num_rows:
                orc.rgms(s.data, w, x, y, s.indptr_i, s.indices_i, s.indptr_j, s.indices_j, s.num_rows, c.n,
                         c.num_rels, feat)
            got[s.row0:s.row1] = y
        assert sum(edges) == c.nnz_j
        assert max(edges) <= c.nnz_j / world + 64  # balanced up to the heaviest destination row
        assert np.array_equal(got, want)  # relation and entry order kept: bit-exact
