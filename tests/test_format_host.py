"""The library's host-side format conversion must be bit-exact with the oracle (which restates
src/sparse/format.cc of the reference) and with the golden fixtures."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from sparsetir_b200 import datagen as dg
from sparsetir_b200 import format as fmt

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _assert_hyb_equal(got, want, parts, nb):
    for p in range(parts):
        for b in range(nb):
            for k in range(3):
                assert got[k][p][b].dtype == np.int32
                assert got[k][p][b].shape == want[k][p][b].shape, (p, b, k)
                assert np.array_equal(got[k][p][b], want[k][p][b]), (p, b, k)


def _scrambled(c: dg.CSR, seed: int) -> dg.CSR:
    """Same matrix with the entries of every row in random order (CSR order is what the
    reference routine follows, sorted or not)."""
    rng = np.random.default_rng(seed)
    idx = c.indices.copy()
    for i in range(c.m):
        s, e = c.indptr[i], c.indptr[i + 1]
        idx[s:e] = rng.permutation(idx[s:e])
    return dg.CSR(c.m, c.n, c.indptr, idx, c.data)


CASES = [
    ("powerlaw", lambda: dg.csr_powerlaw(n=3000, max_deg=2000, seed=1), 1, [1, 2, 4, 8, 16, 32, 64, 128, 256, 512]),
    ("powerlaw4", lambda: dg.csr_powerlaw(n=3000, max_deg=2000, seed=2), 4, [1, 2, 4, 8, 16, 32, 64, 128, 256, 512]),
    ("poisson", lambda: dg.csr_poisson(m=700, n=333, mean_deg=9, seed=3), 3, [1, 2, 4]),
    ("one_bucket", lambda: dg.csr_poisson(m=200, n=200, mean_deg=6, seed=4), 2, [3]),
    ("odd_buckets", lambda: dg.csr_poisson(m=300, n=1000, mean_deg=20, seed=5), 7, [1, 3, 5, 11]),
    ("rect_wide", lambda: dg.random_csr(50, 5000, 4000, seed=6), 4, [1, 2, 4, 8]),
    ("scrambled", lambda: _scrambled(dg.csr_poisson(m=400, n=400, mean_deg=12, seed=7), 7), 3, [2, 4, 8]),
    ("parts_gt_cols", lambda: dg.random_csr(20, 5, 40, seed=8), 8, [1, 2]),
]


@pytest.mark.parametrize("name,make,parts,buckets", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("threads", [1, 3])
def test_column_part_hyb_bit_exact(name, make, parts, buckets, threads):
    c = make()
    got = fmt.column_part_hyb(c.m, c.n, c.indptr, c.indices, parts, buckets, num_threads=threads)
    want = orc.column_part_hyb(c.m, c.n, c.indptr, c.indices, parts, buckets)
    _assert_hyb_equal(got, want, parts, len(buckets))


def test_column_part_hyb_many_threads_large():
    c = dg.csr_powerlaw(n=60000, seed=9)  # large enough for the multi-threaded path
    bk = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512]
    got = fmt.column_part_hyb(c.m, c.n, c.indptr, c.indices, 2, bk, num_threads=8)
    want = orc.column_part_hyb(c.m, c.n, c.indptr, c.indices, 2, bk)
    _assert_hyb_equal(got, want, 2, len(bk))


@pytest.mark.parametrize("tag", ["a", "b", "c", "d", "e", "f"])
def test_column_part_hyb_golden(tag):
    # fixtures written by the reference test's own scipy_column_part_hyb (see their `source` entry)
    g = np.load(os.path.join(GOLD, f"hyb_{tag}.npz"))
    parts, buckets = int(g["parts"]), [int(b) for b in g["buckets"]]
    rows, cols, mask = fmt.column_part_hyb(int(g["m"]), int(g["n"]), g["indptr"], g["indices"],
                                           parts, buckets)
    for p in range(parts):
        for b in range(len(buckets)):
            k = p * len(buckets) + b
            assert np.array_equal(rows[p][b], g[f"rows_{k}"])
            assert np.array_equal(cols[p][b], g[f"cols_{k}"])


def test_column_part_hyb_values_and_positions():
    c = dg.csr_powerlaw(n=2000, max_deg=900, seed=10)
    rows, cols, mask, vals, pos = fmt.column_part_hyb(c.m, c.n, c.indptr, c.indices, 2,
                                                     [1, 4, 16, 64], data=c.data)
    seen = np.zeros(c.nnz, np.int64)
    for p in range(2):
        for b in range(4):
            q, m, v = pos[p][b], mask[p][b], vals[p][b]
            assert np.array_equal(q >= 0, m == 1)
            assert np.array_equal(cols[p][b][m == 1], c.indices[q[m == 1]])
            assert np.array_equal(v[m == 1], c.data[q[m == 1]])
            assert np.all(v[m == 0] == 0) and np.all(cols[p][b][m == 0] == 0)
            np.add.at(seen, q[m == 1], 1)
    assert np.all(seen == 1)  # every stored entry lands in exactly one slot


def test_column_part_hyb_empty_inputs():
    ip = np.zeros(1, np.int32)
    ix = np.zeros(0, np.int32)
    rows, cols, mask = fmt.column_part_hyb(0, 10, ip, ix, 2, [1, 2])
    assert all(r.shape == (0,) for rp in rows for r in rp)
    assert cols[1][1].shape == (0, 2) and mask[0][0].shape == (0, 1)
    # rows without entries produce nothing
    ip = np.zeros(6, np.int32)
    rows, cols, mask = fmt.column_part_hyb(5, 10, ip, ix, 1, [4])
    assert rows[0][0].shape == (0,)


def test_column_part_hyb_rejects_bad_input():
    ip = np.array([0, 1], np.int32)
    with pytest.raises(TypeError, match="int32"):
        fmt.column_part_hyb(1, 4, ip.astype(np.int64), np.array([0], np.int32), 1, [1])
    with pytest.raises(ValueError, match="outside"):
        fmt.column_part_hyb(1, 4, ip, np.array([9], np.int32), 1, [1])
    with pytest.raises(ValueError, match="ascending"):
        fmt.column_part_hyb(1, 4, ip, np.array([0], np.int32), 1, [2, 1])
    with pytest.raises(ValueError, match="monotone"):
        fmt.column_part_hyb(2, 4, np.array([0, 2, 1], np.int32), np.array([0, 1], np.int32), 1, [1])


def test_shard_slices_concatenate_to_global():
    """Row-sharding invariant used by the multi-GPU layer: decomposing contiguous row blocks
    separately gives exactly the row-contiguous pieces of the global arrays (row ids re-based)."""
    c = dg.csr_powerlaw(n=5000, max_deg=3000, seed=12)
    bk, parts = [1, 2, 4, 8, 16, 32], 3
    glob = fmt.column_part_hyb(c.m, c.n, c.indptr, c.indices, parts, bk)
    cuts = fmt.row_partition(c.indptr, 4)
    assert cuts[0] == 0 and cuts[-1] == c.m and np.all(np.diff(cuts) >= 0)
    pieces = []
    for k in range(4):
        r0, r1 = int(cuts[k]), int(cuts[k + 1])
        ip = (c.indptr[r0:r1 + 1] - c.indptr[r0]).astype(np.int32)
        ix = c.indices[c.indptr[r0]:c.indptr[r1]]
        pieces.append((r0, fmt.column_part_hyb(r1 - r0, c.n, ip, ix, parts, bk)))
    for p in range(parts):
        for b in range(len(bk)):
            rows = np.concatenate([pc[0][p][b] + r0 for r0, pc in pieces])
            cols = np.concatenate([pc[1][p][b] for _, pc in pieces])
            mask = np.concatenate([pc[2][p][b] for _, pc in pieces])
            assert np.array_equal(rows, glob[0][p][b])
            assert np.array_equal(cols, glob[1][p][b])
            assert np.array_equal(mask, glob[2][p][b])


def test_row_partition_balances_nnz():
    c = dg.csr_powerlaw(n=20000, seed=13)
    for shards in (1, 2, 4, 8):
        cuts = fmt.row_partition(c.indptr, shards)
        per = np.diff(c.indptr[cuts])
        assert per.sum() == c.nnz
        assert per.max() <= c.nnz / shards + np.diff(c.indptr).max()
    # more shards than rows, and an empty matrix
    assert fmt.row_partition(np.array([0, 3], np.int32), 4).tolist() == [0, 0, 1, 1, 1]
    assert fmt.row_partition(np.zeros(5, np.int32), 2).tolist() == [0, 2, 4]


@pytest.mark.parametrize("t,g", [(4, 1), (8, 4), (16, 16), (3, 2)])
def test_condense_bit_exact(t, g):
    c = dg.random_csr(1000, 1000, 10000, seed=14)
    got = fmt.condense(c.indptr, c.indices, t, g)
    want = orc.condense(c.indptr, c.indices, t, g)
    for a, b in zip(got, want):
        assert a.shape == b.shape and np.array_equal(a, b)


def test_condense_golden_and_empty():
    g = np.load(os.path.join(GOLD, "condense.npz"))
    gi, ti, mk = fmt.condense(g["indptr"], g["indices"], int(g["t"]), 1)
    assert np.array_equal(gi, g["out_indptr"]) and np.array_equal(ti.reshape(-1), g["out_indices"])
    gi, ti, mk = fmt.condense(np.zeros(4, np.int32), np.zeros(0, np.int32), 2, 2)
    assert gi.tolist() == [0, 0, 0] and ti.shape == (0, 2) and mk.shape == (0, 2, 2)


@pytest.mark.parametrize("rows_b,cols_b", [([8, 4, 2, 1], [1, 2, 4, 8]), ([32, 16], [1, 2]), ([1], [4])])
def test_csf_to_ell3d_bit_exact(rows_b, cols_b):
    # the bucket lists of the first case are those of the reference's own (assertion-free) test,
    # tests/python/sparsetir/test_format_conversion_routine.py:218-225
    cf = dg.csf_relational(n=800, num_rels=9, num_edges=9000, seed=15)
    got = fmt.csf_to_ell3d(cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j, rows_b, cols_b)
    want = orc.csf_to_ell3d(cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j, rows_b, cols_b)
    for gl, wl in zip(got, want):
        for a, b in zip(gl, wl):
            assert a.shape == b.shape and np.array_equal(a, b)
    assert sum(int(m.sum()) for m in got[3]) == cf.nnz_j


def test_csf_to_ell3d_empty_relations_and_rows():
    # relation 1 has no rows; one row of relation 2 has no entries
    ip0 = np.array([0, 2, 2, 4], np.int32)
    ix0 = np.array([3, 9, 1, 2], np.int32)
    ip1 = np.array([0, 1, 4, 4, 6], np.int32)
    ix1 = np.array([5, 0, 1, 2, 7, 8], np.int32)
    got = fmt.csf_to_ell3d(ip0, ix0, ip1, ix1, [2, 2], [1, 2])
    want = orc.csf_to_ell3d(ip0, ix0, ip1, ix1, [2, 2], [1, 2])
    for gl, wl in zip(got, want):
        for a, b in zip(gl, wl):
            assert np.array_equal(a, b)
    with pytest.raises(ValueError, match="ascending"):
        fmt.csf_to_ell3d(ip0, ix0, ip1, ix1, [2, 2], [2, 1])


def test_sparse_conv_pairs_generator_has_no_repeated_pair():
    """The stand-in for sparse-convolution neighbour maps: inside an offset every output appears at
    most once, ascending, with exactly one input; values are 1."""
    from sparsetir_b200 import datagen as dg
    cf = dg.sparse_conv_pairs(n_in=500, n_out=700, num_offsets=9, fill=0.5, seed=3)
    assert cf.num_rels == 9 and cf.m == 700 and cf.n == 500
    assert cf.nnz_i == cf.nnz_j and np.array_equal(cf.indptr_j, np.arange(cf.nnz_i + 1))
    for r in range(cf.num_rels):
        outs = cf.indices_i[cf.indptr_i[r]:cf.indptr_i[r + 1]]
        assert np.all(np.diff(outs) > 0) and (len(outs) == 0 or (outs[0] >= 0 and outs[-1] < cf.m))
    assert cf.indices_j.min() >= 0 and cf.indices_j.max() < cf.n and np.all(cf.data == 1.0)
    assert 0.4 < cf.nnz_i / (9 * 700) < 0.6
