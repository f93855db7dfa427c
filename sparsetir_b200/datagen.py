"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark
configurations.  They stand in for the public graphs the reference measures on
(examples/spmm/utils.py:23-52, examples/rgms/rgcn/utils.py:26-38), which need a network.

Every generator takes explicit sizes so the tests can run reduced cases; the defaults are
the full configurations.  One ``numpy.random.Generator(PCG64(seed))`` per call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def _indptr(deg: np.ndarray) -> np.ndarray:
    out = np.zeros(len(deg) + 1, dtype=np.int64)
    np.cumsum(deg, out=out[1:])
    assert out[-1] < 2**31, "int32 index space exceeded"
    return out.astype(np.int32)


def sorted_distinct_columns(rng: np.random.Generator, deg: np.ndarray, n: int) -> np.ndarray:
    """For each row r, ``deg[r]`` distinct column ids in [0, n), ascending.

    Draws deg[r] integers in [0, n-deg[r]] with replacement, sorts them inside the row and adds
    0,1,2,... — the classic multiset→set shift, which yields distinct sorted ids without a
    per-row loop.
    """
    deg = np.asarray(deg, dtype=np.int64)
    assert deg.max(initial=0) <= n
    nnz = int(deg.sum())
    rows = np.repeat(np.arange(len(deg), dtype=np.int64), deg)
    span = (n - deg + 1)[rows]
    draw = np.minimum((rng.random(nnz) * span).astype(np.int64), span - 1)
    key = rows * (n + 1) + draw
    key.sort(kind="stable")
    draw = key - rows * (n + 1)
    start = np.repeat(np.cumsum(deg) - deg, deg)
    rank = np.arange(nnz, dtype=np.int64) - start
    return (draw + rank).astype(np.int32)


@dataclass
class CSR:
    m: int
    n: int
    indptr: np.ndarray   # int32 [m+1]
    indices: np.ndarray  # int32 [nnz]
    data: np.ndarray     # float32 [nnz]

    @property
    def nnz(self) -> int:
        return int(self.indices.shape[0])


def dense_operand(seed: int, rows: int, feat: int, dtype=np.float32) -> np.ndarray:
    """rows x feat, U(-1, 1)."""
    return _rng(seed).uniform(-1.0, 1.0, size=(rows, feat)).astype(dtype)


# ------------------------------------------------------------------ config 1
def csr_poisson(m: int = 4096, n: int = 4096, mean_deg: float = 10.0, seed: int = 0) -> CSR:
    """Row degrees max(1, Poisson(mean_deg)), uniform distinct sorted columns, values U(-1,1)."""
    rng = _rng(seed)
    deg = np.minimum(np.maximum(rng.poisson(mean_deg, size=m), 1), n)
    indices = sorted_distinct_columns(rng, deg, n)
    data = rng.uniform(-1.0, 1.0, size=len(indices)).astype(np.float32)
    return CSR(m, n, _indptr(deg), indices, data)


# ------------------------------------------------------------------ config 2
def csr_powerlaw(n: int = 169_343, zipf_a: float = 2.1, max_deg: int = 13_000, seed: int = 0,
                 chunk_rows: int = 2048) -> CSR:
    """Square power-law graph: row degrees Zipf(zipf_a) clipped to [1, max_deg]; columns drawn by
    preferential attachment (probability proportional to current in-degree + 1), distinct inside a
    row, sorted; values 1/deg(row).

    Rows are processed in chunks of ``chunk_rows``; the attachment weights are those at the start
    of the chunk (a row-by-row update would be quadratic).  Duplicates inside a row are redrawn.
    """
    rng = _rng(seed)
    max_deg = min(max_deg, n)
    deg = np.clip(rng.zipf(zipf_a, size=n), 1, max_deg).astype(np.int64)
    indptr = _indptr(deg)
    nnz = int(indptr[-1])
    indices = np.empty(nnz, dtype=np.int32)
    filled = 0  # entries of `indices` that already take part in the attachment pool

    def draw(k: int) -> np.ndarray:
        idx = rng.integers(0, n + filled, size=k)
        out = idx.copy()
        big = idx >= n
        out[big] = indices[idx[big] - n]
        return out

    for r0 in range(0, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        d = deg[r0:r1]
        cnt = int(d.sum())
        rows = np.repeat(np.arange(r1 - r0, dtype=np.int64), d)
        cols = draw(cnt).astype(np.int64)
        for _ in range(64):
            order = np.argsort(rows * n + cols, kind="stable")
            rows, cols = rows[order], cols[order]
            dup = np.zeros(cnt, dtype=bool)
            dup[1:] = (rows[1:] == rows[:-1]) & (cols[1:] == cols[:-1])
            k = int(dup.sum())
            if k == 0:
                break
            cols[dup] = draw(k)
        else:  # pragma: no cover - only for pathological sizes
            for r in np.unique(rows[dup]):
                sel = rows == r
                cols[sel] = np.sort(rng.choice(n, size=int(sel.sum()), replace=False))
            order = np.argsort(rows * n + cols, kind="stable")
            rows, cols = rows[order], cols[order]
        indices[filled:filled + cnt] = cols
        filled += cnt
    data = np.repeat((1.0 / deg).astype(np.float32), deg)
    return CSR(n, n, indptr, indices, data)


# ------------------------------------------------------------------ config 3
def csr_lognormal(n: int = 232_965, mu: float = 5.5, sigma: float = 1.2, max_deg: int = 21_000,
                  seed: int = 0) -> CSR:
    """Square graph: row degrees round(LogNormal(mu, sigma)) clipped to [1, max_deg], uniform
    distinct sorted columns, values U(0,1)."""
    rng = _rng(seed)
    max_deg = min(max_deg, n)
    deg = np.clip(np.rint(rng.lognormal(mu, sigma, size=n)), 1, max_deg).astype(np.int64)
    indices = sorted_distinct_columns(rng, deg, n)
    data = rng.uniform(0.0, 1.0, size=len(indices)).astype(np.float32)
    return CSR(n, n, _indptr(deg), indices, data)


# ------------------------------------------------------------------ config 4
@dataclass
class BSR:
    mb: int              # block rows
    nb: int              # block columns
    blk: int
    indptr: np.ndarray   # int32 [mb+1]
    indices: np.ndarray  # int32 [nnzb]
    data: np.ndarray     # float16 [nnzb, blk, blk]

    @property
    def nnzb(self) -> int:
        return int(self.indices.shape[0])


def bsr_mask(size: int = 4096, blk: int = 32, density: float = 0.10, seed: int = 0) -> BSR:
    """Block pattern: uniform random at ``density`` plus the block diagonal; block values N(0,1)
    stored as fp16."""
    rng = _rng(seed)
    nb = size // blk
    pattern = rng.random((nb, nb)) < density
    pattern[np.arange(nb), np.arange(nb)] = True
    deg = pattern.sum(axis=1)
    indices = np.nonzero(pattern)[1].astype(np.int32)
    data = rng.standard_normal((len(indices), blk, blk)).astype(np.float16)
    return BSR(nb, nb, blk, _indptr(deg), indices, data)


def dense_operand_normal(seed: int, rows: int, feat: int, dtype=np.float16) -> np.ndarray:
    return _rng(seed).standard_normal((rows, feat)).astype(dtype)


# ------------------------------------------------------------------ config 5
@dataclass
class CSF:
    """Relation-major two-level compressed storage as the reference's rgcn_hetero_forward takes it
    (tests/python/sparsetir/sparse_tir_scripts.py:468-499)."""
    m: int
    n: int
    num_rels: int
    indptr_i: np.ndarray   # int32 [R+1]      rows (dst) that have edges, per relation
    indices_i: np.ndarray  # int32 [nnz_i]    dst row id
    indptr_j: np.ndarray   # int32 [nnz_i+1]
    indices_j: np.ndarray  # int32 [nnz_j]    src column id
    data: np.ndarray       # float32 [nnz_j]

    @property
    def nnz_i(self) -> int:
        return int(self.indices_i.shape[0])

    @property
    def nnz_j(self) -> int:
        return int(self.indices_j.shape[0])


def csf_relational(n: int = 100_000, num_rels: int = 46, num_edges: int = 1_500_000,
                   zipf_a: float = 1.5, seed: int = 0) -> CSF:
    """Edge counts per relation proportional to r^-zipf_a (r = 1..R) normalised to ``num_edges``;
    uniform random endpoints, duplicate (dst, src) pairs kept as separate stored entries; edges of
    a relation sorted by (dst, src); values 1/in-degree of the destination inside the relation."""
    rng = _rng(seed)
    wgt = np.arange(1, num_rels + 1, dtype=np.float64) ** (-zipf_a)
    counts = np.maximum(np.floor(wgt / wgt.sum() * num_edges).astype(np.int64), 1)
    counts[0] += num_edges - counts.sum()
    indptr_i = [0]
    indices_i, deg_all, indices_j, data = [], [], [], []
    for r in range(num_rels):
        e = int(counts[r])
        dst = rng.integers(0, n, size=e)
        src = rng.integers(0, n, size=e)
        order = np.lexsort((src, dst))
        dst, src = dst[order], src[order]
        rows, deg = np.unique(dst, return_counts=True)
        indices_i.append(rows.astype(np.int32))
        deg_all.append(deg)
        indices_j.append(src.astype(np.int32))
        data.append(np.repeat((1.0 / deg).astype(np.float32), deg))
        indptr_i.append(indptr_i[-1] + len(rows))
    deg_all = np.concatenate(deg_all)
    return CSF(n, n, num_rels, np.asarray(indptr_i, dtype=np.int32), np.concatenate(indices_i),
               _indptr(deg_all), np.concatenate(indices_j), np.concatenate(data))


def sparse_conv_pairs(n_in: int = 100_000, n_out: int = 100_000, num_offsets: int = 27,
                      fill: float = 0.5926, seed: int = 0) -> CSF:
    """The neighbour maps of a sparse convolution as a CSF tensor: relation = kernel offset; for
    every offset each output point has, with probability ``fill``, exactly ONE input point
    (uniformly drawn), so a (relation, destination) pair never repeats; values 1.  Outputs are
    ascending inside an offset.  Stand-in for the ``nbmaps`` / ``nbsizes`` of the layer files
    that examples/rgms/sparse_conv/sparse_conv.py:46-60 loads (not available here)."""
    rng = _rng(seed)
    indptr_i = [0]
    indices_i, indices_j = [], []
    for _ in range(num_offsets):
        outs = np.nonzero(rng.random(n_out) < fill)[0].astype(np.int32)
        indices_i.append(outs)
        indices_j.append(rng.integers(0, n_in, size=len(outs)).astype(np.int32))
        indptr_i.append(indptr_i[-1] + len(outs))
    rows = np.concatenate(indices_i)
    return CSF(n_out, n_in, num_offsets, np.asarray(indptr_i, dtype=np.int32), rows,
               np.arange(len(rows) + 1, dtype=np.int32), np.concatenate(indices_j),
               np.ones(len(rows), np.float32))


def relation_weights(seed: int, num_rels: int, feat: int) -> np.ndarray:
    """W[r, fo, fi] ~ N(0, 1/feat)."""
    return (_rng(seed).standard_normal((num_rels, feat, feat)) / np.sqrt(feat)).astype(np.float32)


def random_csr(m: int, n: int, nnz: int, seed: int = 0, values: Optional[str] = "uniform") -> CSR:
    """Uniform random pattern with ``nnz`` distinct positions (the stand-in for
    ``dgl.rand_graph`` in tests/python/sparsetir/test_format_conversion_routine.py:105)."""
    rng = _rng(seed)
    flat = np.sort(rng.choice(m * n, size=nnz, replace=False))
    rows, cols = flat // n, flat % n
    deg = np.bincount(rows, minlength=m)
    data = rng.uniform(-1, 1, size=nnz).astype(np.float32) if values else np.ones(nnz, np.float32)
    return CSR(m, n, _indptr(deg), cols.astype(np.int32), data)
