"""Independent second opinions used to pin the oracle and to build the golden fixtures.

Nothing here shares code with ``oracle/`` or with the library: the format derivations go
through scipy sub-matrix slicing (the approach of the reference's own test,
tests/python/sparsetir/test_format_conversion_routine.py:28-101 and :130-143), the operator
results are fp64 scipy / numpy products.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import scipy.sparse as sp


def scipy_column_part_hyb(indptr, indices, m: int, n: int, column_part: int,
                          bucket_sizes: Sequence[int]) -> Tuple[List[np.ndarray], List[np.ndarray]]:
    """Row ids and column-id matrices per (partition, bucket), flattened partition-major,
    derived from per-partition degree histograms of column slices of a scipy CSR matrix.

    Bucket b of a partition holds the rows whose degree d inside the partition satisfies
    width[b-1] < d <= width[b]; the last bucket holds every row with d > width[-2], cut into
    pieces of width[-1] entries that repeat the row id.  Unused slots hold column 0.
    """
    bucket_sizes = list(bucket_sizes)
    mat = sp.csr_matrix((np.ones(len(indices), dtype=np.int8), indices, indptr), shape=(m, n))
    mat.sort_indices()
    part = (n + column_part - 1) // column_part
    ell_rows: List[np.ndarray] = []
    ell_cols: List[np.ndarray] = []
    for p in range(column_part):
        sub = mat[:, p * part:(p + 1) * part].tocsr()
        sub.sort_indices()
        deg = np.diff(sub.indptr)
        lower = 0
        for b, width in enumerate(bucket_sizes):
            last = b == len(bucket_sizes) - 1
            sel = np.nonzero((deg > lower) if last else ((deg > lower) & (deg <= width)))[0]
            rows_out, cols_out = [], []
            for r in sel:
                cols = sub.indices[sub.indptr[r]:sub.indptr[r + 1]] + p * part
                for s in range(0, len(cols), width):
                    piece = np.zeros(width, dtype=np.int32)
                    chunk = cols[s:s + width]
                    piece[:len(chunk)] = chunk
                    rows_out.append(r)
                    cols_out.append(piece)
            ell_rows.append(np.asarray(rows_out, dtype=np.int32))
            ell_cols.append(np.asarray(cols_out, dtype=np.int32).reshape(len(rows_out), width))
            lower = width
    return ell_rows, ell_cols


def condense_unique(indptr, indices, t: int) -> Tuple[np.ndarray, np.ndarray]:
    """Distinct sorted columns of every tile of t rows (the g = 1 view of condensing)."""
    m = len(indptr) - 1
    out_ptr, out_idx = [0], []
    for r0 in range(0, m, t):
        r1 = min(m, r0 + t)
        u = np.unique(indices[indptr[r0]:indptr[r1]])
        out_idx.append(u)
        out_ptr.append(out_ptr[-1] + len(u))
    cat = np.concatenate(out_idx) if out_idx else np.zeros(0, np.int32)
    return np.asarray(out_ptr), cat


def edge_to_row(indptr, nnz: int) -> np.ndarray:
    return (np.searchsorted(np.asarray(indptr), np.arange(nnz), side="right") - 1).astype(np.int32)


def spmm_f64(indptr, indices, data, x, m: int, n: int) -> np.ndarray:
    a = sp.csr_matrix((np.asarray(data, np.float64), indices, indptr), shape=(m, n))
    return a @ np.asarray(x, np.float64)


def sddmm_f64(indptr, indices, a, b, scale=None) -> np.ndarray:
    rows = np.repeat(np.arange(len(indptr) - 1), np.diff(indptr))
    out = np.einsum("ek,ek->e", np.asarray(a, np.float64)[rows], np.asarray(b, np.float64)[indices])
    return out if scale is None else out * np.asarray(scale, np.float64)


def bsrmm_f64(indptr, indices, blocks, b, nb: int, mb: int, blk: int) -> np.ndarray:
    a = sp.bsr_matrix((np.asarray(blocks, np.float64), indices, indptr),
                      shape=(nb * blk, mb * blk))
    return a @ np.asarray(b, np.float64)


def rgms_f64(data, w, x, indptr_i, indices_i, indptr_j, indices_j, m: int) -> np.ndarray:
    """Y = sum_r A_r X W_r^T with W[r, fo, fi]."""
    x = np.asarray(x, np.float64)
    w = np.asarray(w, np.float64)
    feat = x.shape[1]
    y = np.zeros((m, feat), np.float64)
    for r in range(len(indptr_i) - 1):
        i0, i1 = indptr_i[r], indptr_i[r + 1]
        if i1 == i0:
            continue
        ptr = np.asarray(indptr_j[i0:i1 + 1], np.int64)
        lo, hi = ptr[0], ptr[-1]
        a = sp.csr_matrix((np.asarray(data[lo:hi], np.float64), indices_j[lo:hi], ptr - lo),
                          shape=(i1 - i0, x.shape[0]))
        np.add.at(y, np.asarray(indices_i[i0:i1]), (a @ x) @ w[r].T)
    return y


def hyb_spmm_from_buckets(buckets, x, m: int) -> np.ndarray:
    """fp64 evaluation of the decomposed form: sum over buckets of W[r,s] * X[cols[r,s]]."""
    x = np.asarray(x, np.float64)
    y = np.zeros((m, x.shape[1]), np.float64)
    for w, rows, cols in buckets:
        if len(rows) == 0:
            continue
        contrib = np.einsum("rs,rsf->rf", np.asarray(w, np.float64), x[cols])
        np.add.at(y, rows, contrib)
    return y


def ellmm_f64(a, b, indices, nb: int, col: int, blk: int, feat: int) -> np.ndarray:
    """Block-ELL SpMM in fp64: c[i,bi,f] = sum_j sum_bj a[i,j,bi,bj] * b[indices[i,j],bj,f]."""
    a = np.asarray(a, np.float64).reshape(nb, col, blk, blk)
    b3 = np.asarray(b, np.float64).reshape(-1, blk, feat)
    if col == 0:
        return np.zeros((nb * blk, feat))
    return np.einsum("ijxy,ijyf->ixf", a, b3[np.asarray(indices).reshape(nb, col)]).reshape(nb * blk, feat)


def fusedmm_f64(q, k, v, indptr, indices) -> np.ndarray:
    """Sparse attention in fp64 with the reference's softmax (numerator not shifted by the row
    maximum: exp(s) / sum exp(s - max))."""
    q, k, v = (np.asarray(t, np.float64) for t in (q, k, v))
    m = len(indptr) - 1
    rows = np.repeat(np.arange(m), np.diff(indptr))
    s = np.einsum("ef,ef->e", q[rows], k[indices])
    out = np.zeros((m, v.shape[1]))
    if len(s) == 0:
        return out
    mx = np.full(m, -np.inf)
    np.maximum.at(mx, rows, s)
    den = np.zeros(m)
    np.add.at(den, rows, np.exp(s - mx[rows]))
    np.add.at(out, rows, (np.exp(s) / den[rows])[:, None] * v[indices])
    return out


def row_sums_f64(vals, indptr) -> np.ndarray:
    out = np.zeros(len(indptr) - 1)
    np.add.at(out, np.repeat(np.arange(len(indptr) - 1), np.diff(indptr)), np.asarray(vals, np.float64))
    return out
