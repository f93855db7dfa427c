"""ctypes loader for the CPU oracle (``oracle/sparse_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.

All functions take and return numpy arrays; the ``*_omp`` entry points are the
same loops spread over host threads (used only for timing the CPU baseline).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import List, Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")
_lib = None

_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_u16p = ctypes.POINTER(ctypes.c_uint16)


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file."""
    src = os.path.join(_HERE, "sparse_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.oracle_hyb_create.restype = ctypes.c_void_p
        _lib.oracle_ell3d_create.restype = ctypes.c_void_p
    return _lib


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: Optional[np.ndarray], ty):
    if a is None:
        return ctypes.cast(None, ty)
    return a.ctypes.data_as(ty)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Makes the ``omp`` entry points use every core this process may run on, whatever
    OMP_NUM_THREADS says (launchers such as torchrun set it to 1); returns the thread count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(int(n))
    return num_threads()


# ----------------------------------------------------------------- formats
def column_part_hyb(num_rows: int, num_cols: int, indptr, indices, num_col_parts: int,
                    buckets: Sequence[int], with_pos: bool = False):
    """Returns (row_indices, col_indices, mask[, pos]) as [part][bucket] lists of int32 arrays,
    shaped like the reference's output (src/sparse/format.cc:146-149)."""
    L = lib()
    indptr, indices = _i32(indptr), _i32(indices)
    bk = _i32(list(buckets))
    h = ctypes.c_void_p(L.oracle_hyb_create(int(num_rows), int(num_cols), _p(indptr, _i32p),
                                            _p(indices, _i32p), int(num_col_parts),
                                            _p(bk, _i32p), len(bk)))
    rows_o, cols_o, mask_o, pos_o = [], [], [], []
    try:
        for p in range(num_col_parts):
            rp, cp, mp, pp = [], [], [], []
            for b, width in enumerate(bk):
                n = L.oracle_hyb_nrows(h, p, b)
                r = np.empty((n,), np.int32)
                c = np.empty((n, int(width)), np.int32)
                m = np.empty((n, int(width)), np.int32)
                q = np.empty((n, int(width)), np.int32)
                L.oracle_hyb_copy(h, p, b, _p(r, _i32p), _p(c, _i32p), _p(m, _i32p), _p(q, _i32p))
                rp.append(r); cp.append(c); mp.append(m); pp.append(q)
            rows_o.append(rp); cols_o.append(cp); mask_o.append(mp); pos_o.append(pp)
    finally:
        L.oracle_hyb_free(h)
    if with_pos:
        return rows_o, cols_o, mask_o, pos_o
    return rows_o, cols_o, mask_o


def condense(indptr, indices, t: int, g: int):
    """(group_indptr[ntiles+1], tile_indices[ngroups, g], mask[ngroups, t, g])."""
    L = lib()
    indptr, indices = _i32(indptr), _i32(indices)
    n = len(indptr) - 1
    ng = L.oracle_condense(n, _p(indptr, _i32p), _p(indices, _i32p), int(t), int(g),
                           _p(None, _i32p), _p(None, _i32p), _p(None, _i32p))
    gi = np.empty(((n + t - 1) // t + 1,), np.int32)
    ti = np.empty((ng, g), np.int32)
    mk = np.empty((ng, t, g), np.int32)
    L.oracle_condense(n, _p(indptr, _i32p), _p(indices, _i32p), int(t), int(g),
                      _p(gi, _i32p), _p(ti, _i32p), _p(mk, _i32p))
    return gi, ti, mk


def csf_to_ell3d(indptr0, indices0, indptr1, indices1, nnz_rows_bkt: Sequence[int],
                 nnz_cols_bkt: Sequence[int]):
    """(indptr, row_indices, col_indices, mask), each a per-bucket list."""
    L = lib()
    indptr0, indices0, indptr1, indices1 = map(_i32, (indptr0, indices0, indptr1, indices1))
    rb, cb = _i32(list(nnz_rows_bkt)), _i32(list(nnz_cols_bkt))
    R = len(indptr0) - 1
    h = ctypes.c_void_p(L.oracle_ell3d_create(R, _p(indptr0, _i32p), _p(indices0, _i32p),
                                              _p(indptr1, _i32p), _p(indices1, _i32p),
                                              _p(rb, _i32p), _p(cb, _i32p), len(rb)))
    out = ([], [], [], [])
    try:
        for b in range(len(rb)):
            ng = L.oracle_ell3d_ngroups(h, b, int(rb[b]))
            ip = np.empty((R + 1,), np.int32)
            r = np.empty((ng, int(rb[b])), np.int32)
            c = np.empty((ng, int(rb[b]), int(cb[b])), np.int32)
            m = np.empty((ng, int(rb[b]), int(cb[b])), np.int32)
            L.oracle_ell3d_copy(h, b, _p(ip, _i32p), _p(r, _i32p), _p(c, _i32p), _p(m, _i32p))
            for lst, arr in zip(out, (ip, r, c, m)):
                lst.append(arr)
    finally:
        L.oracle_ell3d_free(h)
    return out


# --------------------------------------------------------------------- ops
def csrmm(a, b, c, indptr, indices, m, n, feat, omp: bool = False) -> np.ndarray:
    """Writes into (and returns) ``c``; rows without entries are left untouched."""
    a, b, indptr, indices = _f32(a), _f32(b), _i32(indptr), _i32(indices)
    assert c.dtype == np.float32 and c.flags.c_contiguous
    fn = lib().oracle_csrmm_omp if omp else lib().oracle_csrmm
    fn(_p(a, _f32p), _p(b, _f32p), _p(c, _f32p), _p(indptr, _i32p), _p(indices, _i32p),
       int(m), int(n), int(feat), int(len(indices)))
    return c


def ell_spmm(w, rows, cols, b, c, feat) -> np.ndarray:
    """Accumulates one (partition, bucket) term into ``c``."""
    w, rows, cols, b = _f32(w), _i32(rows), _i32(cols), _f32(b)
    nrows = len(rows)
    width = (cols.size // nrows) if nrows else 0
    assert c.dtype == np.float32 and c.flags.c_contiguous
    lib().oracle_ell_spmm(_p(w, _f32p), _p(rows, _i32p), _p(cols, _i32p), nrows, width,
                          _p(b, _f32p), _p(c, _f32p), int(feat))
    return c


def edge_to_row(indptr, nnz: int) -> np.ndarray:
    indptr = _i32(indptr)
    out = np.empty((nnz,), np.int32)
    lib().oracle_edge_to_row(_p(indptr, _i32p), len(indptr) - 1, int(nnz), _p(out, _i32p))
    return out


def sddmm(a, b, indptr, indices, m, n, feat, scale=None, omp: bool = False) -> np.ndarray:
    a, b, indptr, indices = _f32(a), _f32(b), _i32(indptr), _i32(indices)
    sc = None if scale is None else _f32(scale)
    c = np.zeros((len(indices),), np.float32)
    fn = lib().oracle_sddmm_omp if omp else lib().oracle_sddmm
    fn(_p(a, _f32p), _p(b, _f32p), _p(c, _f32p), _p(indptr, _i32p), _p(indices, _i32p),
       _p(sc, _f32p), int(m), int(n), int(feat), int(len(indices)))
    return c


def bsrmm_f16(a, b, indptr, indices, nb, mb, blk, feat, omp: bool = False) -> np.ndarray:
    """fp16 blocks and dense operand, fp32 accumulate and output."""
    a = np.ascontiguousarray(a, dtype=np.float16)
    b = np.ascontiguousarray(b, dtype=np.float16)
    indptr, indices = _i32(indptr), _i32(indices)
    c = np.empty((nb * blk * feat,), np.float32)
    fn = lib().oracle_bsrmm_f16_omp if omp else lib().oracle_bsrmm_f16
    fn(_p(a.view(np.uint16), _u16p), _p(b.view(np.uint16), _u16p), _p(c, _f32p),
       _p(indptr, _i32p), _p(indices, _i32p), int(nb), int(mb), int(len(indices)), int(blk),
       int(feat))
    return c


def rgms(a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, m, n, num_rels, feat,
         omp: bool = False) -> np.ndarray:
    """Accumulates into (and returns) ``y``."""
    a, w, x = _f32(a), _f32(w), _f32(x)
    indptr_i, indices_i, indptr_j, indices_j = map(_i32, (indptr_i, indices_i, indptr_j, indices_j))
    assert y.dtype == np.float32 and y.flags.c_contiguous
    fn = lib().oracle_rgms_omp if omp else lib().oracle_rgms
    fn(_p(a, _f32p), _p(w, _f32p), _p(x, _f32p), _p(y, _f32p), _p(indptr_i, _i32p),
       _p(indices_i, _i32p), _p(indptr_j, _i32p), _p(indices_j, _i32p), int(m), int(n),
       int(num_rels), int(feat), int(len(indices_i)), int(len(indices_j)))
    return y


def rgms_ell3d(w, x, y, buckets, feat) -> np.ndarray:
    """Decomposed RGMS over ELL3D buckets; ``buckets`` is a list of ``(a, rows, cols, mid)`` with
    ``a``/``cols`` shaped ``[groups, rows_b, cols_b]`` and ``rows`` ``[groups, rows_b]``.
    Accumulates into (and returns) ``y``."""
    w, x = _f32(w), _f32(x)
    assert y.dtype == np.float32 and y.flags.c_contiguous
    for a, rows, cols, mid in buckets:
        a, rows, cols, mid = _f32(a), _i32(rows), _i32(cols), _i32(mid)
        ng = int(mid.shape[0])
        if ng == 0:
            continue
        rpg = rows.size // ng
        cpr = cols.size // rows.size
        lib().oracle_rgms_ell3d_bucket(_p(a, _f32p), _p(w, _f32p), _p(x, _f32p), _p(y, _f32p),
                                       _p(rows, _i32p), _p(cols, _i32p), _p(mid, _i32p), ng, rpg, cpr,
                                       int(feat))
    return y


def rgms_ell3d_f16(w, x, y, buckets, feat_in: int, feat_out: int) -> np.ndarray:
    """RGMS over ELL3D buckets with fp16 operands and rectangular weights ``w[r, fi, fo]``:
    ``y[rows[g,ii], fo] += a[g,ii,j] * sum_fi x[cols[g,ii,j], fi] * w[mid[g], fi, fo]`` — the two
    iterations of rgcn_hetero_forward in examples/rgms/rgcn/bench_rgcn_tensorcore.py:593-607 with
    every product and sum in fp32 (numpy; parity unpinned: the reference holds no fixture for it
    and cannot run here).  ``y`` is fp32, accumulated into and returned."""
    w = np.asarray(w, dtype=np.float16).astype(np.float32).reshape(-1, feat_in, feat_out)
    x = np.asarray(x, dtype=np.float16).astype(np.float32).reshape(-1, feat_in)
    assert y.dtype == np.float32 and y.flags.c_contiguous
    y2 = y.reshape(-1, feat_out)
    for a, rows, cols, mid in buckets:
        mid = _i32(mid)
        ng = int(mid.shape[0])
        if ng == 0:
            continue
        rows = _i32(rows).reshape(ng, -1)
        cols = _i32(cols).reshape(ng, rows.shape[1], -1)
        a = np.asarray(a, dtype=np.float16).astype(np.float32).reshape(cols.shape)
        for r in np.unique(mid):
            sel = mid == r
            z = (a[sel][..., None] * x[cols[sel]]).sum(axis=2, dtype=np.float32)  # groups x rows x feat_in
            np.add.at(y2, rows[sel].reshape(-1), z.reshape(-1, feat_in) @ w[r])
    return y


def tcspmm_f16(a, b, indptr, indices, mb, t, g, feat) -> np.ndarray:
    """Condensed SpMM: fp16 ``a`` [groups, t, g] and ``b`` [rows, feat], fp32 sums [mb * t, feat]."""
    a = np.ascontiguousarray(a, dtype=np.float16)
    b = np.ascontiguousarray(b, dtype=np.float16)
    indptr, indices = _i32(indptr), _i32(indices)
    c = np.empty((mb * t, feat), np.float32)
    u16p = ctypes.POINTER(ctypes.c_uint16)
    lib().oracle_tcspmm_f16(a.ctypes.data_as(u16p), b.ctypes.data_as(u16p), _p(c, _f32p), _p(indptr, _i32p),
                            _p(indices, _i32p), int(mb), int(t), int(g), int(feat))
    return c


def csr_reduce(a, indptr) -> np.ndarray:
    a, indptr = _f32(a), _i32(indptr)
    n = len(indptr) - 1
    b = np.empty((n,), np.float32)
    lib().oracle_csr_reduce(_p(a, _f32p), _p(b, _f32p), _p(indptr, _i32p), int(n))
    return b


def sparse_softmax(a, indptr) -> np.ndarray:
    a, indptr = _f32(a), _i32(indptr)
    b = np.empty_like(a)
    lib().oracle_sparse_softmax(_p(a, _f32p), _p(b, _f32p), _p(indptr, _i32p), int(len(indptr) - 1))
    return b


def csr2bsr(a, b, indptr_in, indices_in, indptr_out, indices_out, blk) -> np.ndarray:
    """Writes the stored entries into (and returns) the block array ``b`` [nnzb, blk, blk]."""
    a = _f32(a)
    assert b.dtype == np.float32 and b.flags.c_contiguous
    ip, ix, op, ox = map(_i32, (indptr_in, indices_in, indptr_out, indices_out))
    lib().oracle_csr2bsr(_p(a, _f32p), _p(b, _f32p), _p(ip, _i32p), _p(ix, _i32p), _p(op, _i32p),
                         _p(ox, _i32p), int(len(ip) - 1), int(blk))
    return b


def ellmm(a, b, indices, nb, col, blk, feat) -> np.ndarray:
    a, b, indices = _f32(a), _f32(b), _i32(indices)
    c = np.empty((nb * blk, feat), np.float32)
    lib().oracle_ellmm(_p(a, _f32p), _p(b, _f32p), _p(c, _f32p), _p(indices, _i32p), int(nb), int(col),
                       int(blk), int(feat))
    return c


def fusedmm(q, k, v, indptr, indices, m, feat) -> np.ndarray:
    q, k, v, indptr, indices = _f32(q), _f32(k), _f32(v), _i32(indptr), _i32(indices)
    o = np.empty((m, feat), np.float32)
    lib().oracle_fusedmm(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), _p(o, _f32p), _p(indptr, _i32p),
                         _p(indices, _i32p), int(m), int(feat))
    return o
