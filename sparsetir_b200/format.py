"""Host-side format conversion with the names and argument order of ``tvm.sparse``
(python/tvm/sparse/format.py:89-170 of the reference), backed by the library's host C++.

Inputs are CPU int32 arrays (numpy or torch CPU tensors); outputs are numpy int32 arrays in the
reference's nesting.  Unlike the reference, which only accepts int32 NDArrays on the CPU
(src/sparse/format.cc:56-61), other integer dtypes are rejected here too rather than
converted silently.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib as L

_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)


def _as_i32(name: str, a) -> np.ndarray:
    if hasattr(a, "detach"):  # torch tensor
        if a.is_cuda:
            raise ValueError(f"Only support conversion on CPU: {name} is on {a.device}")
        a = a.detach().numpy()
    a = np.asarray(a)
    if a.dtype != np.int32:
        raise TypeError(f"Only support int32 index data type, got {a.dtype} for {name}.")
    return np.ascontiguousarray(a)


def _ptr(a: Optional[np.ndarray], ty):
    return ctypes.cast(None, ty) if a is None else a.ctypes.data_as(ty)


def column_part_hyb(num_rows: int, num_cols: int, indptr, indices, num_col_parts: int,
                    buckets: Sequence[int], data=None, num_threads: int = 0):
    """Partition a CSR matrix by columns and bucket the rows of every partition by length.

    Returns ``(row_indices, col_indices, mask)``, each a ``[num_col_parts][num_buckets]`` list of
    int32 arrays shaped ``[nrows]``, ``[nrows, bucket]``, ``[nrows, bucket]`` — the reference's
    result (python/tvm/sparse/format.py:89-116).  When ``data`` (the CSR values, float32) is
    given, a fourth list ``values`` with ``data`` scattered into the same slots (0 in padding)
    and a fifth list ``csr_pos`` (CSR position of every slot, -1 in padding) are appended.
    """
    lib = L.load()
    indptr = _as_i32("indptr", indptr)
    indices = _as_i32("indices", indices)
    if len(indptr) != num_rows + 1:
        raise ValueError("indptr must have num_rows + 1 entries")
    bk = np.asarray(list(buckets), dtype=np.int32)
    h = lib.sparsetir_column_part_hyb(int(num_rows), int(num_cols), _ptr(indptr, _i32p),
                                      _ptr(indices, _i32p), int(num_col_parts), _ptr(bk, _i32p),
                                      len(bk), int(num_threads))
    if not h:
        raise ValueError(L.last_error())
    dvals = None
    if data is not None:
        dvals = np.ascontiguousarray(np.asarray(data), dtype=np.float32)
        if len(dvals) != len(indices):
            lib.sparsetir_hyb_free(h)
            raise ValueError("data must have one value per stored entry")
    rows_o, cols_o, mask_o, vals_o, pos_o = [], [], [], [], []
    try:
        for p in range(num_col_parts):
            rp, cp, mp, vp, pp = [], [], [], [], []
            for b, width in enumerate(bk):
                n = lib.sparsetir_hyb_num_rows(h, p, b)
                r = np.empty((n,), np.int32)
                c = np.empty((n, int(width)), np.int32)
                m = np.empty((n, int(width)), np.int32)
                q = np.empty((n, int(width)), np.int32) if dvals is not None else None
                v = np.empty((n, int(width)), np.float32) if dvals is not None else None
                rc = lib.sparsetir_hyb_copy_bucket(h, p, b, _ptr(r, _i32p), _ptr(c, _i32p),
                                                   _ptr(m, _i32p), _ptr(q, _i32p),
                                                   _ptr(dvals, _f32p), _ptr(v, _f32p))
                if rc != 0:
                    raise ValueError(L.last_error())
                rp.append(r); cp.append(c); mp.append(m); vp.append(v); pp.append(q)
            rows_o.append(rp); cols_o.append(cp); mask_o.append(mp); vals_o.append(vp); pos_o.append(pp)
    finally:
        lib.sparsetir_hyb_free(h)
    if dvals is not None:
        return rows_o, cols_o, mask_o, vals_o, pos_o
    return rows_o, cols_o, mask_o


def condense(indptr, indices, t: int, g: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Condense a CSR matrix to (t x 1) tiles and group g tiles together.

    Returns ``(group_indptr[ceil(n/t)+1], tile_indices[groups, g], mask[groups, t, g])``
    (python/tvm/sparse/format.py:119-139 of the reference)."""
    lib = L.load()
    indptr = _as_i32("indptr", indptr)
    indices = _as_i32("indices", indices)
    n = len(indptr) - 1
    ntiles = (n + t - 1) // t
    gi = np.empty((ntiles + 1,), np.int32)
    ng = lib.sparsetir_condense(n, _ptr(indptr, _i32p), _ptr(indices, _i32p), int(t), int(g),
                                _ptr(gi, _i32p), _ptr(None, _i32p), _ptr(None, _i32p))
    if ng < 0:
        raise ValueError(L.last_error())
    ti = np.empty((ng, g), np.int32)
    mk = np.empty((ng, t, g), np.int32)
    rc = lib.sparsetir_condense(n, _ptr(indptr, _i32p), _ptr(indices, _i32p), int(t), int(g),
                                _ptr(gi, _i32p), _ptr(ti, _i32p), _ptr(mk, _i32p))
    if rc < 0:
        raise ValueError(L.last_error())
    return gi, ti, mk


def csf_to_ell3d(csf_indptr_0, csf_indices_0, csf_indptr_1, csf_indices_1,
                 nnz_rows_bkt: Sequence[int], nnz_cols_bkt: Sequence[int]):
    """3-level CSF (relation, row, column) to per-bucket ELL3D.

    Returns ``(indptr, row_indices, col_indices, mask)``, each a per-bucket list with shapes
    ``[num_rels+1]``, ``[groups, rows_b]``, ``[groups, rows_b, cols_b]``, ``[groups, rows_b, cols_b]``
    (python/tvm/sparse/format.py:142-170 of the reference)."""
    lib = L.load()
    ip0, ix0 = _as_i32("csf_indptr_0", csf_indptr_0), _as_i32("csf_indices_0", csf_indices_0)
    ip1, ix1 = _as_i32("csf_indptr_1", csf_indptr_1), _as_i32("csf_indices_1", csf_indices_1)
    rb = np.asarray(list(nnz_rows_bkt), dtype=np.int32)
    cb = np.asarray(list(nnz_cols_bkt), dtype=np.int32)
    if len(rb) != len(cb):
        raise ValueError("Input nnz_rows and nnz_cols should have same length.")
    R = len(ip0) - 1
    h = lib.sparsetir_csf_to_ell3d(R, _ptr(ip0, _i32p), _ptr(ix0, _i32p), _ptr(ip1, _i32p),
                                   _ptr(ix1, _i32p), _ptr(rb, _i32p), _ptr(cb, _i32p), len(rb))
    if not h:
        raise ValueError(L.last_error())
    out: Tuple[List, List, List, List] = ([], [], [], [])
    try:
        for b in range(len(rb)):
            ng = lib.sparsetir_ell3d_num_groups(h, b)
            ip = np.empty((R + 1,), np.int32)
            r = np.empty((ng, int(rb[b])), np.int32)
            c = np.empty((ng, int(rb[b]), int(cb[b])), np.int32)
            m = np.empty((ng, int(rb[b]), int(cb[b])), np.int32)
            if lib.sparsetir_ell3d_copy_bucket(h, b, _ptr(ip, _i32p), _ptr(r, _i32p),
                                               _ptr(c, _i32p), _ptr(m, _i32p)) != 0:
                raise ValueError(L.last_error())
            for lst, arr in zip(out, (ip, r, c, m)):
                lst.append(arr)
    finally:
        lib.sparsetir_ell3d_free(h)
    return out


def row_partition(indptr, num_shards: int) -> np.ndarray:
    """nnz-balanced contiguous row cuts, int64 ``[num_shards + 1]`` (multi-GPU layer)."""
    lib = L.load()
    indptr = _as_i32("indptr", indptr)
    cuts = np.empty((num_shards + 1,), np.int64)
    rc = lib.sparsetir_row_partition(len(indptr) - 1, _ptr(indptr, _i32p), int(num_shards),
                                     cuts.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)))
    if rc != 0:
        raise ValueError(L.last_error())
    return cuts
