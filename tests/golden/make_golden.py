"""Regenerates the golden fixtures in this directory:  python tests/golden/make_golden.py

The reference cannot be imported on the build machine (its Python package needs a compiled
TVM), so the fixtures hold seeded inputs together with expected outputs computed by
independent means (tests/refimpl.py): the scipy slicing derivation that the reference's own
format test uses for the hyb arrays, numpy ``unique`` for condensing, ``searchsorted`` for the
edge->row lookup and fp64 scipy/numpy products for the operators.  Neither the oracle nor the
library takes part in producing them.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import refimpl  # noqa: E402
from sparsetir_b200 import datagen as dg  # noqa: E402


def save(name, **arrays):
    np.savez_compressed(os.path.join(HERE, name), **arrays)
    print(name, {k: getattr(v, "shape", v) for k, v in arrays.items()})


def main():
    # format conversion: the shape of the reference test (1000 nodes, 10000 edges, 4 parts, [1,2,4])
    g = dg.random_csr(1000, 1000, 10000, seed=7)
    for tag, parts, buckets in (("a", 4, [1, 2, 4]), ("b", 1, [1, 2, 4, 8]), ("c", 3, [2, 8])):
        rows, cols = refimpl.scipy_column_part_hyb(g.indptr, g.indices, g.m, g.n, parts, buckets)
        arrays = {"indptr": g.indptr, "indices": g.indices, "parts": np.int64(parts),
                  "buckets": np.asarray(buckets, np.int64)}
        for k, (r, c) in enumerate(zip(rows, cols)):
            arrays[f"rows_{k}"] = r
            arrays[f"cols_{k}"] = c
        save(f"hyb_{tag}.npz", **arrays)
    ptr, idx = refimpl.condense_unique(g.indptr, g.indices, 4)
    save("condense.npz", indptr=g.indptr, indices=g.indices, t=np.int64(4), out_indptr=ptr,
         out_indices=idx)

    # edge -> row with empty rows at both ends and in the middle
    deg = np.array([0, 0, 3, 0, 1, 0, 0, 5, 2, 0], dtype=np.int64)
    ip = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    save("edge_to_row.npz", indptr=ip, mid=refimpl.edge_to_row(ip, int(ip[-1])))

    # operators, small, fp64 expectations
    c1 = dg.csr_poisson(m=96, n=80, mean_deg=5.0, seed=1)
    x = dg.dense_operand(2, c1.n, 24)
    save("csrmm.npz", indptr=c1.indptr, indices=c1.indices, data=c1.data, x=x,
         y=refimpl.spmm_f64(c1.indptr, c1.indices, c1.data, x, c1.m, c1.n))

    c3 = dg.csr_lognormal(n=120, mu=2.0, sigma=1.0, max_deg=60, seed=3)
    a = dg.dense_operand(4, c3.m, 32)
    b = dg.dense_operand(5, c3.n, 32)
    save("sddmm.npz", indptr=c3.indptr, indices=c3.indices, scale=c3.data, a=a, b=b,
         out=refimpl.sddmm_f64(c3.indptr, c3.indices, a, b),
         out_scaled=refimpl.sddmm_f64(c3.indptr, c3.indices, a, b, c3.data))

    bs = dg.bsr_mask(size=256, blk=32, density=0.2, seed=6)
    bd = dg.dense_operand_normal(7, 256, 64)
    save("bsrmm.npz", indptr=bs.indptr, indices=bs.indices, data=bs.data, b=bd,
         c=refimpl.bsrmm_f64(bs.indptr, bs.indices, bs.data, bd, bs.mb, bs.nb, bs.blk))

    cf = dg.csf_relational(n=300, num_rels=5, num_edges=2000, seed=8)
    xr = dg.dense_operand(9, cf.n, 64)
    wr = dg.relation_weights(10, cf.num_rels, 64)
    save("rgms.npz", indptr_i=cf.indptr_i, indices_i=cf.indices_i, indptr_j=cf.indptr_j,
         indices_j=cf.indices_j, data=cf.data, x=xr, w=wr,
         y=refimpl.rgms_f64(cf.data, wr, xr, cf.indptr_i, cf.indices_i, cf.indptr_j,
                            cf.indices_j, cf.m))


if __name__ == "__main__":
    main()
