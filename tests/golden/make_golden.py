"""Regenerates the golden fixtures in this directory:

    python tests/golden/make_golden.py [--reference /path/to/SparseTIR]

The format fixtures (``hyb_*.npz``, ``condense.npz``) are produced by the REFERENCE'S OWN test
functions, executed unmodified: ``scipy_column_part_hyb`` and ``condense_py`` are taken out of
``tests/python/sparsetir/test_format_conversion_routine.py`` of a SparseTIR checkout as syntax
trees (the module itself cannot be imported: its first lines import dgl and a compiled tvm,
which the two functions never touch) and run on seeded inputs.  ``scipy_column_part_hyb`` takes
a DGL graph only to ask it for ``g.adj(transpose=True, scipy_fmt="csr")``; it is given an
object that answers that one call with the scipy CSR matrix.  Every such fixture records the
file, the function and its line range in its ``source`` entry.  tests/refimpl.py (a vectorised
re-derivation written for this repository) must agree with them and is kept as a second opinion.

The operator fixtures hold seeded inputs with fp64 scipy / numpy results (the reference stores
no numeric vectors).  Neither the oracle nor the library takes part in producing any fixture.
"""
import argparse
import ast
import os
import sys
import types
from typing import List

import numpy as np
import scipy.sparse as sp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import refimpl  # noqa: E402
from sparsetir_b200 import datagen as dg  # noqa: E402


def save(name, **arrays):
    np.savez_compressed(os.path.join(HERE, name), **arrays)
    print(name, {k: getattr(v, "shape", v) for k, v in arrays.items()})


REF_TEST = "tests/python/sparsetir/test_format_conversion_routine.py"


def reference_test_functions(ref_root, names):
    """The named top-level functions of the reference's format test, compiled from its own
    source text without running the module's imports.  Returns {name: (callable, 'first-last')}."""
    path = os.path.join(ref_root, REF_TEST)
    with open(path) as f:
        tree = ast.parse(f.read(), filename=path)
    env = {"np": np, "List": List,
           # only named in an annotation of scipy_column_part_hyb
           "dgl": types.SimpleNamespace(DGLHeteroGraph=object)}
    out = {}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            mod = ast.Module(body=[node], type_ignores=[])
            exec(compile(mod, path, "exec"), env)
            out[node.name] = (env[node.name], f"{node.lineno}-{node.end_lineno}")
    missing = set(names) - set(out)
    if missing:
        raise RuntimeError(f"{path} has no function(s) {sorted(missing)}")
    return out


class _GraphStandIn:
    """Answers the one question scipy_column_part_hyb asks of its graph argument."""

    def __init__(self, mat):
        self._mat = mat

    def adj(self, transpose=True, scipy_fmt="csr"):
        assert transpose is True and scipy_fmt == "csr"
        return self._mat


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SPARSETIR_REFERENCE"),
                    help="SparseTIR checkout (or set SPARSETIR_REFERENCE)")
    ref_root = ap.parse_args().reference
    if not ref_root:
        ap.error("give the SparseTIR checkout with --reference or SPARSETIR_REFERENCE")
    fns = reference_test_functions(ref_root, ("scipy_column_part_hyb", "condense_py"))
    hyb_fn, hyb_lines = fns["scipy_column_part_hyb"]
    cond_fn, cond_lines = fns["condense_py"]

    # format conversion: the shape of the reference test (1000 nodes, 10000 edges, 4 parts, [1,2,4]),
    # then a rectangular matrix and a small power-law graph whose hub rows are split many times
    g = dg.random_csr(1000, 1000, 10000, seed=7)
    g_rect = dg.random_csr(600, 900, 7000, seed=11)
    g_hub = dg.csr_powerlaw(n=400, seed=5, max_deg=300)
    cases = (("a", g, 4, [1, 2, 4]), ("b", g, 1, [1, 2, 4, 8]), ("c", g, 3, [2, 8]),
             ("d", g_rect, 2, [1, 2, 4, 8, 16]), ("e", g_hub, 1, [1, 2]), ("f", g_hub, 4, [1, 4, 16]))
    for tag, gr, parts, buckets in cases:
        mat = sp.csr_matrix((np.ones(gr.nnz, np.float32), gr.indices, gr.indptr), shape=(gr.m, gr.n))
        rows, cols = hyb_fn(_GraphStandIn(mat), parts, list(buckets))
        # the vectorised re-derivation agrees with the reference's function
        rows2, cols2 = refimpl.scipy_column_part_hyb(gr.indptr, gr.indices, gr.m, gr.n, parts, buckets)
        assert len(rows) == len(rows2) == parts * len(buckets)
        for k in range(len(rows)):
            assert np.array_equal(np.asarray(rows[k]), rows2[k]) and np.array_equal(cols[k], cols2[k])
        arrays = {"indptr": gr.indptr, "indices": gr.indices, "parts": np.int64(parts),
                  "m": np.int64(gr.m), "n": np.int64(gr.n),
                  "buckets": np.asarray(buckets, np.int64),
                  "source": np.str_(f"{REF_TEST}:{hyb_lines} scipy_column_part_hyb, executed unmodified")}
        for k, (r, c) in enumerate(zip(rows, cols)):
            arrays[f"rows_{k}"] = np.asarray(r, np.int32)
            arrays[f"cols_{k}"] = np.asarray(c, np.int32)
        save(f"hyb_{tag}.npz", **arrays)
    ptr, idx = cond_fn(g.indptr, g.indices, 4)
    ptr2, idx2 = refimpl.condense_unique(g.indptr, g.indices, 4)
    assert np.array_equal(ptr, ptr2) and np.array_equal(idx, idx2)
    save("condense.npz", indptr=g.indptr, indices=g.indices, t=np.int64(4), out_indptr=ptr,
         out_indices=idx,
         source=np.str_(f"{REF_TEST}:{cond_lines} condense_py, executed unmodified"))

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
