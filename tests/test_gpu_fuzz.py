"""Seeded random sweeps of the CUDA operators against the CPU oracle: sizes, degree
distributions (empty rows, hub rows), feature widths and decompositions are drawn at random, so
that dispatch boundaries nobody thought of listing by hand are crossed too.  Same tolerances as
the hand-written parity tests."""
import numpy as np
import pytest
import torch

import refimpl
import test_gpu_ops as T
from oracle import oracle as orc
from sparsetir_b200 import _lib as L
from sparsetir_b200 import datagen as dg
from sparsetir_b200 import ops

pytestmark = pytest.mark.gpu

FEATS = [1, 2, 3, 4, 7, 8, 12, 16, 20, 24, 32, 33, 48, 64, 65, 96, 100, 128, 160, 192, 256, 260, 384, 512]


def random_csr(rng: np.random.Generator, m: int, n: int, values="uniform") -> dg.CSR:
    """Degrees from a mixture: empty rows, short geometric rows, a few hub rows."""
    kind = rng.integers(0, 4)
    if kind == 0:
        deg = rng.poisson(rng.uniform(0.2, 12.0), size=m)
    elif kind == 1:
        deg = rng.geometric(rng.uniform(0.05, 0.6), size=m) - 1
    elif kind == 2:
        deg = np.clip(rng.zipf(rng.uniform(1.6, 2.6), size=m), 0, n)
    else:
        deg = np.zeros(m, np.int64)
        live = rng.random(m) < rng.uniform(0.05, 0.9)
        deg[live] = rng.integers(1, 40, size=int(live.sum()))
    deg = np.minimum(deg, n).astype(np.int64)
    hubs = rng.integers(0, 3)
    if hubs and m > 0:
        deg[rng.integers(0, m, size=hubs)] = rng.integers(n // 2, n + 1, size=hubs)
    indices = dg.sorted_distinct_columns(rng, deg, n)
    if values == "uniform":
        data = rng.uniform(-1.0, 1.0, size=len(indices)).astype(np.float32)
    else:
        data = np.ones(len(indices), np.float32)
    return dg.CSR(m, n, dg._indptr(deg), indices, data)


def pick_feat(rng):
    return int(FEATS[rng.integers(0, len(FEATS))])


@pytest.mark.parametrize("seed", range(24))
def test_fuzz_csrmm(cuda_device, seed):
    rng = np.random.default_rng(1000 + seed)
    m, n = int(rng.integers(1, 2500)), int(rng.integers(1, 2500))
    if seed % 6 == 0:
        m, n = int(rng.integers(8192, 12000)), int(rng.integers(300, 5000))  # sizes that take the hub-row path
    c = random_csr(rng, m, n)
    feat = pick_feat(rng)
    x = dg.dense_operand(seed, n, feat)
    T.parity(T.run_csrmm(c, x, cuda_device, scalars=bool(seed & 1), prefill=float(seed % 3)),
             T.oracle_csrmm(c, x), refimpl.spmm_f64(c.indptr, c.indices, c.data, x, c.m, c.n))


@pytest.mark.parametrize("seed", range(24))
def test_fuzz_hyb_spmm(cuda_device, seed):
    rng = np.random.default_rng(2000 + seed)
    n = int(rng.integers(2, 3000))
    c = random_csr(rng, n, n)
    feat = pick_feat(rng)
    parts = int(rng.integers(1, 5))
    nb = int(rng.integers(1, 8))
    buckets = sorted(set(int(b) for b in rng.choice([1, 2, 3, 4, 5, 8, 16, 24, 32, 64, 128, 256, 512], size=nb)))
    x = dg.dense_operand(seed, n, feat)
    host, devb = T.hyb_device_buckets(c, parts, buckets, cuda_device)
    y = torch.zeros(c.m * feat, device=cuda_device)
    ops.hyb_spmm(*ops.hyb_args(T.dev(x, cuda_device), y, devb, feat, L.HYB_ALL_ATOMIC if parts > 1 else 0))
    torch.cuda.synchronize()
    T.parity(y, T.oracle_hyb(host, x, c.m), refimpl.spmm_f64(c.indptr, c.indices, c.data, x, c.m, c.n))


@pytest.mark.parametrize("seed", range(24))
def test_fuzz_sddmm(cuda_device, seed):
    rng = np.random.default_rng(3000 + seed)
    m, n = int(rng.integers(1, 2000)), int(rng.integers(1, 2000))
    c = random_csr(rng, m, n)
    feat = pick_feat(rng)
    a = dg.dense_operand(seed, m, feat)
    b = dg.dense_operand(seed + 1, n, feat)
    want = orc.sddmm(a, b, c.indptr, c.indices, m, n, feat)
    got = T.run_sddmm(c, a, b, cuda_device, scalars=bool(seed & 1))
    if c.nnz:
        T.parity(got, want, refimpl.sddmm_f64(c.indptr, c.indices, a, b), groups=T.edge_rows(c.indptr))


@pytest.mark.parametrize("seed", range(16))
def test_fuzz_bsrmm(cuda_device, seed):
    rng = np.random.default_rng(4000 + seed)
    blk = int(rng.choice([4, 8, 16, 32, 64]))
    mb = int(rng.integers(1, 40))
    feat = int(rng.choice([8, 24, 32, 40, 64, 96, 128, 256, 512]))
    bs = dg.bsr_mask(size=mb * blk, blk=blk, density=float(rng.uniform(0.02, 0.5)), seed=seed)
    b = dg.dense_operand_normal(seed, mb * blk, feat)
    want = orc.bsrmm_f16(bs.data, b, bs.indptr, bs.indices, bs.mb, bs.nb, blk, feat, omp=True)
    T.close(T.run_bsrmm(bs, b, cuda_device), want, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("seed", range(20))
def test_fuzz_rgms_both_formats(cuda_device, seed):
    rng = np.random.default_rng(5000 + seed)
    n = int(rng.integers(10, 3000))
    rels = int(rng.integers(1, 60))
    edges = int(rng.integers(2 * rels, 30000))
    feat = int(rng.choice([64, 64, 64, 32, 128, 16, 8, 48]))
    cf = dg.csf_relational(n=n, num_rels=rels, num_edges=edges, zipf_a=float(rng.uniform(1.3, 2.5)), seed=seed)
    x = dg.dense_operand(seed, cf.n, feat)
    w = dg.relation_weights(seed + 1, cf.num_rels, feat)
    want = T.oracle_rgms(cf, x, w)
    # fp32 sums in another order than the oracle's: held to the stated tolerance against the float64
    # result, or to twice the oracle's own error where hundreds of edges end in one output
    T.parity(T.run_rgms(cf, x, w, cuda_device, scalars=bool(seed & 1)), want, T.rgms_truth(cf, x, w))
    cols_bkt = sorted(set(int(b) for b in rng.choice([1, 2, 4, 8, 16, 32], size=int(rng.integers(1, 5)))))
    # the ELL3D buckets carry the 0/1 mask as weights (as the reference example prepares them)
    buckets = T.ell3d_buckets(cf, cols_bkt)
    want3 = orc.rgms_ell3d(w, x, np.zeros((cf.m, feat), np.float32), buckets, feat)
    T.parity(T.run_rgms_ell3d(cf, x, w, buckets, cuda_device, feat), want3,
             T.rgms_truth(cf, x, w, data=np.ones(cf.nnz_j, np.float32)))


@pytest.mark.parametrize("seed", range(12))
def test_fuzz_tcspmm(cuda_device, seed):
    rng = np.random.default_rng(6000 + seed)
    n = int(rng.integers(20, 2500))
    g = random_csr(rng, n, n, values="ones")
    t = int(rng.choice([4, 8, 16, 32]))
    gs = int(rng.choice([8, 16]))
    feat = int(rng.choice([32, 64, 96, 128, 256, 512]))
    x16 = dg.dense_operand(seed, n, feat).astype(np.float16)
    got, want = T.run_tcspmm(g, x16, t, gs, cuda_device, torch.float32)
    np.testing.assert_allclose(got, want, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("seed", range(16))
def test_fuzz_row_wise_operators_and_attention(cuda_device, seed):
    rng = np.random.default_rng(7000 + seed)
    n = int(rng.integers(1, 2500))
    c = random_csr(rng, n, n)
    d = cuda_device
    if c.nnz == 0:
        return
    vals = rng.uniform(-3.0, 3.0, size=c.nnz).astype(np.float32)
    a = T.dev(vals, d)
    ip = T.dev(c.indptr, d)
    red = torch.full((n,), 5.0, device=d)
    ops.csr_reduce(a, red, ip)
    sm = torch.zeros(c.nnz, device=d)
    ops.sparse_softmax(a, sm, ip, T.dev(c.indices, d))
    torch.cuda.synchronize()
    T.parity(red, orc.csr_reduce(vals, c.indptr), refimpl.row_sums_f64(vals, c.indptr))
    T.close(sm, orc.sparse_softmax(vals, c.indptr), rtol=1e-4, atol=1e-6)
    feat = int(rng.choice([16, 24, 32, 64, 128, 256]))
    q = dg.dense_operand(seed, n, feat) * 0.3
    k = dg.dense_operand(seed + 1, n, feat) * 0.3
    v = dg.dense_operand(seed + 2, n, feat)
    o = torch.full((n * feat,), 2.0, device=d)
    ops.fusedmm(T.dev(q.reshape(-1), d), T.dev(k.reshape(-1), d), T.dev(v.reshape(-1), d), o, ip, T.dev(c.indices, d))
    torch.cuda.synchronize()
    T.parity(o, orc.fusedmm(q, k, v, c.indptr, c.indices, n, feat), refimpl.fusedmm_f64(q, k, v, c.indptr, c.indices))


@pytest.mark.parametrize("seed", range(16))
def test_fuzz_rgms_f16_rectangular(cuda_device, seed):
    rng = np.random.default_rng(8000 + seed)
    n = int(rng.integers(50, 3000))
    rels = int(rng.integers(1, 40))
    edges = int(rng.integers(2 * rels, 30000))
    feat_in = int(rng.choice([64, 128, 192, 256, 32, 16, 40, 8]))
    feat_out = int(rng.choice([64, 128, 192, 256, 32, 96, 24, 320]))
    cf = dg.csf_relational(n=n, num_rels=rels, num_edges=edges, zipf_a=float(rng.uniform(0.3, 2.5)), seed=seed)
    x16 = dg.dense_operand(seed, cf.n, feat_in).astype(np.float16)
    w16 = T.rect_weights(seed + 1, cf.num_rels, feat_in, feat_out)
    cols_bkt = sorted(set(int(b) for b in rng.choice([1, 2, 4, 8, 16, 32], size=int(rng.integers(1, 5)))))
    buckets = T.ell3d_buckets(cf, cols_bkt, group=int(rng.choice([1, 8, 32])))
    want = orc.rgms_ell3d_f16(w16, x16, np.zeros((cf.m, feat_out), np.float32), buckets, feat_in, feat_out)
    out_dtype = torch.float32 if seed & 1 else torch.float16
    got = T.run_rgms_ell3d_f16(cf, x16, w16, buckets, cuda_device, feat_in, feat_out, out_dtype)
    scale = max(1.0, float(np.abs(want).max()))
    T.close(got, want, rtol=1e-2, atol=(2e-2 if out_dtype == torch.float32 else 6e-2) * scale)
