"""Parity of the CUDA kernels with the CPU oracle, called through the packed C ABI exactly like
the reference calls a built operator.  Tolerances are the ones stated for this path: bit-exact
integers; fp32 rtol 1e-4 / atol 1e-5; fp16 inputs with fp32 accumulation rtol 1e-2."""
import ctypes
import os

import numpy as np
import pytest
import torch

import refimpl
from oracle import oracle as orc
from sparsetir_b200 import _lib as L
from sparsetir_b200 import datagen as dg
from sparsetir_b200 import format as fmt
from sparsetir_b200 import ops

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
RTOL, ATOL = 1e-4, 1e-5


def dev(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def close(got: torch.Tensor, want: np.ndarray, rtol=RTOL, atol=ATOL):
    np.testing.assert_allclose(got.cpu().numpy().reshape(want.shape), want, rtol=rtol, atol=atol)


def parity(got, oracle: np.ndarray, truth: np.ndarray, rtol=RTOL, atol=ATOL, groups=None):
    """The stated fp32 bar, held against a float64 result instead of being widened by hand.

    ``truth`` is the float64 value of the same expression, ``oracle`` the CPU oracle's fp32
    result (reference summation order).  Every element of ``got`` must be within the stated
    tolerance of ``truth`` — or, where fp32 sums of that length cannot get that close, within
    twice the error the oracle itself makes: element-wise against the largest oracle error of
    the same output row (rounding errors of two different summation orders are independent
    element by element; their scale is a property of the row's sum).  ``groups`` gives the row
    of every element of a flat per-position result; 2-D results use their first axis.
    Also asserts that the oracle meets the same bound, so a wrong oracle cannot loosen it."""
    g = (got.detach().float().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got))
    truth = np.asarray(truth, np.float64)
    g = g.reshape(truth.shape).astype(np.float64)
    o = np.asarray(oracle).reshape(truth.shape).astype(np.float64)
    err_g, err_o = np.abs(g - truth), np.abs(o - truth)
    if truth.ndim == 2:
        row_o = np.broadcast_to(err_o.max(axis=1, keepdims=True), truth.shape) if truth.size else err_o
    elif groups is not None and truth.size:
        top = np.zeros(int(np.max(groups)) + 1)
        np.maximum.at(top, groups, err_o)
        row_o = top[groups]
    else:
        row_o = err_o
    stated = atol + rtol * np.abs(truth)
    bound = np.maximum(stated, 2.0 * row_o)
    bad = err_g > bound
    if bad.any():
        k = int(np.argmax(err_g - bound))
        raise AssertionError(
            f"{int(bad.sum())} of {bad.size} elements beyond max(stated tolerance, 2 x oracle error): "
            f"worst at flat index {k}: got {g.flat[k]!r}, float64 {truth.flat[k]!r}, error {err_g.flat[k]:.3e}, "
            f"stated {stated.flat[k]:.3e}, oracle error of its row {row_o.flat[k]:.3e}; "
            f"max GPU error {err_g.max():.3e}, max oracle error {err_o.max():.3e}")
    return float(err_g.max()), float(err_o.max())


def edge_rows(indptr) -> np.ndarray:
    return np.repeat(np.arange(len(indptr) - 1), np.diff(indptr))


# ------------------------------------------------------------------------------ csrmm
def run_csrmm(c: dg.CSR, x: np.ndarray, device, scalars=False, prefill=0.0):
    feat = x.shape[1]
    y = torch.full((c.m * feat,), prefill, dtype=torch.float32, device=device)
    args = [dev(c.data, device), dev(x.reshape(-1), device), y, dev(c.indptr, device),
            dev(c.indices, device)]
    if scalars:
        args += [c.m, c.n, feat, c.nnz]
    ops.csrmm(*args)
    torch.cuda.synchronize()
    return y.reshape(c.m, feat)


def oracle_csrmm(c: dg.CSR, x: np.ndarray):
    y = np.zeros((c.m, x.shape[1]), np.float32)
    return orc.csrmm(c.data, x, y, c.indptr, c.indices, c.m, c.n, x.shape[1])


@pytest.mark.parametrize("feat", [1, 3, 4, 24, 32, 64, 100, 128, 256, 512, 640])
def test_csrmm_matches_oracle(cuda_device, feat):
    c = dg.csr_poisson(m=1000, n=700, mean_deg=10, seed=feat)
    x = dg.dense_operand(1, c.n, feat)
    close(run_csrmm(c, x, cuda_device, scalars=feat % 2 == 0), oracle_csrmm(c, x))


def test_csrmm_config1_full_size(cuda_device):
    c = dg.csr_poisson(seed=0)  # 4096 x 4096, Poisson(10)
    x = dg.dense_operand(0, c.n, 64)
    got = run_csrmm(c, x, cuda_device)
    close(got, oracle_csrmm(c, x))
    close(got, refimpl.spmm_f64(c.indptr, c.indices, c.data, x, c.m, c.n).astype(np.float32))


def test_csrmm_golden(cuda_device):
    g = np.load(os.path.join(GOLD, "csrmm.npz"))
    c = dg.CSR(g["y"].shape[0], g["x"].shape[0], g["indptr"], g["indices"], g["data"])
    close(run_csrmm(c, g["x"], cuda_device), g["y"].astype(np.float32))


def test_csrmm_empty_rows_are_zeroed_and_long_rows(cuda_device):
    # empty rows at the start, middle and end; one row far longer than the rest
    deg = np.array([0, 0, 5, 0, 900, 1, 0, 0, 3, 0, 0], np.int64)
    rng = np.random.default_rng(0)
    ip = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    ix = dg.sorted_distinct_columns(rng, deg, 1000)
    c = dg.CSR(len(deg), 1000, ip, ix, rng.uniform(-1, 1, len(ix)).astype(np.float32))
    x = dg.dense_operand(3, 1000, 64)
    got = run_csrmm(c, x, cuda_device, prefill=9.0)
    close(got, oracle_csrmm(c, x))
    assert torch.all(got[[0, 1, 3, 6, 7, 9, 10]] == 0)


def test_csrmm_powerlaw_rows(cuda_device):
    c = dg.csr_powerlaw(n=20000, seed=5)
    x = dg.dense_operand(6, c.n, 32)
    close(run_csrmm(c, x, cuda_device), oracle_csrmm(c, x))


def test_csrmm_unaligned_operands(cuda_device):
    c = dg.csr_poisson(m=300, n=300, mean_deg=7, seed=8)
    x = dg.dense_operand(9, c.n, 16)
    base = torch.zeros(c.n * 16 + 1, dtype=torch.float32, device=cuda_device)
    base[1:] = dev(x.reshape(-1), cuda_device)
    y = torch.zeros(c.m * 16, dtype=torch.float32, device=cuda_device)
    ops.csrmm(dev(c.data, cuda_device), base[1:], y, dev(c.indptr, cuda_device), dev(c.indices, cuda_device))
    close(y, oracle_csrmm(c, x))


def test_csrmm_all_rows_empty_and_zero_sizes(cuda_device):
    y = torch.full((5 * 8,), 3.0, device=cuda_device)
    e_f = torch.zeros(0, device=cuda_device)
    e_i = torch.zeros(0, dtype=torch.int32, device=cuda_device)
    ops.csrmm(e_f, torch.ones(4 * 8, device=cuda_device), y,
              torch.zeros(6, dtype=torch.int32, device=cuda_device), e_i, 5, 4, 8, 0)
    torch.cuda.synchronize()
    assert torch.all(y == 0)


# ------------------------------------------------------------------------------ hyb spmm
def hyb_device_buckets(c: dg.CSR, parts, buckets, device, weights="values"):
    rows, cols, mask, vals, pos = fmt.column_part_hyb(c.m, c.n, c.indptr, c.indices, parts, buckets,
                                                     data=c.data)
    host, devb = [], []
    for p in range(parts):
        for b in range(len(buckets)):
            w = vals[p][b] if weights == "values" else mask[p][b].astype(np.float32)
            host.append((w, rows[p][b], cols[p][b]))
            devb.append((dev(w, device), dev(rows[p][b], device), dev(cols[p][b], device)))
    return host, devb


def oracle_hyb(host, x, m):
    y = np.zeros((m, x.shape[1]), np.float32)
    for w, rows, cols in host:
        orc.ell_spmm(w, rows, cols, x, y, x.shape[1])
    return y


BK10 = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512]


@pytest.mark.parametrize("feat", [32, 64, 128, 256, 512])
@pytest.mark.parametrize("parts", [1, 2, 4])
def test_hyb_spmm_matches_oracle(cuda_device, feat, parts):
    c = dg.csr_powerlaw(n=6000, max_deg=4000, seed=parts)
    x = dg.dense_operand(feat, c.n, feat)
    host, devb = hyb_device_buckets(c, parts, BK10, cuda_device)
    y = torch.zeros(c.m * feat, device=cuda_device)
    flags = L.HYB_ALL_ATOMIC if parts > 1 else 0
    ops.hyb_spmm(*ops.hyb_args(dev(x, cuda_device), y, devb, feat, flags))
    torch.cuda.synchronize()
    want = oracle_hyb(host, x, c.m)
    close(y, want)
    # and the decomposition computes the same product as the CSR form
    close(y, refimpl.spmm_f64(c.indptr, c.indices, c.data, x, c.m, c.n).astype(np.float32))


def test_hyb_spmm_full_size_graph_properties(cuda_device):
    # the bench workload at full size (169,343 nodes), checked through properties that need no CPU
    # pass over it: the hyb product equals the CSR product of the same matrix, the operator is
    # linear in X, and a sample of rows matches the oracle
    c = dg.csr_powerlaw(seed=0)
    feat = 64
    d = cuda_device
    x1 = dev(dg.dense_operand(1, c.n, feat), d)
    x2 = dev(dg.dense_operand(2, c.n, feat), d)
    _, devb = hyb_device_buckets(c, 1, BK10, d)

    def hyb(x):
        y = torch.zeros(c.m * feat, device=d)
        ops.hyb_spmm(*ops.hyb_args(x, y, devb, feat, 0))
        return y

    y1, y2 = hyb(x1), hyb(x2)
    y12 = hyb(2.0 * x1 - 0.5 * x2)
    ycsr = torch.zeros(c.m * feat, device=d)
    ops.csrmm(dev(c.data, d), x1.reshape(-1), ycsr, dev(c.indptr, d), dev(c.indices, d))
    torch.cuda.synchronize()
    torch.testing.assert_close(y1, ycsr, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(y12, 2.0 * y1 - 0.5 * y2, rtol=RTOL, atol=4 * ATOL)
    rows = np.random.default_rng(0).choice(c.m, size=2000, replace=False)
    rows = np.concatenate([rows, np.argsort(np.diff(c.indptr))[-5:]])  # and the five longest rows
    x1h = x1.cpu().numpy()
    y1h = y1.cpu().numpy().reshape(c.m, feat)
    for r in rows:
        sl = slice(c.indptr[r], c.indptr[r + 1])
        want = (c.data[sl, None].astype(np.float64) * x1h[c.indices[sl]]).sum(0)
        np.testing.assert_allclose(y1h[r], want, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("parts", [1, 2, 4])
def test_hyb_spmm_config2_whole_output_all_feature_sizes(cuda_device, parts):
    # the bench workload at full size, every output element, all five feature sizes, with 1, 2 and
    # 4 column partitions: against the oracle's CSR loop nest on the same matrix (OpenMP over rows,
    # same summation order per row) and the float64 product
    c = dg.csr_powerlaw(seed=0)
    d = cuda_device
    _, devb = hyb_device_buckets(c, parts, BK10, d)
    orc.use_all_cores()
    for feat in (32, 64, 128, 256, 512):
        x = dg.dense_operand(100 + feat, c.n, feat)
        y = torch.zeros(c.m * feat, device=d)
        ops.hyb_spmm(*ops.hyb_args(dev(x, d), y, devb, feat, L.HYB_ALL_ATOMIC if parts > 1 else 0))
        torch.cuda.synchronize()
        want = orc.csrmm(c.data, x, np.zeros((c.m, feat), np.float32), c.indptr, c.indices, c.m, c.n, feat,
                         omp=True)
        parity(y, want, refimpl.spmm_f64(c.indptr, c.indices, c.data, x, c.m, c.n))
        if parts == 1:  # one writer per output row: repeated calls give the same bits
            y2 = torch.zeros(c.m * feat, device=d)
            ops.hyb_spmm(*ops.hyb_args(dev(x, d), y2, devb, feat, 0))
            torch.cuda.synchronize()
            assert torch.equal(y, y2)
        del y


@pytest.mark.parametrize("feat,buckets,parts", [(8, [1, 3, 5], 1), (20, [2, 7], 3), (33, [1, 2, 4], 2),
                                                (640, [4, 64], 1), (1, [1, 2], 1)])
def test_hyb_spmm_odd_shapes(cuda_device, feat, buckets, parts):
    c = dg.csr_poisson(m=500, n=800, mean_deg=9, seed=feat)
    x = dg.dense_operand(2, c.n, feat)
    host, devb = hyb_device_buckets(c, parts, buckets, cuda_device)
    y = torch.zeros(c.m * feat, device=cuda_device)
    ops.hyb_spmm(*ops.hyb_args(dev(x, cuda_device), y, devb, feat, L.HYB_ALL_ATOMIC if parts > 1 else 0))
    torch.cuda.synchronize()
    close(y, oracle_hyb(host, x, c.m))


def test_hyb_spmm_mask_weights_like_reference_example(cuda_device):
    # examples/spmm/bench_spmm.py:212-214 feeds the mask as weights (unweighted copy_u_sum)
    c = dg.csr_powerlaw(n=3000, max_deg=2000, seed=21)
    x = dg.dense_operand(22, c.n, 64)
    host, devb = hyb_device_buckets(c, 2, [1, 2, 4, 8], cuda_device, weights="mask")
    y = torch.zeros(c.m * 64, device=cuda_device)
    ops.hyb_spmm(*ops.hyb_args(dev(x, cuda_device), y, devb, 64, L.HYB_ALL_ATOMIC))
    torch.cuda.synchronize()
    ones = dg.CSR(c.m, c.n, c.indptr, c.indices, np.ones(c.nnz, np.float32))
    close(y, oracle_csrmm(ones, x))


def test_hyb_spmm_zero_and_rearm_flags(cuda_device):
    c = dg.csr_powerlaw(n=4000, max_deg=3000, seed=23)
    x = dg.dense_operand(24, c.n, 128)
    host, devb = hyb_device_buckets(c, 1, [1, 2, 4, 8, 16], cuda_device)  # many split rows
    want = oracle_hyb(host, x, c.m)
    xd = dev(x, cuda_device)
    # ZERO_C: garbage in C does not matter
    y = torch.full((c.m * 128,), 5.0, device=cuda_device)
    ops.hyb_spmm(*ops.hyb_args(xd, y, devb, 128, L.HYB_ZERO_C))
    close(y, want)
    # every row has one writer: repeated calls on the same C, with or without the re-arm flag,
    # leave the same bits, whatever C held in the rows that occur in a bucket
    y = torch.zeros(c.m * 128, device=cuda_device)
    ops.hyb_spmm(*ops.hyb_args(xd, y, devb, 128))
    first = y.clone()
    close(first, want)
    for flags in (0, L.HYB_REARM, 0):
        ops.hyb_spmm(*ops.hyb_args(xd, y, devb, 128, flags))
        assert torch.equal(y, first)
    # ALL_ATOMIC adds into C: with the re-arm flag the call clears C first
    host4, devb4 = hyb_device_buckets(c, 4, [1, 2, 4, 8, 16], cuda_device)
    y = torch.zeros(c.m * 128, device=cuda_device)
    for _ in range(2):
        ops.hyb_spmm(*ops.hyb_args(xd, y, devb4, 128, L.HYB_REARM | L.HYB_ALL_ATOMIC))
    close(y, oracle_hyb(host4, x, c.m))
    # without it a second call adds the product once more (the reference's atomic buckets)
    y = torch.zeros(c.m * 128, device=cuda_device)
    for _ in range(2):
        ops.hyb_spmm(*ops.hyb_args(xd, y, devb4, 128, L.HYB_ALL_ATOMIC))
    close(y, 2 * oracle_hyb(host4, x, c.m), atol=2 * ATOL)


@pytest.mark.parametrize("buckets", [[1, 2, 4], [2, 8], [1, 2, 4, 8, 16, 32, 64], [4, 512], [8, 1024], [16, 24, 200]])
@pytest.mark.parametrize("feat", [32, 64, 256, 512])
def test_hyb_spmm_split_and_wide_rows_have_one_writer(cuda_device, buckets, feat):
    # hub rows of up to 5,000 entries: split into many ELL rows of the last bucket (narrow last
    # buckets: pieces inside and across work items; wide ones: spans of one block plus the scratch
    # rows).  The result must match the oracle and be bit-identical when repeated, also on a C
    # that holds garbage in the rows the matrix touches.
    deg = np.random.default_rng(3).integers(0, 12, size=3000).astype(np.int64)
    deg[[0, 1, 2, 1500, 2998, 2999]] = [5000, 513, 1025, 2999, 4, 700]
    rng = np.random.default_rng(4)
    ix = dg.sorted_distinct_columns(rng, deg, 6000)
    c = dg.CSR(3000, 6000, dg._indptr(deg), ix, rng.uniform(-1, 1, size=len(ix)).astype(np.float32))
    x = dg.dense_operand(5, c.n, feat)
    host, devb = hyb_device_buckets(c, 1, buckets, cuda_device)
    touched = torch.from_numpy((deg > 0).repeat(feat)).to(cuda_device)
    y = torch.zeros(c.m * feat, device=cuda_device)
    ops.hyb_spmm(*ops.hyb_args(dev(x, cuda_device), y, devb, feat))
    torch.cuda.synchronize()
    parity(y, oracle_hyb(host, x, c.m), refimpl.spmm_f64(c.indptr, c.indices, c.data, x, c.m, c.n))
    y2 = torch.where(touched, torch.full_like(y, 7.0), torch.zeros_like(y))
    for _ in range(3):
        ops.hyb_spmm(*ops.hyb_args(dev(x, cuda_device), y2, devb, feat))
        torch.cuda.synchronize()
        assert torch.equal(y, y2)


def test_hyb_spmm_scratch_limit_falls_back_to_atomics_in_child_process(cuda_device):
    # SPARSETIR_HYB_SCRATCH_MB=0 (read once per process): no scratch rows for split rows, the call
    # clears C and adds everything atomically instead
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
            "import numpy as np, torch, test_gpu_ops as T\n"
            "from sparsetir_b200 import datagen as dg, ops\n"
            "d = torch.device('cuda', 0)\n"
            "c = dg.csr_powerlaw(n=4000, max_deg=3000, seed=23)\n"
            "x = dg.dense_operand(24, c.n, 64)\n"
            "host, devb = T.hyb_device_buckets(c, 1, [1, 2, 4, 8], d)\n"
            "y = torch.full((c.m * 64,), 3.0, device=d)\n"
            "y.view(c.m, 64)[np.diff(c.indptr) == 0] = 0\n"
            "ops.hyb_spmm(*ops.hyb_args(T.dev(x, d), y, devb, 64))\n"
            "torch.cuda.synchronize()\n"
            "T.close(y, T.oracle_hyb(host, x, c.m))\n"
            "print('fallback ok')" % (root, os.path.join(root, "tests")))
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, SPARSETIR_HYB_SCRATCH_MB="0"),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "fallback ok" in r.stdout, r.stdout + r.stderr


def test_hyb_spmm_no_buckets_and_empty_buckets(cuda_device):
    x = torch.ones(4 * 8, device=cuda_device)
    y = torch.zeros(4 * 8, device=cuda_device)
    ops.hyb_spmm(x, y, 8)
    e_f = torch.zeros(0, device=cuda_device)
    e_i = torch.zeros(0, dtype=torch.int32, device=cuda_device)
    ops.hyb_spmm(x, y, e_f, e_i, e_i, 8)
    torch.cuda.synchronize()
    assert torch.all(y == 0)


def test_hyb_spmm_raw_entry_matches_packed(cuda_device):
    import ctypes
    c = dg.csr_powerlaw(n=2000, max_deg=900, seed=25)
    x = dg.dense_operand(26, c.n, 64)
    host, devb = hyb_device_buckets(c, 1, [1, 2, 4, 8], cuda_device)
    xd = dev(x, cuda_device)
    y1 = torch.zeros(c.m * 64, device=cuda_device)
    ops.hyb_spmm(*ops.hyb_args(xd, y1, devb, 64))
    arr = (L.EllBucket * len(devb))()
    for k, (w, r, cc) in enumerate(devb):
        arr[k] = L.EllBucket(w.data_ptr(), r.data_ptr(), cc.data_ptr(), r.numel(),
                             cc.numel() // max(1, r.numel()))
    y2 = torch.zeros(c.m * 64, device=cuda_device)
    rc = L.load().sparsetir_hyb_spmm_raw(xd.data_ptr(), y2.data_ptr(), arr, len(devb), c.m, c.n, 64, 0,
                                         0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, L.last_error()
    torch.cuda.synchronize()
    assert torch.equal(y2, y1)  # one writer per row: the same bits through either entry point
    # the scratch a call needs can be asked for and reserved up front
    sb, cb = ctypes.c_size_t(0), ctypes.c_size_t(0)
    assert L.load().sparsetir_hyb_spmm_workspace(arr, len(devb), 64, ctypes.byref(sb), ctypes.byref(cb)) == 0
    n_last = devb[-1][1].numel()
    assert sb.value == n_last * 64 * 4 and cb.value == n_last * 2 * 4


# ------------------------------------------------------------------------------ sddmm
def run_sddmm(c: dg.CSR, a, b, device, scale=None, scalars=False):
    out = torch.full((c.nnz,), -7.0, device=device)
    args = [dev(a.reshape(-1), device), dev(b.reshape(-1), device), out, dev(c.indptr, device),
            dev(c.indices, device)]
    if scalars:
        args += [c.m, c.n, a.shape[1], c.nnz]
    if scale is not None:
        args.append(dev(scale, device))
    ops.sddmm(*args)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("feat", [1, 4, 8, 20, 32, 64, 96, 128, 160, 200, 256, 320, 512, 516, 1024])
def test_sddmm_matches_oracle(cuda_device, feat):
    c = dg.csr_lognormal(n=900, mu=3.0, sigma=1.0, max_deg=500, seed=feat)
    a = dg.dense_operand(1, c.m, feat)
    b = dg.dense_operand(2, c.n, feat)
    want = orc.sddmm(a, b, c.indptr, c.indices, c.m, c.n, feat)
    parity(run_sddmm(c, a, b, cuda_device, scalars=feat % 8 == 0), want,
           refimpl.sddmm_f64(c.indptr, c.indices, a, b), groups=edge_rows(c.indptr))


def test_sddmm_scale_and_golden(cuda_device):
    g = np.load(os.path.join(GOLD, "sddmm.npz"))
    c = dg.CSR(g["a"].shape[0], g["b"].shape[0], g["indptr"], g["indices"], g["scale"])
    close(run_sddmm(c, g["a"], g["b"], cuda_device), g["out"].astype(np.float32))
    close(run_sddmm(c, g["a"], g["b"], cuda_device, scale=g["scale"]), g["out_scaled"].astype(np.float32))
    close(run_sddmm(c, g["a"], g["b"], cuda_device, scale=g["scale"], scalars=True),
          orc.sddmm(g["a"], g["b"], c.indptr, c.indices, c.m, c.n, 32, scale=g["scale"]))


def test_sddmm_empty_rows_and_tails(cuda_device):
    # long runs of empty rows (walk falls back to the search), chunk and batch tails
    deg = np.zeros(3000, np.int64)
    deg[[0, 5, 6, 700, 2999]] = [3, 1, 290, 37, 2]
    rng = np.random.default_rng(1)
    ip = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    ix = dg.sorted_distinct_columns(rng, deg, 400)
    c = dg.CSR(3000, 400, ip, ix, np.ones(len(ix), np.float32))
    for feat in (32, 64, 128):
        a = dg.dense_operand(3, c.m, feat)
        b = dg.dense_operand(4, c.n, feat)
        close(run_sddmm(c, a, b, cuda_device), orc.sddmm(a, b, c.indptr, c.indices, c.m, c.n, feat))


def test_sddmm_long_chunks_and_feature_tiles(cuda_device):
    # more than 2^22 stored positions (the kernel then gives a warp 1024 of them) and feature
    # counts that take several launches, with and without the per-position scale
    c = dg.csr_lognormal(n=20000, mu=5.3, sigma=0.6, max_deg=4000, seed=11)
    assert c.nnz > (1 << 22)
    scale = np.random.default_rng(5).random(c.nnz, dtype=np.float32)
    for feat, sc in ((32, None), (96, scale)):
        a = dg.dense_operand(5, c.m, feat)
        b = dg.dense_operand(6, c.n, feat)
        want = orc.sddmm(a, b, c.indptr, c.indices, c.m, c.n, feat, scale=sc)
        parity(run_sddmm(c, a, b, cuda_device, scale=sc), want,
               refimpl.sddmm_f64(c.indptr, c.indices, a, b, sc), groups=edge_rows(c.indptr))


def test_sddmm_operands_not_32_byte_aligned(cuda_device):
    # operands that start 16 bytes into an allocation take the 16-byte-vector kernel
    c = dg.csr_lognormal(n=700, mu=3.0, sigma=1.0, max_deg=300, seed=3)
    feat = 64
    a = dg.dense_operand(7, c.m, feat)
    b = dg.dense_operand(8, c.n, feat)
    abuf = torch.zeros(a.size + 4, device=cuda_device)
    bbuf = torch.zeros(b.size + 4, device=cuda_device)
    abuf[4:] = dev(a.reshape(-1), cuda_device)
    bbuf[4:] = dev(b.reshape(-1), cuda_device)
    out = torch.full((c.nnz,), -7.0, device=cuda_device)
    ip, ix = dev(c.indptr, cuda_device), dev(c.indices, cuda_device)
    rc = L.load().sparsetir_sddmm_raw(abuf.data_ptr() + 16, bbuf.data_ptr() + 16, out.data_ptr(),
                                      ip.data_ptr(), ix.data_ptr(), None, c.m, c.n, feat, c.nnz,
                                      0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, L.last_error()
    torch.cuda.synchronize()
    parity(out, orc.sddmm(a, b, c.indptr, c.indices, c.m, c.n, feat),
           refimpl.sddmm_f64(c.indptr, c.indices, a, b), groups=edge_rows(c.indptr))


def test_sddmm_full_size_graph_properties(cuda_device):
    # config 3 at full size (232,965 nodes, about 117 M stored positions): sampled positions
    # against float64 dot products (first, last, and the rows around the longest one included),
    # and linearity in the row-side operand
    c = dg.csr_lognormal(seed=0)
    feat = 32
    d = cuda_device
    a1 = dg.dense_operand(1, c.m, feat)
    b = dg.dense_operand(2, c.n, feat)
    ip, ix = dev(c.indptr, d), dev(c.indices, d)
    bd = dev(b.reshape(-1), d)

    def run(a):
        out = torch.empty(c.nnz, device=d)
        ops.sddmm(dev(a.reshape(-1), d), bd, out, ip, ix)
        return out

    o1 = run(a1)
    a2 = dg.dense_operand(3, c.m, feat)
    o2 = run(a2)
    o12 = run((1.5 * a1 - 2.0 * a2).astype(np.float32))
    torch.cuda.synchronize()
    torch.testing.assert_close(o12, 1.5 * o1 - 2.0 * o2, rtol=RTOL, atol=8 * ATOL)
    rng = np.random.default_rng(0)
    pos = np.concatenate([rng.integers(0, c.nnz, size=20000), [0, c.nnz - 1]])
    longest = int(np.argmax(np.diff(c.indptr)))
    pos = np.concatenate([pos, np.arange(c.indptr[longest], min(c.nnz, c.indptr[longest] + 300))])
    rows = np.searchsorted(c.indptr, pos, side="right") - 1
    want = np.einsum("ij,ij->i", a1[rows].astype(np.float64), b[c.indices[pos]].astype(np.float64))
    np.testing.assert_allclose(o1.cpu().numpy()[pos], want, rtol=RTOL, atol=ATOL)
    # every one of the 117 M positions against the oracle's loop nest (OpenMP over rows) and, in
    # blocks of rows, against float64 dot products
    orc.use_all_cores()
    whole = orc.sddmm(a1, b, c.indptr, c.indices, c.m, c.n, feat, omp=True)
    got = o1.cpu().numpy()
    a64, b64 = a1.astype(np.float64), b.astype(np.float64)
    worst_gpu = worst_oracle = 0.0
    for r0 in range(0, c.m, 16384):
        r1 = min(c.m, r0 + 16384)
        p0, p1 = int(c.indptr[r0]), int(c.indptr[r1])
        rows_blk = np.repeat(np.arange(r0, r1), np.diff(c.indptr[r0:r1 + 1]))
        truth = np.einsum("ij,ij->i", a64[rows_blk], b64[c.indices[p0:p1]])
        eg, eo = parity(got[p0:p1], whole[p0:p1], truth, groups=rows_blk - r0)
        worst_gpu, worst_oracle = max(worst_gpu, eg), max(worst_oracle, eo)
    print(f"sddmm config 3 whole: max error vs float64: GPU {worst_gpu:.3e}, oracle {worst_oracle:.3e}")


def test_edge_to_row_bit_exact(cuda_device):
    g = np.load(os.path.join(GOLD, "edge_to_row.npz"))
    c = dg.csr_lognormal(n=5000, mu=2.0, sigma=1.5, max_deg=3000, seed=7)
    for ip in (g["indptr"], c.indptr):
        nnz = int(ip[-1])
        mid = torch.full((nnz,), -1, dtype=torch.int32, device=cuda_device)
        ops.sddmm_edge_to_row(dev(ip, cuda_device), mid)
        torch.cuda.synchronize()
        assert np.array_equal(mid.cpu().numpy(), orc.edge_to_row(ip, nnz))


# ------------------------------------------------------------------------------ bsrmm
def run_bsrmm(bs: dg.BSR, b: np.ndarray, device):
    feat = b.shape[1]
    c = torch.full((bs.mb * bs.blk * feat,), 3.0, device=device)
    ops.bsrmm(dev(bs.data.reshape(-1), device), dev(b.reshape(-1), device), c, dev(bs.indptr, device),
              dev(bs.indices, device), bs.mb, bs.nb, bs.nnzb, bs.blk, feat)
    torch.cuda.synchronize()
    return c


@pytest.mark.parametrize("size,blk,feat", [(512, 32, 128), (512, 32, 512), (256, 16, 64), (384, 32, 96),
                                           (96, 8, 40), (1024, 64, 256), (4096, 32, 512)])
def test_bsrmm_matches_oracle(cuda_device, size, blk, feat):
    bs = dg.bsr_mask(size=size, blk=blk, density=0.1, seed=size + feat)
    b = dg.dense_operand_normal(1, size, feat)
    want = orc.bsrmm_f16(bs.data, b, bs.indptr, bs.indices, bs.mb, bs.nb, blk, feat, omp=True)
    # fp16 inputs, fp32 accumulation: rtol 1e-2; sums of ~blk*deg products of N(0,1) values
    close(run_bsrmm(bs, b, cuda_device), want, rtol=1e-2, atol=1e-2)


def test_bsrmm_golden_and_empty_block_rows(cuda_device):
    g = np.load(os.path.join(GOLD, "bsrmm.npz"))
    bs = dg.BSR(len(g["indptr"]) - 1, g["b"].shape[0] // 32, 32, g["indptr"], g["indices"], g["data"])
    close(run_bsrmm(bs, g["b"], cuda_device), g["c"].astype(np.float32), rtol=1e-2, atol=1e-2)
    # block-rows 0 and 2 empty -> zeros
    ip = np.array([0, 0, 2, 2], np.int32)
    ix = np.array([0, 2], np.int32)
    rng = np.random.default_rng(0)
    data = rng.standard_normal((2, 32, 32)).astype(np.float16)
    bs = dg.BSR(3, 3, 32, ip, ix, data)
    b = dg.dense_operand_normal(2, 96, 64)
    got = run_bsrmm(bs, b, cuda_device)
    close(got, orc.bsrmm_f16(data, b, ip, ix, 3, 3, 32, 64), rtol=1e-2, atol=1e-2)
    assert torch.all(got.reshape(3, 32, 64)[[0, 2]] == 0)


# ------------------------------------------------------------------------------ rgms
def run_rgms(cf: dg.CSF, x, w, device, scalars=False):
    feat = x.shape[1]
    y = torch.zeros(cf.m * feat, device=device)
    args = [dev(cf.data, device), dev(w.reshape(-1), device), dev(x.reshape(-1), device), y,
            dev(cf.indptr_i, device), dev(cf.indices_i, device), dev(cf.indptr_j, device),
            dev(cf.indices_j, device)]
    if scalars:
        args += [cf.m, cf.n, cf.num_rels, feat, cf.nnz_i, cf.nnz_j]
    ops.rgms(*args)
    torch.cuda.synchronize()
    return y


def rgms_truth(cf: dg.CSF, x, w, data=None):
    return refimpl.rgms_f64(cf.data if data is None else data, w, x, cf.indptr_i, cf.indices_i,
                            cf.indptr_j, cf.indices_j, cf.m)


def oracle_rgms(cf: dg.CSF, x, w):
    y = np.zeros((cf.m, x.shape[1]), np.float32)
    return orc.rgms(cf.data, w, x, y, cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j, cf.m,
                    cf.n, cf.num_rels, x.shape[1], omp=True)


@pytest.mark.parametrize("feat", [8, 32, 64, 128, 48])
def test_rgms_matches_oracle(cuda_device, feat):
    cf = dg.csf_relational(n=3000, num_rels=11, num_edges=40000, seed=feat)
    x = dg.dense_operand(1, cf.n, feat)
    w = dg.relation_weights(2, cf.num_rels, feat)
    close(run_rgms(cf, x, w, cuda_device, scalars=feat == 64), oracle_rgms(cf, x, w))


def test_rgms_golden_many_relations_and_empty(cuda_device):
    g = np.load(os.path.join(GOLD, "rgms.npz"))
    cf = dg.CSF(g["y"].shape[0], g["x"].shape[0], len(g["indptr_i"]) - 1, g["indptr_i"], g["indices_i"],
                g["indptr_j"], g["indices_j"], g["data"])
    close(run_rgms(cf, g["x"], g["w"], cuda_device), g["y"].astype(np.float32))
    # more relations than threads in a block, most of them tiny or empty
    cf = dg.csf_relational(n=500, num_rels=300, num_edges=3000, zipf_a=2.5, seed=3)
    ip = cf.indptr_i.copy()
    x = dg.dense_operand(4, cf.n, 64)
    w = dg.relation_weights(5, cf.num_rels, 64)
    close(run_rgms(cf, x, w, cuda_device), oracle_rgms(cf, x, w))
    assert np.any(np.diff(ip) <= 1)


def test_rgms_larger_graph_eager_and_captured(cuda_device):
    # a few hundred tiles per block of the persistent kernel, and the same call captured into a
    # CUDA graph and replayed (the scratch buffer exists after the eager call)
    cf = dg.csf_relational(n=30000, num_rels=13, num_edges=260001, seed=21)
    assert cf.nnz_i >= 65536
    x = dg.dense_operand(22, cf.n, 64)
    w = dg.relation_weights(23, cf.num_rels, 64)
    want = oracle_rgms(cf, x, w)
    truth = rgms_truth(cf, x, w)
    parity(run_rgms(cf, x, w, cuda_device), want, truth)
    d = cuda_device
    y = torch.zeros(cf.m * 64, device=d)
    args = [dev(cf.data, d), dev(w.reshape(-1), d), dev(x.reshape(-1), d), y, dev(cf.indptr_i, d),
            dev(cf.indices_i, d), dev(cf.indptr_j, d), dev(cf.indices_j, d)]
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        ops.rgms(*args)  # warm-up on the capturing stream: its scratch buffer
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            y.zero_()
            ops.rgms(*args)
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    parity(y, want, truth)


def test_rgms_config5_full_size(cuda_device):
    # 100,000 nodes, 46 relations, 1.5 M edges, feat 64: the whole result at the stated tolerance
    # against the float64 result (the oracle's sequential fp32 sums are up to 9e-6 off it themselves)
    cf = dg.csf_relational(seed=0)
    x = dg.dense_operand(1, cf.n, 64)
    w = dg.relation_weights(2, cf.num_rels, 64)
    want = oracle_rgms(cf, x, w)
    got = run_rgms(cf, x, w, cuda_device)
    err_gpu, err_oracle = parity(got, want, rgms_truth(cf, x, w))
    print(f"rgms config 5: max error vs float64: GPU {err_gpu:.3e}, oracle {err_oracle:.3e}")
    assert err_gpu <= max(2 * err_oracle, 1e-5)


def test_rgms_one_launch_form_in_child_process(cuda_device, tmp_path):
    # SPARSETIR_RGMS_PATH=fused (read once per process): gather, 3xTF32 product and scatter in one
    # persistent launch without scratch memory.  Same parity bar; tiles with more entries than the
    # staging buffer holds (a relation whose rows have ~40 entries) and many tiny relations included.
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
            "import ctypes, numpy as np, torch, test_gpu_ops as T\n"
            "from sparsetir_b200 import _lib as L, datagen as dg\n"
            "d = torch.device('cuda', 0)\n"
            "for n, rels, edges, seed in ((3000, 11, 40000, 64), (300, 3, 30000, 12), (500, 300, 3000, 3), (30000, 13, 260001, 21)):\n"
            "    cf = dg.csf_relational(n=n, num_rels=rels, num_edges=edges, seed=seed)\n"
            "    x = dg.dense_operand(1, cf.n, 64); w = dg.relation_weights(2, cf.num_rels, 64)\n"
            "    T.parity(T.run_rgms(cf, x, w, d), T.oracle_rgms(cf, x, w), T.rgms_truth(cf, x, w))\n"
            "k = ctypes.c_uint(9); assert L.load().sparsetir_tc_timeouts(0, ctypes.byref(k)) == 0 and k.value == 0\n"
            "print('one launch ok')" % (root, os.path.join(root, "tests")))
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, SPARSETIR_RGMS_PATH="fused"),
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "one launch ok" in r.stdout, r.stdout + r.stderr


def test_rgms_accumulates_into_y(cuda_device):
    cf = dg.csf_relational(n=400, num_rels=4, num_edges=3000, seed=6)
    x = dg.dense_operand(7, cf.n, 64)
    w = dg.relation_weights(8, cf.num_rels, 64)
    want = oracle_rgms(cf, x, w)
    y = torch.ones(cf.m * 64, device=cuda_device)
    ops.rgms(dev(cf.data, cuda_device), dev(w.reshape(-1), cuda_device), dev(x.reshape(-1), cuda_device), y,
             dev(cf.indptr_i, cuda_device), dev(cf.indices_i, cuda_device), dev(cf.indptr_j, cuda_device),
             dev(cf.indices_j, cuda_device))
    close(y, want + 1.0)


# ------------------------------------------------------------------------------ rgms on ELL3D
def ell3d_buckets(cf: dg.CSF, cols_bkt, group=32):
    """Host buckets (a, rows, cols, mid) the way the reference example prepares them
    (examples/rgms/rgcn/bench_rgcn_composable.py:123-138, :196-208): mask as the weights."""
    rows_bkt = [max(1, group // c) for c in cols_bkt]
    ip, rows, cols, mask = fmt.csf_to_ell3d(cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j,
                                            rows_bkt, cols_bkt)
    out = []
    for b in range(len(cols_bkt)):
        mid = np.repeat(np.arange(cf.num_rels, dtype=np.int32), np.diff(ip[b]))
        out.append((mask[b].astype(np.float32), rows[b], cols[b], mid))
    return out


def run_rgms_ell3d(cf, x, w, buckets, device, feat):
    y = torch.zeros(cf.m * feat, device=device)
    devb = [tuple(dev(t, device) for t in bk) for bk in buckets]
    ops.rgms_ell3d(*ops.rgms_ell3d_args(dev(w, device), dev(x, device), y, devb, feat))
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize("feat", [16, 32, 64, 128])
def test_rgms_ell3d_matches_oracle_and_the_csf_form(cuda_device, feat):
    cf = dg.csf_relational(n=3000, num_rels=9, num_edges=50000, seed=feat)
    x = dg.dense_operand(1, cf.n, feat)
    w = dg.relation_weights(2, cf.num_rels, feat)
    buckets = ell3d_buckets(cf, [1, 2, 4, 8])
    want = orc.rgms_ell3d(w, x, np.zeros((cf.m, feat), np.float32), buckets, feat)
    got = run_rgms_ell3d(cf, x, w, buckets, cuda_device, feat)
    # the buckets carry the 0/1 mask: the float64 result is that of the CSF form with unit values
    truth = rgms_truth(cf, x, w, data=np.ones(cf.nnz_j, np.float32))
    parity(got, want, truth)
    # the same matrix in the CSF form with unit values gives the same Y
    ones = dg.CSF(cf.m, cf.n, cf.num_rels, cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j,
                  np.ones(cf.nnz_j, np.float32))
    parity(got, oracle_rgms(ones, x, w), truth)


def test_rgms_ell3d_wide_and_empty_buckets(cuda_device):
    # rows longer than the widest bucket are split; a bucket of 64 columns is accumulated
    # atomically; bucket 16 stays empty for this degree distribution of tiny relations
    cf = dg.csf_relational(n=300, num_rels=3, num_edges=30000, seed=12)  # ~33 entries per (rel, row)
    feat = 64
    x = dg.dense_operand(3, cf.n, feat)
    w = dg.relation_weights(4, cf.num_rels, feat)
    for cols_bkt in ([64], [1, 16, 64], [4]):
        buckets = ell3d_buckets(cf, cols_bkt, group=64)
        want = orc.rgms_ell3d(w, x, np.zeros((cf.m, feat), np.float32), buckets, feat)
        parity(run_rgms_ell3d(cf, x, w, buckets, cuda_device, feat), want,
               rgms_truth(cf, x, w, data=np.ones(cf.nnz_j, np.float32)))


# ------------------------------------------------------------------------------ rgms, fp16, rectangular
def run_rgms_ell3d_f16(cf, x16, w16, buckets, device, feat_in, feat_out, out_dtype):
    y = torch.zeros(cf.m * feat_out, device=device, dtype=out_dtype)
    devb = [(dev(a.astype(np.float16), device), dev(r, device), dev(c, device), dev(m, device))
            for a, r, c, m in buckets]
    ops.rgms_ell3d_f16(*ops.rgms_ell3d_f16_args(dev(w16, device), dev(x16, device), y, devb, feat_in, feat_out))
    torch.cuda.synchronize()
    return y.float()


def rect_weights(seed, num_rels, feat_in, feat_out):
    return (np.random.default_rng(seed).standard_normal((num_rels, feat_in, feat_out)) /
            np.sqrt(feat_in)).astype(np.float16)


@pytest.mark.parametrize("feat_in,feat_out", [(64, 64), (64, 128), (128, 64), (128, 256), (256, 128), (192, 192),
                                              (32, 64), (64, 32), (48, 80), (16, 8), (320, 64)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
def test_rgms_ell3d_f16_matches_oracle(cuda_device, feat_in, feat_out, out_dtype):
    cf = dg.csf_relational(n=2500, num_rels=7, num_edges=30000, seed=feat_in + feat_out)
    x16 = dg.dense_operand(1, cf.n, feat_in).astype(np.float16)
    w16 = rect_weights(2, cf.num_rels, feat_in, feat_out)
    buckets = ell3d_buckets(cf, [1, 2, 4, 8])
    want = orc.rgms_ell3d_f16(w16, x16, np.zeros((cf.m, feat_out), np.float32), buckets, feat_in, feat_out)
    got = run_rgms_ell3d_f16(cf, x16, w16, buckets, cuda_device, feat_in, feat_out, out_dtype)
    # fp16 operands, fp32 sums (the aggregated rows pass through fp16 once): rtol 1e-2; a float16
    # result also rounds every addition into Y
    close(got, want, rtol=1e-2, atol=2e-2 if out_dtype == torch.float32 else 6e-2)


@pytest.mark.parametrize("feat_in,feat_out,out_dtype", [(64, 128, torch.float32), (128, 64, torch.float16),
                                                        (256, 256, torch.float32), (64, 32, torch.float32)])
def test_rgms_ell3d_f16_sparse_convolution_shape(cuda_device, feat_in, feat_out, out_dtype):
    # what the sparse convolution driver builds: one relation per kernel offset (27), every
    # (input, output) pair its own ELL row (buckets = [1]), unit values.  Tensor-core shapes take
    # the one-launch form (X rows gathered inside the kernel), 64 -> 32 the row-scaling launch and
    # the CUDA-core transform.
    cf = dg.csf_relational(n=4000, num_rels=27, num_edges=60000, zipf_a=0.3, seed=5)
    x16 = dg.dense_operand(3, cf.n, feat_in).astype(np.float16)
    w16 = rect_weights(4, cf.num_rels, feat_in, feat_out)
    buckets = ell3d_buckets(cf, [1], group=1)
    assert all(c.shape[-1] == 1 for _, _, c, _ in buckets)
    # non-unit values too: the one-launch form applies them in the epilogue
    a, r, c, m = buckets[0]
    a = (a * np.random.default_rng(9).uniform(0.5, 1.5, size=a.shape)).astype(np.float16).astype(np.float32)
    buckets = [(a, r, c, m)]
    want = orc.rgms_ell3d_f16(w16, x16, np.zeros((cf.m, feat_out), np.float32), buckets, feat_in, feat_out)
    got = run_rgms_ell3d_f16(cf, x16, w16, buckets, cuda_device, feat_in, feat_out, out_dtype)
    close(got, want, rtol=1e-2, atol=2e-2 if out_dtype == torch.float32 else 6e-2)
    # the same as a dense computation: Y[o] = sum over (r, i -> o) of a X[i] W_r
    y = np.zeros((cf.m, feat_out), np.float64)
    xs, ws = x16.astype(np.float64), w16.astype(np.float64)
    av = a.reshape(-1).astype(np.float64)
    for rel in range(cf.num_rels):
        for t in range(cf.indptr_i[rel], cf.indptr_i[rel + 1]):
            sl = slice(cf.indptr_j[t], cf.indptr_j[t + 1])
            y[cf.indices_i[t]] += (av[sl, None] * xs[cf.indices_j[sl]]).sum(0) @ ws[rel]
    close(got, y.astype(np.float32), rtol=1e-2, atol=2e-2 if out_dtype == torch.float32 else 6e-2)


@pytest.mark.parametrize("feat_in,feat_out,out_dtype,n_out", [(64, 128, torch.float32, 5000), (128, 64, torch.float16, 3001),
                                                              (64, 64, torch.float32, 130), (256, 256, torch.float16, 2048)])
def test_rgms_ell3d_f16_sparse_convolution_maps_without_repeats(cuda_device, feat_in, feat_out, out_dtype, n_out):
    # neighbour maps in which a (kernel offset, output) pair never repeats and all values are 1:
    # the destination-stationary form (no reductions into Y); Y already holds values
    cf = dg.sparse_conv_pairs(n_in=4000, n_out=n_out, num_offsets=27, fill=0.6, seed=feat_in + n_out)
    x16 = dg.dense_operand(3, cf.n, feat_in).astype(np.float16)
    w16 = rect_weights(4, cf.num_rels, feat_in, feat_out)
    buckets = ell3d_buckets(cf, [1], group=1)
    y0 = np.random.default_rng(1).uniform(-1, 1, size=(cf.m, feat_out)).astype(np.float16).astype(np.float32)
    want = orc.rgms_ell3d_f16(w16, x16, y0.copy(), buckets, feat_in, feat_out)
    y = dev(y0.reshape(-1), cuda_device).to(out_dtype)
    devb = [(dev(a.astype(np.float16), cuda_device), dev(r, cuda_device), dev(c, cuda_device), dev(m, cuda_device))
            for a, r, c, m in buckets]
    ops.rgms_ell3d_f16(*ops.rgms_ell3d_f16_args(dev(w16, cuda_device), dev(x16, cuda_device), y, devb, feat_in, feat_out))
    torch.cuda.synchronize()
    close(y.float(), want, rtol=1e-2, atol=2e-2 if out_dtype == torch.float32 else 6e-2)
    # one repeated pair, or one value that is not 0 / 1, sends the same call to the form with reductions
    a, r, c, m = buckets[0]
    r2 = r.copy()
    r2[1] = r2[0]  # rows 0 and 1 of relation 0 now share their destination
    a3 = a.copy()
    a3[2] = 0.5
    for bk in ([(a, r2, c, m)], [(a3, r, c, m)]):
        want2 = orc.rgms_ell3d_f16(w16, x16, np.zeros((cf.m, feat_out), np.float32), bk, feat_in, feat_out)
        got2 = run_rgms_ell3d_f16(cf, x16, w16, bk, cuda_device, feat_in, feat_out, out_dtype)
        close(got2, want2, rtol=1e-2, atol=2e-2 if out_dtype == torch.float32 else 6e-2)


def test_rgms_ell3d_f16_reduction_free_form_forced_in_child_process(cuda_device, tmp_path):
    # by default only feat_in = 64 with a float32 Y takes the destination-stationary form; the
    # switch (read once per process) sends every eligible shape through it
    import subprocess
    import sys
    cf = dg.sparse_conv_pairs(n_in=3000, n_out=2500, num_offsets=27, fill=0.6, seed=77)
    buckets = ell3d_buckets(cf, [1], group=1)
    a, r, c, m = buckets[0]
    cases = {}
    for name, (fi, fo, dt) in {"h": (128, 64, "float16"), "w": (256, 256, "float32"), "s": (64, 192, "float16")}.items():
        x16 = dg.dense_operand(3, cf.n, fi).astype(np.float16)
        w16 = rect_weights(4, cf.num_rels, fi, fo)
        want = orc.rgms_ell3d_f16(w16, x16, np.zeros((cf.m, fo), np.float32), buckets, fi, fo)
        cases.update({f"x_{name}": x16, f"w_{name}": w16, f"want_{name}": want,
                      f"meta_{name}": np.array([fi, fo, 1 if dt == "float16" else 0])})
    case = str(tmp_path / "case.npz")
    np.savez(case, a=a.astype(np.float16), r=r, c=c, m=m, **cases)
    code = ("import numpy as np, torch, sys; sys.path.insert(0, %r); from sparsetir_b200 import ops\n"
            "z = np.load(%r); d = torch.device('cuda', 0)\n"
            "t = lambda v: torch.from_numpy(np.ascontiguousarray(v)).to(d)\n"
            "bk = [(t(z['a']), t(z['r']), t(z['c']), t(z['m']))]\n"
            "for n in 'hws':\n"
            "    fi, fo, half = (int(v) for v in z['meta_' + n])\n"
            "    y = torch.zeros(z['want_' + n].size, device=d, dtype=torch.float16 if half else torch.float32)\n"
            "    ops.rgms_ell3d_f16(*ops.rgms_ell3d_f16_args(t(z['w_' + n]), t(z['x_' + n]), y, bk, fi, fo))\n"
            "    torch.cuda.synchronize()\n"
            "    np.testing.assert_allclose(y.float().cpu().numpy().reshape(z['want_' + n].shape), z['want_' + n], rtol=1e-2, atol=6e-2 if half else 2e-2)\n"
            "print('reduction-free ok')" % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), case))
    res = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, SPARSETIR_RGMS_F16_PATH="os"),
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "reduction-free ok" in res.stdout, res.stdout + res.stderr


def test_rgms_ell3d_f16_empty_buckets_and_accumulation(cuda_device):
    cf = dg.csf_relational(n=300, num_rels=3, num_edges=4000, seed=8)
    feat_in, feat_out = 64, 64
    x16 = dg.dense_operand(5, cf.n, feat_in).astype(np.float16)
    w16 = rect_weights(6, cf.num_rels, feat_in, feat_out)
    buckets = ell3d_buckets(cf, [1, 16, 64], group=64)  # bucket 16 or 64 may stay empty
    want = orc.rgms_ell3d_f16(w16, x16, np.ones((cf.m, feat_out), np.float32), buckets, feat_in, feat_out)
    y = torch.ones(cf.m * feat_out, device=cuda_device)
    devb = [(dev(a.astype(np.float16), cuda_device), dev(r, cuda_device), dev(c, cuda_device), dev(m, cuda_device))
            for a, r, c, m in buckets]
    ops.rgms_ell3d_f16(*ops.rgms_ell3d_f16_args(dev(w16, cuda_device), dev(x16, cuda_device), y, devb, feat_in, feat_out))
    torch.cuda.synchronize()
    close(y, want, rtol=1e-2, atol=3e-2)
    # no buckets at all: nothing happens
    y0 = torch.full((cf.m * feat_out,), 2.0, device=cuda_device)
    ops.rgms_ell3d_f16(dev(w16.reshape(-1), cuda_device), dev(x16.reshape(-1), cuda_device), y0, feat_in, feat_out)
    torch.cuda.synchronize()
    assert torch.all(y0 == 2.0)


# ------------------------------------------------------------------------------ tcspmm
def run_tcspmm(g: dg.CSR, x16, t, gs, device, out_dtype, weights=None):
    """Condense the graph on the host (ConDense), then the condensed SpMM on the GPU."""
    gi, ti, mk = fmt.condense(g.indptr, g.indices, t, gs)
    a16 = mk.astype(np.float16) if weights is None else weights(mk)
    mb, nb, feat = len(gi) - 1, -(-g.n // gs), x16.shape[1]
    xb = np.zeros((nb * gs, feat), np.float16)
    xb[:g.n] = x16
    c = torch.full((mb * t * feat,), 3.0, device=device, dtype=out_dtype)
    ops.tcspmm(dev(a16.reshape(-1), device), dev(xb.reshape(-1), device), c, dev(gi, device),
               dev(ti.reshape(-1), device), mb, nb, len(ti), feat, t, gs)
    torch.cuda.synchronize()
    want = orc.tcspmm_f16(a16, xb, gi, ti.reshape(-1), mb, t, gs, feat)
    return c.float().cpu().numpy().reshape(mb * t, feat), want


@pytest.mark.parametrize("t,gs,feat", [(16, 16, 128), (8, 16, 128), (32, 16, 256), (16, 16, 512),
                                       (16, 16, 96), (16, 8, 128), (4, 16, 64)])
def test_tcspmm_matches_oracle(cuda_device, t, gs, feat):
    g = dg.csr_powerlaw(n=3000, max_deg=1500, seed=t + feat)
    x16 = dg.dense_operand(1, g.n, feat).astype(np.float16)
    got, want = run_tcspmm(g, x16, t, gs, cuda_device, torch.float32)
    np.testing.assert_allclose(got, want, rtol=1e-2, atol=1e-2)
    # unit weights: the condensed product is the plain SpMM of the 0/1 matrix
    ones = np.zeros((g.m, feat), np.float32)
    orc.csrmm(np.ones(g.nnz, np.float32), x16.astype(np.float32), ones, g.indptr, g.indices, g.m, g.n, feat)
    np.testing.assert_allclose(got[:g.m], ones, rtol=1e-2, atol=1e-2)


def test_tcspmm_half_output_weights_and_empty_tiles(cuda_device):
    # the reference's output dtype (float16), non-unit weights, and row tiles without any entry
    deg = np.zeros(640, np.int64)
    deg[:200] = np.random.default_rng(2).integers(1, 40, size=200)
    deg[600:] = 3
    rng = np.random.default_rng(3)
    ix = dg.sorted_distinct_columns(rng, deg, 640)
    g = dg.CSR(640, 640, np.concatenate([[0], np.cumsum(deg)]).astype(np.int32), ix, np.ones(len(ix), np.float32))
    x16 = dg.dense_operand(4, g.n, 128).astype(np.float16)
    wts = lambda mk: (mk * np.random.default_rng(5).uniform(0.5, 1.5, size=mk.shape)).astype(np.float16)  # noqa: E731
    got, want = run_tcspmm(g, x16, 16, 16, cuda_device, torch.float16, weights=wts)
    np.testing.assert_allclose(got, want, rtol=1e-2, atol=3e-2)  # one rounding to half on top
    assert np.all(got[16 * 13:16 * 37] == 0)  # tiles 13..36 have no entries


# ------------------------------------------------------------------ reduce / softmax / csr2bsr / ellmm
@pytest.mark.parametrize("gen", ["short", "long"])
def test_csr_reduce_and_sparse_softmax(cuda_device, gen):
    c = (dg.csr_powerlaw(n=5000, max_deg=3000, seed=2) if gen == "short"
         else dg.csr_lognormal(n=800, mu=4.5, sigma=0.8, max_deg=700, seed=3))
    a = (dg.dense_operand(1, c.nnz, 1).reshape(-1) * 4).astype(np.float32)
    ip, ix = dev(c.indptr, cuda_device), dev(c.indices, cuda_device)
    b = torch.full((c.m,), 9.0, device=cuda_device)
    ops.csr_reduce(dev(a, cuda_device), b, ip, ix, c.m, c.n, c.nnz)   # csr_reduce signature
    b2 = torch.full((c.m,), 9.0, device=cuda_device)
    ops.csr_reduce(dev(a, cuda_device), b2, ip)                        # segment_reduce, sizes inferred
    torch.cuda.synchronize()
    want = orc.csr_reduce(a, c.indptr)
    truth = refimpl.row_sums_f64(a, c.indptr)
    parity(b, want, truth)
    parity(b2, want, truth)
    sm = torch.full((c.nnz,), -1.0, device=cuda_device)
    ops.sparse_softmax(dev(a, cuda_device), sm, ip, ix)
    torch.cuda.synchronize()
    close(sm, orc.sparse_softmax(a, c.indptr), rtol=1e-4, atol=1e-6)


def test_csr2bsr_bit_exact(cuda_device):
    c = dg.csr_powerlaw(n=1000, max_deg=400, seed=6)
    for blk in (4, 32):
        rows = np.repeat(np.arange(c.m), np.diff(c.indptr))
        mb, nbk = -(-c.m // blk), -(-c.n // blk)
        pattern = np.zeros((mb, nbk), bool)
        pattern[rows // blk, c.indices // blk] = True
        pattern[np.arange(mb), np.arange(mb) % nbk] = True  # blocks that receive nothing stay as they are
        ip_out = np.concatenate([[0], np.cumsum(pattern.sum(1))]).astype(np.int32)
        ix_out = np.nonzero(pattern)[1].astype(np.int32)
        b = torch.full((len(ix_out) * blk * blk,), -2.0, device=cuda_device)
        ops.csr2bsr(dev(c.data, cuda_device), b, dev(c.indptr, cuda_device), dev(c.indices, cuda_device),
                    dev(ip_out, cuda_device), dev(ix_out, cuda_device), c.m, c.n, mb, nbk, c.nnz, len(ix_out), blk)
        torch.cuda.synchronize()
        want = orc.csr2bsr(c.data, np.full((len(ix_out), blk, blk), -2.0, np.float32), c.indptr, c.indices,
                           ip_out, ix_out, blk)
        assert np.array_equal(b.cpu().numpy().reshape(want.shape), want)


@pytest.mark.parametrize("nb,mb,col,blk,feat", [(40, 50, 3, 16, 128), (9, 9, 5, 32, 96), (17, 30, 1, 4, 200),
                                                (6, 6, 0, 8, 32)])
def test_ellmm_matches_oracle(cuda_device, nb, mb, col, blk, feat):
    rng = np.random.default_rng(nb + feat)
    a = rng.standard_normal((nb, col, blk, blk)).astype(np.float32)
    ix = rng.integers(0, mb, size=(nb, col)).astype(np.int32)
    b = rng.standard_normal((mb * blk, feat)).astype(np.float32)
    c = torch.full((nb * blk * feat,), 5.0, device=cuda_device)
    ops.ellmm(dev(a.reshape(-1), cuda_device), dev(b.reshape(-1), cuda_device), c, dev(ix.reshape(-1), cuda_device),
              nb, mb, feat, col, blk)
    torch.cuda.synchronize()
    parity(c, orc.ellmm(a, b, ix, nb, col, blk, feat), refimpl.ellmm_f64(a, b, ix, nb, col, blk, feat))


# ------------------------------------------------------------------------------ fusedmm
@pytest.mark.parametrize("feat", [16, 32, 64, 128, 256, 512, 24])
def test_fusedmm_matches_oracle(cuda_device, feat, tmp_path):
    c = dg.csr_lognormal(n=1500, mu=3.0, sigma=1.2, max_deg=1200, seed=feat)
    deg = np.diff(c.indptr)
    scale = 1.0 / np.sqrt(feat)
    q = (dg.dense_operand(1, c.m, feat) * scale * 2).astype(np.float32)
    k = dg.dense_operand(2, c.n, feat)
    v = dg.dense_operand(3, c.n, feat)
    o = torch.full((c.m * feat,), 7.0, device=cuda_device)
    ops.fusedmm(dev(q.reshape(-1), cuda_device), dev(k.reshape(-1), cuda_device), dev(v.reshape(-1), cuda_device),
                o, dev(c.indptr, cuda_device), dev(c.indices, cuda_device))
    torch.cuda.synchronize()
    want = orc.fusedmm(q, k, v, c.indptr, c.indices, c.m, feat)
    parity(o, want, refimpl.fusedmm_f64(q, k, v, c.indptr, c.indices))
    assert deg.max() > 64
    if feat in (32, 64, 128, 256):  # the one-pass kernel for the same call (the switch is read per process)
        import subprocess
        import sys
        case = str(tmp_path / "case.npz")
        truth = refimpl.fusedmm_f64(q, k, v, c.indptr, c.indices)
        np.savez(case, q=q, k=k, v=v, indptr=c.indptr, indices=c.indices, want=want, truth=truth)
        code = ("import numpy as np, torch, sys; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
                "from sparsetir_b200 import ops; import test_gpu_ops as T\n"
                "z = np.load(%r); d = torch.device('cuda', 0)\n"
                "t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(d)\n"
                "o = torch.zeros(z['want'].size, device=d)\n"
                "ops.fusedmm(t(z['q'].reshape(-1)), t(z['k'].reshape(-1)), t(z['v'].reshape(-1)), o, t(z['indptr']), t(z['indices']))\n"
                "torch.cuda.synchronize()\n"
                "T.parity(o, z['want'], z['truth'])\n"
                "print('one-pass ok')" % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                          os.path.dirname(os.path.abspath(__file__)), case))
        r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, SPARSETIR_FUSEDMM_PATH="fused"),
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0 and "one-pass ok" in r.stdout, r.stdout + r.stderr


def test_fusedmm_empty_rows_and_scalars(cuda_device):
    deg = np.zeros(300, np.int64)
    deg[[3, 4, 100, 299]] = [2, 70, 1, 33]
    rng = np.random.default_rng(1)
    ix = dg.sorted_distinct_columns(rng, deg, 300)
    ip = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    feat = 64
    q, k, v = (dg.dense_operand(s, 300, feat) * 0.3 for s in (4, 5, 6))
    o = torch.full((300 * feat,), 7.0, device=cuda_device)
    ops.fusedmm(dev(q.reshape(-1), cuda_device), dev(k.reshape(-1), cuda_device), dev(v.reshape(-1), cuda_device),
                o, dev(ip, cuda_device), dev(ix, cuda_device), 300, 300, len(ix), feat)
    torch.cuda.synchronize()
    want = orc.fusedmm(q, k, v, ip, ix, 300, feat)
    parity(o, want, refimpl.fusedmm_f64(q, k, v, ip, ix))
    assert np.all(want[0] == 0) and torch.all(o.view(300, feat)[0] == 0)


# ------------------------------------------------------------------------------ streams
def test_calls_run_on_the_current_torch_stream(cuda_device):
    c = dg.csr_poisson(m=2000, n=2000, mean_deg=10, seed=30)
    x = dg.dense_operand(31, c.n, 64)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        got = run_csrmm(c, x, cuda_device)
        assert L.load().sparsetir_get_stream(0) == s.cuda_stream
    close(got, oracle_csrmm(c, x))


def test_two_host_threads_keep_their_own_streams(cuda_device):
    # the stream of a packed call belongs to the calling thread (the reference keeps it in its
    # thread-local CUDAThreadEntry): two threads on one device, each inside its own torch stream
    import threading
    c = dg.csr_poisson(m=3000, n=3000, mean_deg=12, seed=40)
    want = {}
    xs = {}
    for k in (0, 1):
        xs[k] = dg.dense_operand(41 + k, c.n, 64)
        want[k] = oracle_csrmm(c, xs[k])
    lib = L.load()
    streams = {k: torch.cuda.Stream() for k in (0, 1)}
    seen, got, errors = {}, {}, []
    gate = threading.Barrier(2)

    def work(k):
        try:
            torch.cuda.set_device(cuda_device)
            with torch.cuda.stream(streams[k]):
                a, x = dev(c.data, cuda_device), dev(xs[k].reshape(-1), cuda_device)
                ip, ix = dev(c.indptr, cuda_device), dev(c.indices, cuda_device)
                y = torch.zeros(c.m * 64, device=cuda_device)
                call = ops.csrmm.prepare(a, x, y, ip, ix)
                for _ in range(20):
                    gate.wait()
                    call()   # sets this thread's stream, then launches on it
                    assert lib.sparsetir_get_stream(0) == streams[k].cuda_stream
                seen[k] = lib.sparsetir_get_stream(0)
                streams[k].synchronize()
                got[k] = y
        except Exception as e:  # surfaced by the main thread
            errors.append(repr(e))
            gate.abort()

    threads = [threading.Thread(target=work, args=(k,)) for k in (0, 1)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert seen[0] == streams[0].cuda_stream and seen[1] == streams[1].cuda_stream and seen[0] != seen[1]
    for k in (0, 1):
        close(got[k], want[k])
    # a thread that never set a stream uses the process-wide default
    holder = []
    t = threading.Thread(target=lambda: holder.append(lib.sparsetir_get_stream(0)))
    t.start()
    t.join()
    assert holder[0] in (None, 0)
    assert lib.sparsetir_set_default_stream(0, ctypes.c_void_p(streams[0].cuda_stream)) == 0
    t = threading.Thread(target=lambda: holder.append(lib.sparsetir_get_stream(0)))
    t.start()
    t.join()
    assert holder[1] == streams[0].cuda_stream
    assert lib.sparsetir_set_default_stream(0, None) == 0


def test_reserved_workspace_lets_the_first_call_be_captured(cuda_device):
    # hyb SpMM with split rows needs scratch rows and counters; reserved up front for a fresh
    # stream, the very first call on that stream can be captured into a CUDA graph (an allocation
    # inside the capture would fail it)
    c = dg.csr_powerlaw(n=5000, max_deg=3000, seed=50)
    x = dg.dense_operand(51, c.n, 128)
    host, devb = hyb_device_buckets(c, 1, [1, 2, 4, 8, 16, 32], cuda_device)
    want = oracle_hyb(host, x, c.m)
    arr = (L.EllBucket * len(devb))()
    for k, (w, r, cc) in enumerate(devb):
        arr[k] = L.EllBucket(w.data_ptr(), r.data_ptr(), cc.data_ptr(), r.numel(), cc.numel() // max(1, r.numel()))
    sb, cb = ctypes.c_size_t(0), ctypes.c_size_t(0)
    lib = L.load()
    assert lib.sparsetir_hyb_spmm_workspace(arr, len(devb), 128, ctypes.byref(sb), ctypes.byref(cb)) == 0
    assert sb.value > 0 and cb.value > 0
    s = torch.cuda.Stream()
    assert lib.sparsetir_reserve_workspace(0, ctypes.c_void_p(s.cuda_stream), sb.value, cb.value) == 0, L.last_error()
    xd = dev(x, cuda_device)
    y = torch.zeros(c.m * 128, device=cuda_device)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            ops.hyb_spmm(*ops.hyb_args(xd, y, devb, 128))
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    close(y, want)
    assert torch.cuda.mem_get_info()[0] >= free_before - (8 << 20)  # the graph itself, nothing else


def test_validate_mode_refuses_bad_indices(cuda_device):
    # SPARSETIR_VALIDATE / sparsetir_set_validate: index arrays are checked on the device before
    # the operator runs; a bad one makes the call fail with a message instead of a wild access
    lib = L.load()
    c = dg.csr_poisson(m=500, n=400, mean_deg=6, seed=60)
    x = dg.dense_operand(61, c.n, 32)
    d = cuda_device
    assert lib.sparsetir_set_validate(1) == 0
    try:
        close(run_csrmm(c, x, d), oracle_csrmm(c, x))      # good input passes
        bad_ix = c.indices.copy()
        bad_ix[17] = c.n                                     # one column past the end
        y = torch.zeros(c.m * 32, device=d)
        with pytest.raises(ops.SparseTIRError, match=r"indices\[17\] = 400 is out of range"):
            ops.csrmm(dev(c.data, d), dev(x.reshape(-1), d), y, dev(c.indptr, d), dev(bad_ix, d))
        bad_ip = c.indptr.copy()
        bad_ip[100] = bad_ip[101] + 1                        # decreasing row pointer
        with pytest.raises(ops.SparseTIRError, match="indptr decreases at position 101"):
            ops.csrmm(dev(c.data, d), dev(x.reshape(-1), d), y, dev(bad_ip, d), dev(c.indices, d))
        out = torch.zeros(c.nnz, device=d)
        a = dg.dense_operand(62, c.m, 32)
        with pytest.raises(ops.SparseTIRError, match="out of range"):
            ops.sddmm(dev(a.reshape(-1), d), dev(x.reshape(-1), d), out, dev(c.indptr, d), dev(bad_ix, d))
        # hyb: a row id beyond m
        host, devb = hyb_device_buckets(c, 1, [1, 2, 4, 8], d)
        w, r, cc = devb[-1]
        r2 = r.clone()
        r2[0] = c.m + 5
        with pytest.raises(ops.SparseTIRError, match="row_indices"):
            ops.hyb_spmm(*ops.hyb_args(dev(x, d), y, devb[:-1] + [(w, r2, cc)], 32))
        # RGMS: a destination row beyond m
        cf = dg.csf_relational(n=300, num_rels=4, num_edges=2000, seed=63)
        xi = dg.dense_operand(64, cf.n, 64)
        wi = dg.relation_weights(65, cf.num_rels, 64)
        bad_i = cf.indices_i.copy()
        bad_i[-1] = cf.m
        yy = torch.zeros(cf.m * 64, device=d)
        with pytest.raises(ops.SparseTIRError, match=r"indices_i"):
            ops.rgms(dev(cf.data, d), dev(wi.reshape(-1), d), dev(xi.reshape(-1), d), yy, dev(cf.indptr_i, d),
                     dev(bad_i, d), dev(cf.indptr_j, d), dev(cf.indices_j, d))
        # the context is still usable
        close(run_csrmm(c, x, d), oracle_csrmm(c, x))
    finally:
        lib.sparsetir_set_validate(0)


def test_tensor_core_waits_never_ran_out(cuda_device):
    """Runs after the BSR / RGMS tests above: no bounded barrier wait of the tensor-core kernels
    may have hit its limit."""
    import ctypes
    n = ctypes.c_uint(123)
    assert L.load().sparsetir_tc_timeouts(0, ctypes.byref(n)) == 0, L.last_error()
    assert n.value == 0


# ------------------------------------------------------------------ 32-byte-lane SpMM variants
_WIDE_LANE_CHILD = r"""
import sys
import numpy as np, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
from oracle import oracle as orc
from sparsetir_b200 import datagen as dg, format as fmt, ops
d = torch.device("cuda", 0)
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(d)
g = dg.csr_powerlaw(n=3000, max_deg=1500, seed=4)
for feat in (32, 64, 128, 512):
    x = dg.dense_operand(9, g.n, feat)
    want = np.zeros((g.m, feat), np.float32)
    orc.csrmm(g.data, x, want, g.indptr, g.indices, g.m, g.n, feat)
    y = torch.full((g.m * feat,), 5.0, device=d)
    ops.csrmm(dev(g.data), dev(x.reshape(-1)), y, dev(g.indptr), dev(g.indices))
    torch.cuda.synchronize()
    np.testing.assert_allclose(y.cpu().numpy().reshape(g.m, feat), want, rtol=1e-4, atol=1e-5)
    bk = [1, 2, 4, 8, 16]
    rows, cols, mask, vals, pos = fmt.column_part_hyb(g.m, g.n, g.indptr, g.indices, 1, bk, data=g.data)
    devb = [(dev(vals[0][k]), dev(rows[0][k]), dev(cols[0][k])) for k in range(len(bk))]
    y2 = torch.zeros(g.m * feat, device=d)
    ops.hyb_spmm(*ops.hyb_args(dev(x), y2, devb, feat))
    torch.cuda.synchronize()
    np.testing.assert_allclose(y2.cpu().numpy().reshape(g.m, feat), want, rtol=1e-4, atol=1e-5)
print("wide lanes ok")
"""


def test_spmm_32_byte_lane_variants_in_child_process(cuda_device):
    # SPARSETIR_LANE_FLOATS is read once per process, so the variants run in a child
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, SPARSETIR_LANE_FLOATS="8")
    code = _WIDE_LANE_CHILD.format(root=root, tests=os.path.join(root, "tests"))
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "wide lanes ok" in r.stdout, r.stdout + r.stderr


def test_csrmm_hub_rows_take_the_long_row_launches(cuda_device):
    # a matrix large enough for the hub-row path, with rows far beyond the 2048-entry threshold
    # next to short and empty ones
    deg = np.random.default_rng(4).integers(0, 6, size=9000).astype(np.int64)
    deg[[0, 4000, 4001, 8999]] = [5000, 2049, 2048, 7001]
    rng = np.random.default_rng(5)
    ix = dg.sorted_distinct_columns(rng, deg, 9000)
    c = dg.CSR(9000, 9000, np.concatenate([[0], np.cumsum(deg)]).astype(np.int32), ix,
               rng.uniform(-1, 1, size=len(ix)).astype(np.float32))
    for feat in (32, 128, 512):
        x = dg.dense_operand(feat, c.n, feat)
        parity(run_csrmm(c, x, cuda_device), oracle_csrmm(c, x),
               refimpl.spmm_f64(c.indptr, c.indices, c.data, x, c.m, c.n))
