"""The allocation-free RGMS entry point (collected last on purpose: a failure here must not
hide the result of any other test when the suite stops at the first failure).

``sparsetir_rgms_noalloc`` serves callers that may not touch the CUDA allocator when they run the
operator; it keeps its intermediate in an array built into the library.  It must give the same
result as the regular ``sparsetir_rgms`` — on the first call and on a second call that finds the
previous call's data still in the shared array — and both must match the CPU oracle at the
stated tolerance."""
import ctypes

import numpy as np
import pytest
import torch

import refimpl
import test_gpu_ops as T
from sparsetir_b200 import _lib as L
from sparsetir_b200 import datagen as dg
from sparsetir_b200 import ops

pytestmark = pytest.mark.gpu

# fp32 bar of this operator (the tensor-core path carries ~21 mantissa bits; sums are re-associated)
RTOL, ATOL = 1e-4, 1e-5


def _dev(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def _run_noalloc(cf, x, w, device):
    t = [_dev(v, device) for v in (cf.data, w.reshape(-1), x.reshape(-1))]
    idx = [_dev(v, device) for v in (cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j)]
    y = torch.zeros(cf.m * 64, device=device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.load().sparsetir_rgms_noalloc(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), y.data_ptr(),
                                         idx[0].data_ptr(), idx[1].data_ptr(), idx[2].data_ptr(),
                                         idx[3].data_ptr(), cf.m, cf.n, cf.num_rels, 64, cf.nnz_i,
                                         cf.nnz_j, 0, stream)
    assert rc == 0, L.last_error()
    torch.cuda.synchronize()
    return y


def _run_regular(cf, x, w, device):
    y = torch.zeros(cf.m * 64, device=device)
    ops.rgms(_dev(cf.data, device), _dev(w.reshape(-1), device), _dev(x.reshape(-1), device), y,
             _dev(cf.indptr_i, device), _dev(cf.indices_i, device), _dev(cf.indptr_j, device),
             _dev(cf.indices_j, device))
    torch.cuda.synchronize()
    return y


def test_noalloc_matches_regular_entry_point_twice(cuda_device):
    # two different problems back to back: the second one is smaller, so stale rows of the first
    # stay in the shared array beyond its range and must not leak into the result
    for seed, n, edges in ((1, 5000, 60000), (2, 1500, 9000)):
        cf = dg.csf_relational(n=n, num_rels=7, num_edges=edges, seed=seed)
        x = dg.dense_operand(seed + 10, cf.n, 64)
        w = dg.relation_weights(seed + 20, cf.num_rels, 64)
        got = _run_noalloc(cf, x, w, cuda_device).cpu().numpy()
        want = _run_regular(cf, x, w, cuda_device).cpu().numpy()
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
        # and against the oracle (reference summation order) and the float64 result
        T.parity(got, T.oracle_rgms(cf, x, w), T.rgms_truth(cf, x, w), rtol=RTOL, atol=ATOL)


def test_noalloc_second_call_takes_no_device_memory(cuda_device):
    # the array came into being with the first call on this device (above, or here); a later call
    # leaves the amount of free device memory where it was
    cf = dg.csf_relational(n=1500, num_rels=7, num_edges=9000, seed=2)
    x = dg.dense_operand(12, cf.n, 64)
    w = dg.relation_weights(22, cf.num_rels, 64)
    _run_noalloc(cf, x, w, cuda_device)
    t = [_dev(v, cuda_device) for v in (cf.data, w.reshape(-1), x.reshape(-1))]
    idx = [_dev(v, cuda_device) for v in (cf.indptr_i, cf.indices_i, cf.indptr_j, cf.indices_j)]
    y = torch.zeros(cf.m * 64, device=cuda_device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = L.load().sparsetir_rgms_noalloc(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), y.data_ptr(),
                                         idx[0].data_ptr(), idx[1].data_ptr(), idx[2].data_ptr(),
                                         idx[3].data_ptr(), cf.m, cf.n, cf.num_rels, 64, cf.nnz_i,
                                         cf.nnz_j, 0, stream)
    assert rc == 0, L.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before


def test_noalloc_refuses_what_does_not_fit(cuda_device):
    lib = L.load()
    z = ctypes.c_void_p(0)
    rc = lib.sparsetir_rgms_noalloc(z, z, z, z, z, z, z, z, 10, 10, 1, 32, 5, 5, 0, None)
    assert rc == -1 and "feat_size must be 64" in L.last_error()
    rc = lib.sparsetir_rgms_noalloc(z, z, z, z, z, z, z, z, 10, 10, 1, 64, 131073, 5, 0, None)
    assert rc == -1 and "exceeds the built-in scratch" in L.last_error()
