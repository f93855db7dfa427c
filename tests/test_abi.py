"""The C-ABI library loads, exports every symbol the header declares, and validates packed
arguments like the host stub the reference generates.  No device work happens here: every call
below is rejected during argument checking, before any CUDA call."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from sparsetir_b200 import _lib as L
from sparsetir_b200 import ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "sparsetir_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"SPARSETIR_API\s+[^;(]*?\b(sparsetir_\w+)\s*\(", text)
    assert len(names) >= 25
    return names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(L.LIB_PATH)
    for name in header_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_declarations_cover_the_header():
    declared = set(L.PACKED_SYMBOLS) | set(L.PLAIN_SYMBOLS)
    assert declared == set(header_symbols())
    lib = L.load()
    assert lib.sparsetir_version() >= 100 and lib.sparsetir_sm_arch() == 100


def test_header_compiles_as_c():
    import subprocess
    import tempfile

    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.c")
        open(src, "w").write('#include "sparsetir_b200.h"\nint main(void){return sizeof(TVMValue)==8?0:1;}\n')
        subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                        src, "-o", os.path.join(d, "t")], check=True)
        subprocess.run([os.path.join(d, "t")], check=True)


def test_struct_layouts_match_dlpack_and_tvm():
    assert ctypes.sizeof(L.TVMValue) == 8
    assert ctypes.sizeof(L.DLTensor) == 48
    assert L.DLTensor.shape.offset == 24 and L.DLTensor.byte_offset.offset == 40
    assert ctypes.sizeof(L.EllBucket) == 32


def test_stream_registry_roundtrip():
    lib = L.load()
    assert lib.sparsetir_set_stream(3, ctypes.c_void_p(0x1230)) == 0
    assert lib.sparsetir_get_stream(3) == 0x1230
    assert lib.sparsetir_set_stream(3, None) == 0
    assert lib.sparsetir_get_stream(3) in (None, 0)
    assert lib.sparsetir_set_stream(1000, None) == -1
    assert "out of range" in L.last_error()


def _cpu(n, dtype=torch.float32):
    return torch.zeros(n, dtype=dtype)


def test_cpu_tensors_are_rejected_no_fallback():
    with pytest.raises(ops.SparseTIRError, match="no CPU path"):
        ops.csrmm(_cpu(3), _cpu(8), _cpu(8), _cpu(3, torch.int32), _cpu(3, torch.int32))


@pytest.mark.parametrize("fn,nargs", [(ops.csrmm, 4), (ops.sddmm, 7), (ops.bsrmm, 5), (ops.rgms, 9),
                                      (ops.sddmm_edge_to_row, 1)])
def test_wrong_argument_count(fn, nargs):
    with pytest.raises(ops.SparseTIRError, match="num_args"):
        fn(*[_cpu(2) for _ in range(nargs)])


def _fake_cuda(n, code, bits, ndim=1, strides=None, byte_offset=0, device_id=0):
    """A DLTensor that claims to live on a CUDA device; argument checking never dereferences it."""
    keep = (ctypes.c_int64 * ndim)(*([n] + [1] * (ndim - 1)))
    t = L.DLTensor(data=ctypes.c_void_p(0x1000), device=L.DLDevice(L.kDLCUDA, device_id), ndim=ndim,
                   dtype=L.DLDataType(code, bits, 1),
                   shape=ctypes.cast(keep, ctypes.POINTER(ctypes.c_int64)),
                   strides=None, byte_offset=byte_offset)
    t._keep = keep
    if strides is not None:
        s = (ctypes.c_int64 * ndim)(*strides)
        t.strides = ctypes.cast(s, ctypes.POINTER(ctypes.c_int64))
        t._keep2 = s
    return t


def f32(n, **kw):
    return _fake_cuda(n, L.kDLFloat, 32, **kw)


def i32(n, **kw):
    return _fake_cuda(n, L.kDLInt, 32, **kw)


def test_csrmm_validation_messages():
    good = lambda: [f32(5), f32(4 * 8), f32(3 * 8), i32(4), i32(5)]  # noqa: E731
    a = good(); a[0] = _fake_cuda(5, L.kDLFloat, 64)
    with pytest.raises(ops.SparseTIRError, match="a.dtype is expected to be float32"):
        ops.csrmm(*a)
    a = good(); a[3] = _fake_cuda(4, L.kDLInt, 64)
    with pytest.raises(ops.SparseTIRError, match="indptr.dtype is expected to be int32"):
        ops.csrmm(*a)
    a = good(); a[1] = f32(32, ndim=2)
    with pytest.raises(ops.SparseTIRError, match="b.ndim is expected to equal 1"):
        ops.csrmm(*a)
    a = good(); a[2] = f32(24, strides=[2])
    with pytest.raises(ops.SparseTIRError, match="compact"):
        ops.csrmm(*a)
    a = good(); a[2] = f32(24, byte_offset=16)
    with pytest.raises(ops.SparseTIRError, match="byte_offset"):
        ops.csrmm(*a)
    a = good(); a[4] = i32(5, device_id=1)
    with pytest.raises(ops.SparseTIRError, match="device_id"):
        ops.csrmm(*a)
    a = good(); a[4] = i32(6)
    with pytest.raises(ops.SparseTIRError, match="indices.shape"):
        ops.csrmm(*a)
    with pytest.raises(ops.SparseTIRError, match="unsatisfied constraint"):
        ops.csrmm(*good(), 3, 4, 8, 6)
    with pytest.raises(ops.SparseTIRError, match="to be int"):
        ops.csrmm(*good(), 3, 4, 8.0, 5)
    with pytest.raises(ops.SparseTIRError, match="to be pointer"):
        ops.csrmm(1, *good()[1:])
    with pytest.raises(ops.SparseTIRError, match="null handle"):
        ops.csrmm(None, *good()[1:])


def test_hyb_validation_messages():
    with pytest.raises(ops.SparseTIRError, match="tensor arguments"):
        ops.hyb_spmm(f32(8), f32(8), f32(4), i32(4), 4)
    with pytest.raises(ops.SparseTIRError, match="scalar arguments"):
        ops.hyb_spmm(f32(8), f32(8), f32(4), i32(4), i32(4))
    with pytest.raises(ops.SparseTIRError, match="multiple of len\\(rows\\)"):
        ops.hyb_spmm(f32(8), f32(8), f32(5), i32(2), i32(5), 4)
    with pytest.raises(ops.SparseTIRError, match="w.shape"):
        ops.hyb_spmm(f32(8), f32(8), f32(3), i32(2), i32(4), 4)
    with pytest.raises(ops.SparseTIRError, match="multiples of feat_size"):
        ops.hyb_spmm(f32(9), f32(8), f32(4), i32(2), i32(4), 4)
    many = [f32(8), f32(8)] + [f32(4), i32(4), i32(4)] * (L.HYB_MAX_BUCKETS + 1)
    with pytest.raises(ops.SparseTIRError, match="exceed the maximum"):
        ops.hyb_spmm(*many, 4)


def test_other_ops_validation_messages():
    with pytest.raises(ops.SparseTIRError, match="scale.shape"):
        ops.sddmm(f32(3 * 8), f32(4 * 8), f32(5), i32(4), i32(5), f32(6))
    with pytest.raises(ops.SparseTIRError, match="a.dtype is expected to be float16"):
        ops.bsrmm(f32(4), f32(4), f32(4), i32(2), i32(1), 1, 1, 1, 2, 1)
    with pytest.raises(ops.SparseTIRError, match="not num_rels \\* feat_size\\^2"):
        ops.rgms(f32(3), f32(2 * 10), f32(8), f32(8), i32(3), i32(2), i32(3), i32(3))
    with pytest.raises(ops.SparseTIRError, match="indptr_j.shape"):
        ops.rgms(f32(3), f32(2 * 16), f32(8), f32(8), i32(3), i32(2), i32(4), i32(3))


def f16(n, **kw):
    return _fake_cuda(n, L.kDLFloat, 16, **kw)


def test_later_operators_validation_messages():
    # condensed SpMM: lengths must match the scalars; the output may be float16 or float32
    with pytest.raises(ops.SparseTIRError, match="num_args should be 11"):
        ops.tcspmm(f16(4), f16(4), f16(4), i32(2), i32(4))
    with pytest.raises(ops.SparseTIRError, match="a.shape"):
        ops.tcspmm(f16(5), f16(16 * 8), f16(16 * 8), i32(2), i32(16), 1, 1, 1, 8, 16, 16)
    with pytest.raises(ops.SparseTIRError, match="c.dtype is expected to be float16"):
        ops.tcspmm(f16(256), f16(16 * 8), _fake_cuda(16 * 8, L.kDLFloat, 64), i32(2), i32(16), 1, 1, 1, 8, 16, 16)
    # ELL3D RGMS: (w, x, y) + 4 tensors per bucket + feat_size
    with pytest.raises(ops.SparseTIRError, match="expected \\(w, x, y"):
        ops.rgms_ell3d(f32(16), f32(8), f32(8), f32(4), i32(2), 4)
    with pytest.raises(ops.SparseTIRError, match="do not describe groups x rows x columns"):
        ops.rgms_ell3d(f32(16), f32(8), f32(8), f32(6), i32(3), i32(6), i32(2), 4)
    # fp16 RGMS with rectangular weights: two trailing scalars, float16 operands, y float16 or float32
    with pytest.raises(ops.SparseTIRError, match="expected \\(w, x, y"):
        ops.rgms_ell3d_f16(f16(16), f16(8), f32(8), f16(4), i32(4), i32(4), i32(2), 4)
    with pytest.raises(ops.SparseTIRError, match="w.dtype is expected to be float16"):
        ops.rgms_ell3d_f16(f32(16), f16(8), f32(8), 4, 4)
    with pytest.raises(ops.SparseTIRError, match="must be multiples of feat_in\\*feat_out"):
        ops.rgms_ell3d_f16(f16(17), f16(8), f32(8), 4, 4)
    with pytest.raises(ops.SparseTIRError, match="do not describe groups x rows x columns"):
        ops.rgms_ell3d_f16(f16(32), f16(8), f16(16), f16(6), i32(3), i32(6), i32(2), 4, 8)
    # the small row-wise operators
    with pytest.raises(ops.SparseTIRError, match="indptr.shape"):
        ops.csr_reduce(f32(5), f32(3), i32(5))
    with pytest.raises(ops.SparseTIRError, match="b.shape"):
        ops.sparse_softmax(f32(5), f32(4), i32(4), i32(5))
    with pytest.raises(ops.SparseTIRError, match="blk_size must be positive"):
        ops.csr2bsr(f32(5), f32(4), i32(4), i32(5), i32(2), i32(1), 0)
    with pytest.raises(ops.SparseTIRError, match="fewer block rows"):
        ops.csr2bsr(f32(5), f32(4), i32(10), i32(5), i32(2), i32(1), 2)
    with pytest.raises(ops.SparseTIRError, match="indices.shape"):
        ops.ellmm(f32(2 * 3 * 16), f32(5 * 4 * 8), f32(2 * 4 * 8), i32(5), 2, 5, 8, 3, 4)
