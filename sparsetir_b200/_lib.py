"""Loads ``libsparsetir_b200.so`` and declares the C ABI of ``include/sparsetir_b200.h``.

There is no fallback of any kind: if the shared library is missing, or a symbol the header
declares is not exported, importing the operators fails with an error that says so.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# SPARSETIR_B200_LIBRARY names another build of the same library (kernel experiments)
LIB_PATH = os.environ.get("SPARSETIR_B200_LIBRARY") or os.path.join(_PKG, "libsparsetir_b200.so")

# ---- ctypes mirrors of the structs in include/sparsetir_b200.h ---------------------------------


class DLDevice(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int32), ("device_id", ctypes.c_int32)]


class DLDataType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class DLTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("device", DLDevice),
        ("ndim", ctypes.c_int32),
        ("dtype", DLDataType),
        ("shape", ctypes.POINTER(ctypes.c_int64)),
        ("strides", ctypes.POINTER(ctypes.c_int64)),
        ("byte_offset", ctypes.c_uint64),
    ]


class TVMValue(ctypes.Union):
    _fields_ = [
        ("v_int64", ctypes.c_int64),
        ("v_float64", ctypes.c_double),
        ("v_handle", ctypes.c_void_p),
        ("v_str", ctypes.c_char_p),
        ("v_type", DLDataType),
        ("v_device", DLDevice),
    ]


class EllBucket(ctypes.Structure):
    _fields_ = [
        ("w", ctypes.c_void_p),
        ("rows", ctypes.c_void_p),
        ("cols", ctypes.c_void_p),
        ("nrows", ctypes.c_int32),
        ("width", ctypes.c_int32),
    ]


kDLCPU, kDLCUDA, kDLCUDAHost = 1, 2, 3
kDLInt, kDLUInt, kDLFloat = 0, 1, 2
kTVMArgInt, kTVMArgFloat, kTVMOpaqueHandle, kTVMNullptr = 0, 2, 3, 4
kTVMDLTensorHandle, kTVMNDArrayHandle = 7, 13

HYB_ZERO_C, HYB_REARM, HYB_ALL_ATOMIC = 1, 2, 4
HYB_MAX_BUCKETS = 64

PACKED_SYMBOLS = (
    "sparsetir_csrmm",
    "sparsetir_hyb_spmm",
    "sparsetir_hyb_spmm_peers",
    "sparsetir_sddmm",
    "sparsetir_sddmm_peers",
    "sparsetir_sddmm_edge_to_row",
    "sparsetir_bsrmm",
    "sparsetir_rgms",
    "sparsetir_rgms_ell3d",
    "sparsetir_rgms_ell3d_f16",
    "sparsetir_tcspmm",
    "sparsetir_csr_reduce",
    "sparsetir_sparse_softmax",
    "sparsetir_csr2bsr",
    "sparsetir_ellmm",
    "sparsetir_fusedmm",
)

# every other exported symbol: name -> (restype, argtypes)
_vp, _i, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)
_f32p = ctypes.POINTER(ctypes.c_float)
PLAIN_SYMBOLS = {
    "sparsetir_get_last_error": (ctypes.c_char_p, []),
    "sparsetir_set_stream": (_i, [_i, _vp]),
    "sparsetir_set_default_stream": (_i, [_i, _vp]),
    "sparsetir_get_stream": (_vp, [_i]),
    "sparsetir_reserve_workspace": (_i, [_i, _vp, ctypes.c_size_t, ctypes.c_size_t]),
    "sparsetir_hyb_spmm_tile": (_i, [_i, _i, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]),
    "sparsetir_hyb_spmm_workspace": (_i, [ctypes.POINTER(EllBucket), _i, _i,
                                          ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]),
    "sparsetir_set_validate": (_i, [_i]),
    "sparsetir_peer_scatter": (_i, [_i, _vp, _vp, ctypes.c_size_t, _i, ctypes.POINTER(ctypes.c_void_p)]),
    "sparsetir_version": (_i, []),
    "sparsetir_sm_arch": (_i, []),
    "sparsetir_tc_timeouts": (_i, [_i, ctypes.POINTER(ctypes.c_uint)]),
    "sparsetir_csrmm_raw": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "sparsetir_hyb_spmm_raw": (_i, [_vp, _vp, ctypes.POINTER(EllBucket), _i, _i, _i, _i, _i, _i, _vp]),
    "sparsetir_hyb_spmm_peers_raw": (_i, [_vp, _vp, ctypes.POINTER(EllBucket), _i, _i, _i, _i, _i, _i,
                                          ctypes.POINTER(ctypes.c_void_p), _i, _vp]),
    "sparsetir_sddmm_raw": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "sparsetir_sddmm_peers_raw": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                                       ctypes.POINTER(ctypes.c_void_p), _i, _vp]),
    "sparsetir_sddmm_edge_to_row_raw": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "sparsetir_bsrmm_raw": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "sparsetir_rgms_raw": (_i, [_vp] * 8 + [_i] * 7 + [_vp]),
    "sparsetir_rgms_workspace": (_i, [_i, _i, ctypes.POINTER(ctypes.c_size_t)]),
    "sparsetir_csr_reduce_raw": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "sparsetir_sparse_softmax_raw": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "sparsetir_csr2bsr_raw": (_i, [_vp] * 6 + [_i, _i, _i, _i, _vp]),
    "sparsetir_ellmm_raw": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "sparsetir_fusedmm_raw": (_i, [_vp] * 6 + [_i, _i, _i, _i, _i, _vp]),
    "sparsetir_tcspmm_raw": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "sparsetir_rgms_ell3d_raw": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "sparsetir_rgms_ell3d_f16_raw": (_i, [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "sparsetir_rgms_noalloc": (_i, [_vp] * 8 + [_i] * 7 + [_vp]),
    "sparsetir_column_part_hyb": (_vp, [_i, _i, _i32p, _i32p, _i, _i32p, _i, _i]),
    "sparsetir_hyb_num_rows": (_i64, [_vp, _i, _i]),
    "sparsetir_hyb_copy_bucket": (_i, [_vp, _i, _i, _i32p, _i32p, _i32p, _i32p, _f32p, _f32p]),
    "sparsetir_hyb_free": (None, [_vp]),
    "sparsetir_condense": (_i64, [_i, _i32p, _i32p, _i, _i, _i32p, _i32p, _i32p]),
    "sparsetir_csf_to_ell3d": (_vp, [_i, _i32p, _i32p, _i32p, _i32p, _i32p, _i32p, _i]),
    "sparsetir_ell3d_num_groups": (_i64, [_vp, _i]),
    "sparsetir_ell3d_copy_bucket": (_i, [_vp, _i, _i32p, _i32p, _i32p, _i32p]),
    "sparsetir_ell3d_free": (None, [_vp]),
    "sparsetir_row_partition": (_i, [_i, _i32p, _i, _i64p]),
}

PACKED_ARGTYPES = [ctypes.POINTER(TVMValue), ctypes.POINTER(ctypes.c_int), ctypes.c_int,
                   ctypes.POINTER(TVMValue), ctypes.POINTER(ctypes.c_int), ctypes.c_void_p]

_lib = None


class LibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """The loaded library; raises LibraryError when it is absent or incomplete."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryError(
            f"{LIB_PATH} is missing: build it with `python -m sparsetir_b200.build` "
            "(this package has no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name in PACKED_SYMBOLS:
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise LibraryError(f"{LIB_PATH} does not export {name}") from e
        fn.restype = ctypes.c_int
        fn.argtypes = PACKED_ARGTYPES
    for name, (res, args) in PLAIN_SYMBOLS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise LibraryError(f"{LIB_PATH} does not export {name}") from e
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    msg = load().sparsetir_get_last_error()
    return msg.decode("utf-8", "replace") if msg else ""
