"""Python host side of the operator boundary.

``PackedFunc`` mirrors how a built SparseTIR operator is called in the reference
(``f(*args)`` on a ``tvm.runtime.Module``, python/tvm/runtime/module.py:239; timing with
``f.time_evaluator``, src/runtime/profiling.cc:742-795): positional DLTensor / integer
arguments in the reference's order, outputs written in place, asynchronous on the current
stream, a raised error when the callee returns -1.  Tensors are ``torch.Tensor`` objects on a
CUDA device; torch is used only for device memory and streams.

The module-level callables ``csrmm``, ``hyb_spmm``, ``sddmm``, ``sddmm_edge_to_row``, ``bsrmm``
and ``rgms`` are the packed entry points of ``include/sparsetir_b200.h``.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import _lib as L


class SparseTIRError(RuntimeError):
    """Raised when an entry point returns -1 (the counterpart of tvm.TVMError)."""


_DTYPES = {
    torch.float32: (L.kDLFloat, 32),
    torch.float16: (L.kDLFloat, 16),
    torch.float64: (L.kDLFloat, 64),
    torch.int32: (L.kDLInt, 32),
    torch.int64: (L.kDLInt, 64),
    torch.uint8: (L.kDLUInt, 8),
}


def to_dltensor(t: torch.Tensor, keepalive: List) -> L.DLTensor:
    """Borrowed DLTensor view of a torch tensor (no copy)."""
    if t.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {t.dtype}")
    code, bits = _DTYPES[t.dtype]
    shape = (ctypes.c_int64 * max(1, t.dim()))(*t.shape)
    strides = None
    if not t.is_contiguous():
        strides = (ctypes.c_int64 * max(1, t.dim()))(*t.stride())
    keepalive.extend([shape, strides, t])
    if t.is_cuda:
        dev = L.DLDevice(L.kDLCUDA, t.device.index if t.device.index is not None else
                         torch.cuda.current_device())
    else:
        dev = L.DLDevice(L.kDLCPU, 0)
    return L.DLTensor(
        data=ctypes.c_void_p(t.data_ptr() if t.numel() > 0 else 0),
        device=dev, ndim=t.dim(), dtype=L.DLDataType(code, bits, 1),
        shape=ctypes.cast(shape, ctypes.POINTER(ctypes.c_int64)),
        strides=ctypes.cast(strides, ctypes.POINTER(ctypes.c_int64)) if strides is not None else None,
        byte_offset=0)


def use_current_stream(device: Optional[torch.device] = None) -> None:
    """Registers torch's current stream of ``device`` as the library's stream for it."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    rc = L.load().sparsetir_set_stream(idx, ctypes.c_void_p(torch.cuda.current_stream(idx).cuda_stream))
    if rc != 0:
        raise SparseTIRError(L.last_error())


class PreparedCall:
    """One packed call with its argument arrays already built (see PackedFunc.prepare)."""

    __slots__ = ("_fn", "_values", "_codes", "_n", "_keep", "_dev_index", "_ret", "_ret_code",
                 "_set_stream")

    def __init__(self, fn, values, codes, n, keep, device):
        self._fn, self._values, self._codes, self._n, self._keep = fn, values, codes, n, keep
        self._dev_index = None
        if device is not None:
            self._dev_index = device.index if device.index is not None else torch.cuda.current_device()
        self._ret = L.TVMValue()
        self._ret_code = ctypes.c_int(0)
        self._set_stream = L.load().sparsetir_set_stream

    def __call__(self) -> None:
        if self._dev_index is not None:
            self._set_stream(self._dev_index,
                             ctypes.c_void_p(torch.cuda.current_stream(self._dev_index).cuda_stream))
        rc = self._fn(self._values, self._codes, self._n, ctypes.byref(self._ret),
                      ctypes.byref(self._ret_code), None)
        if rc != 0:
            raise SparseTIRError(L.last_error())


class PackedFunc:
    """A TVMBackendPackedCFunc symbol of the library, callable like the reference's functions."""

    def __init__(self, symbol: str):
        self.symbol = symbol
        self._fn = None

    @property
    def entry_name(self) -> str:
        return self.symbol

    def _resolve(self):
        if self._fn is None:
            self._fn = getattr(L.load(), self.symbol)
        return self._fn

    def __call__(self, *args) -> None:
        self.prepare(*args)()

    def prepare(self, *args) -> "PreparedCall":
        """Packs the arguments once; the returned object repeats the call without rebuilding
        the DLTensor descriptors (the tensors must stay alive and keep their storage)."""
        fn = self._resolve()
        n = len(args)
        values = (L.TVMValue * max(1, n))()
        codes = (ctypes.c_int * max(1, n))()
        keep: List = []
        device = None
        for i, a in enumerate(args):
            if isinstance(a, torch.Tensor):
                dl = to_dltensor(a, keep)
                keep.append(dl)
                values[i].v_handle = ctypes.cast(ctypes.pointer(dl), ctypes.c_void_p)
                codes[i] = L.kTVMDLTensorHandle
                if a.is_cuda and device is None:
                    device = a.device
            elif isinstance(a, L.DLTensor):
                keep.append(a)
                values[i].v_handle = ctypes.cast(ctypes.pointer(a), ctypes.c_void_p)
                codes[i] = L.kTVMDLTensorHandle
            elif isinstance(a, bool) or isinstance(a, int):
                values[i].v_int64 = int(a)
                codes[i] = L.kTVMArgInt
            elif isinstance(a, float):
                values[i].v_float64 = a
                codes[i] = L.kTVMArgFloat
            elif a is None:
                values[i].v_handle = None
                codes[i] = L.kTVMNullptr
            else:
                raise TypeError(f"argument {i}: unsupported type {type(a)}")
        return PreparedCall(fn, values, codes, n, keep, device)

    def time_evaluator(self, number: int = 10, repeat: int = 1):
        """Mirror of the reference's time_evaluator: one untimed call, then ``repeat`` measurements
        of ``number`` back-to-back calls between two device events; returns a callable that
        gives the list of per-call mean seconds."""

        def run(*args) -> List[float]:
            call = self.prepare(*args)
            call()
            out = []
            for _ in range(repeat):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(number):
                    call()
                e1.record()
                e1.synchronize()
                out.append(e0.elapsed_time(e1) * 1e-3 / number)
            return out

        return run


csrmm = PackedFunc("sparsetir_csrmm")
hyb_spmm = PackedFunc("sparsetir_hyb_spmm")
hyb_spmm_peers = PackedFunc("sparsetir_hyb_spmm_peers")
sddmm = PackedFunc("sparsetir_sddmm")
sddmm_peers = PackedFunc("sparsetir_sddmm_peers")
sddmm_edge_to_row = PackedFunc("sparsetir_sddmm_edge_to_row")
bsrmm = PackedFunc("sparsetir_bsrmm")
rgms = PackedFunc("sparsetir_rgms")
rgms_ell3d = PackedFunc("sparsetir_rgms_ell3d")
rgms_ell3d_f16 = PackedFunc("sparsetir_rgms_ell3d_f16")
tcspmm = PackedFunc("sparsetir_tcspmm")
csr_reduce = PackedFunc("sparsetir_csr_reduce")
sparse_softmax = PackedFunc("sparsetir_sparse_softmax")
csr2bsr = PackedFunc("sparsetir_csr2bsr")
ellmm = PackedFunc("sparsetir_ellmm")
fusedmm = PackedFunc("sparsetir_fusedmm")


def hyb_args(x: torch.Tensor, y: torch.Tensor, buckets: Sequence[Sequence[torch.Tensor]],
             feat_size: int, flags: int = 0, peer_c: Optional[Sequence[int]] = None) -> list:
    """Argument list of ``hyb_spmm`` in the reference's layout
    (examples/spmm/bench_spmm.py:207-222): ``[b, c] + [w, rows, cols] per bucket`` followed by
    the scalars this library needs because it is not specialised at build time.  With ``peer_c``
    (addresses of the peers' copies of ``y``) the list is that of ``hyb_spmm_peers``."""
    args = [x.reshape(-1), y.reshape(-1)]
    for w, rows, cols in buckets:
        args += [w.reshape(-1), rows.reshape(-1), cols.reshape(-1)]
    args.append(int(feat_size))
    if flags or peer_c is not None:
        args.append(int(flags))
    if peer_c is not None:
        args += [int(a) for a in peer_c]
    return args


def rgms_ell3d_args(w: torch.Tensor, x: torch.Tensor, y: torch.Tensor,
                    buckets: Sequence[Sequence[torch.Tensor]], feat_size: int) -> list:
    """Argument list of ``rgms_ell3d`` in the reference's layout
    (examples/rgms/rgcn/bench_rgcn_composable.py:196-208): ``[w, x, y]``, then ``a, rows, cols`` per
    bucket, then ``mid`` per bucket, then ``feat_size``.  ``buckets`` holds ``(a, rows, cols, mid)``."""
    args = [w.reshape(-1), x.reshape(-1), y.reshape(-1)]
    for a, rows, cols, _ in buckets:
        args += [a.reshape(-1), rows.reshape(-1), cols.reshape(-1)]
    args += [mid.reshape(-1) for _, _, _, mid in buckets]
    args.append(int(feat_size))
    return args


def rgms_ell3d_f16_args(w: torch.Tensor, x: torch.Tensor, y: torch.Tensor,
                        buckets: Sequence[Sequence[torch.Tensor]], feat_in: int, feat_out: int) -> list:
    """Argument list of ``rgms_ell3d_f16`` in the reference's layout
    (examples/rgms/rgcn/bench_rgcn_tensorcore.py:842-852): ``[w, x, y]``, then ``a, rows, cols`` per
    bucket, then ``mid`` per bucket, then the two feature sizes.  ``buckets`` holds
    ``(a, rows, cols, mid)`` with ``a`` in float16."""
    args = [w.reshape(-1), x.reshape(-1), y.reshape(-1)]
    for a, rows, cols, _ in buckets:
        args += [a.reshape(-1), rows.reshape(-1), cols.reshape(-1)]
    args += [mid.reshape(-1) for _, _, _, mid in buckets]
    args += [int(feat_in), int(feat_out)]
    return args
