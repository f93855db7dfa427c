"""Sparse convolution through the RGMS operator: the caller side of
examples/rgms/sparse_conv/sparse_conv.py:93-125 of the reference.

A sparse (submanifold / strided / transposed) convolution layer arrives the way torchsparse
hands it over: ``inputs [n_in, feat_in]``, ``weights [K, feat_in, feat_out]`` (one matrix per
kernel offset), ``nbmaps [pairs, 2]`` listing (input point, output point) pairs grouped by kernel
offset, ``nbsizes [K]`` the number of pairs of every offset, and ``transposed`` (the maps of a
transposed convolution are stored the other way round).  The layer computes

    y[o] = sum over offsets k, pairs (i, o) of offset k:  x[i] @ weights[k]

The reference turns the maps into a heterogeneous graph with one relation per kernel offset
(sparse_conv.py:93-104), that graph into a 3-level CSF tensor in which EVERY output point is a
level-0 row of EVERY relation (examples/rgms/sparse_conv/rgms.py:677-692), the CSF tensor into
ELL3D buckets with ``buckets = [1]`` and groups of ``ty * 16 = 128`` rows (rgms.py:701-710), and
calls the tensor-core RGMS function with ``W`` as ``[K, feat_in, feat_out]`` (the two
``transpose(-1, -2)`` of sparse_conv.py:113 and rgms.py:842 cancel).  The same steps here, with the
library's ``csf_to_ell3d`` and ``sparsetir_rgms_ell3d_f16``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import format as fmt
from . import ops


def relations_from_maps(nbmaps, nbsizes, transposed: bool) -> List[Tuple[np.ndarray, np.ndarray]]:
    """(sources, destinations) of every kernel offset, as sparse_conv.py:96-103 slices them:
    offset ``rel`` owns ``nbsizes[rel]`` consecutive rows of ``nbmaps``; column 0 is the input
    point and column 1 the output point, swapped for a transposed convolution."""
    maps = np.asarray(nbmaps.cpu() if isinstance(nbmaps, torch.Tensor) else nbmaps)
    sizes = [int(s) for s in (nbsizes.tolist() if hasattr(nbsizes, "tolist") else nbsizes)]
    if maps.ndim != 2 or maps.shape[1] != 2:
        raise ValueError("nbmaps must have shape [pairs, 2]")
    if sum(sizes) > maps.shape[0]:
        raise ValueError("nbsizes counts more pairs than nbmaps holds")
    out, offset = [], 0
    for size in sizes:
        i = maps[offset:offset + size, 0]
        o = maps[offset:offset + size, 1]
        offset += size
        if transposed:
            i, o = o, i
        out.append((np.asarray(i, np.int64), np.asarray(o, np.int64)))
    return out


def csf_from_relations(rels: Sequence[Tuple[np.ndarray, np.ndarray]], num_dst: int):
    """The CSF arrays rgms.py:677-697 builds from the graph: per relation the CSC of its
    (destination x source) adjacency over ALL ``num_dst`` destinations, so
    ``indptr_0 = [0, m, 2m, ...]`` and ``indices_0 = arange(m)`` repeated; level 1 lists the
    sources of every destination (pairs of one destination keep their order in the maps)."""
    m = int(num_dst)
    indptr_0 = (np.arange(len(rels) + 1, dtype=np.int64) * m)
    indices_0 = np.tile(np.arange(m, dtype=np.int32), len(rels))
    ptr_parts, idx_parts, base = [np.zeros(1, np.int64)], [], 0
    for src, dst in rels:
        order = np.argsort(dst, kind="stable")
        counts = np.bincount(dst, minlength=m)
        if len(counts) > m:
            raise ValueError("an output index exceeds the number of output points")
        ptr_parts.append(base + np.cumsum(counts))
        idx_parts.append(src[order].astype(np.int32))
        base += len(src)
    indptr_1 = np.concatenate(ptr_parts)
    indices_1 = np.concatenate(idx_parts) if idx_parts else np.zeros(0, np.int32)
    if indptr_0[-1] > np.iinfo(np.int32).max or base > np.iinfo(np.int32).max:
        raise ValueError("the layer is too large for 32-bit indices")
    return indptr_0.astype(np.int32), indices_0, indptr_1.astype(np.int32), indices_1


def ell3d_from_maps(nbmaps, nbsizes, transposed: bool, num_inputs: int,
                    num_outputs: Optional[int] = None, group_size: int = 128,
                    buckets: Sequence[int] = (1,)):
    """Host side of the conversion: ``(buckets, num_outputs, num_pairs)`` with one
    ``(a float16, rows, cols, mid)`` tuple of numpy arrays per ELL3D bucket — the arrays the
    reference passes to the built function (rgms.py:846-855): the 0/1 mask as values, the row and
    column ids of CSFToELL3D, and the relation of every group."""
    rels = relations_from_maps(nbmaps, nbsizes, bool(transposed))
    top_dst = max((int(d.max()) for _, d in rels if len(d)), default=-1)
    top_src = max((int(s.max()) for s, _ in rels if len(s)), default=-1)
    m = int(num_outputs) if num_outputs is not None else top_dst + 1
    if top_dst >= m or top_src >= int(num_inputs):
        raise ValueError("nbmaps names a point beyond the given number of points")
    if any(len(d) and (int(d.min()) < 0 or int(s.min()) < 0) for s, d in rels):
        raise ValueError("nbmaps holds a negative index")
    buckets = [int(b) for b in buckets]
    ip0, ix0, ip1, ix1 = csf_from_relations(rels, m)
    indptr, rows, cols, mask = fmt.csf_to_ell3d(ip0, ix0, ip1, ix1,
                                                [group_size // b for b in buckets], buckets)
    out = []
    for b in range(len(buckets)):
        mid = np.repeat(np.arange(len(rels), dtype=np.int32), np.diff(indptr[b]))
        out.append((mask[b].astype(np.float16), rows[b], cols[b], mid))
    return out, m, int(sum(len(s) for s, _ in rels))


class SparseConvPlan:
    """The structure of one layer, converted once (host side) and kept on the device.

    ``plan(inputs, weights)`` then runs the operator; the maps of a layer do not change between
    calls, so the host conversion is not part of the steady state (the reference also converts
    before it times, rgms.py:677-710 against :861-864)."""

    def __init__(self, nbmaps, nbsizes, transposed: bool, num_inputs: int,
                 num_outputs: Optional[int] = None, device: Optional[torch.device] = None,
                 group_size: int = 128, buckets: Sequence[int] = (1,)):
        host, self.num_outputs, self.num_pairs = ell3d_from_maps(
            nbmaps, nbsizes, transposed, num_inputs, num_outputs, group_size, buckets)
        self.num_inputs = int(num_inputs)
        self.num_offsets = len(nbsizes)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.buckets = [tuple(torch.from_numpy(np.ascontiguousarray(a)).to(self.device) for a in bk)
                        for bk in host]

    def __call__(self, inputs: torch.Tensor, weights: torch.Tensor,
                 out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
        if inputs.dim() != 2 or weights.dim() != 3:
            raise ValueError("inputs must be [n_in, feat_in] and weights [K, feat_in, feat_out]")
        if inputs.shape[0] != self.num_inputs or weights.shape[0] != self.num_offsets:
            raise ValueError("inputs / weights do not match the layer this plan was made for")
        feat_in, feat_out = int(weights.shape[1]), int(weights.shape[2])
        if inputs.shape[1] != feat_in:
            raise ValueError("inputs and weights disagree on feat_in")
        x = inputs.to(self.device, torch.float16).contiguous()
        w = weights.to(self.device, torch.float16).contiguous()
        if out is None:
            out = torch.zeros(self.num_outputs, feat_out, dtype=out_dtype, device=self.device)
        elif tuple(out.shape) != (self.num_outputs, feat_out) or not out.is_contiguous():
            raise ValueError("out must be a contiguous [num_outputs, feat_out] tensor (it is added to)")
        ops.rgms_ell3d_f16(*ops.rgms_ell3d_f16_args(w, x, out, self.buckets, feat_in, feat_out))
        return out


def sparse_conv(inputs: torch.Tensor, weights: torch.Tensor, nbmaps, nbsizes, transposed: bool = False,
                num_outputs: Optional[int] = None, out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """One call with the reference driver's inputs (sparse_conv.py:52-61): ``y [n_out, feat_out]``,
    float16 like the reference's output unless ``out_dtype`` says float32."""
    plan = SparseConvPlan(nbmaps, nbsizes, transposed, int(inputs.shape[0]), num_outputs,
                          device=inputs.device if inputs.is_cuda else None)
    return plan(inputs, weights, out_dtype=out_dtype)
