"""Multi-GPU layer: row sharding of the sparse operand across the GPUs of one box.

The reference is single-GPU; this layer is new.  Every operator of the path is independent per
output row, so the matrix is cut into contiguous row blocks with balanced numbers of stored
entries (``sparsetir_row_partition``, host C++), one block per rank, one rank per GPU.  Each rank
decomposes and multiplies its own block; the dense operand is replicated.  The only collectives
are a broadcast of the dense operand and an all-gather of the (unequal) output row blocks, both
through ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).  No kernel reads another
GPU's memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from . import format as fmt


@dataclass
class RowShard:
    """Rows [row0, row1) of a CSR matrix with its own zero-based indptr."""
    rank: int
    world: int
    row0: int
    row1: int
    num_cols: int
    indptr: np.ndarray   # int32 [row1 - row0 + 1]
    indices: np.ndarray  # int32 [nnz of the shard]
    data: Optional[np.ndarray]
    cuts: np.ndarray     # int64 [world + 1], the same on every rank

    @property
    def num_rows(self) -> int:
        return self.row1 - self.row0

    @property
    def nnz(self) -> int:
        return int(self.indices.shape[0])

    def rows_per_rank(self) -> List[int]:
        return [int(self.cuts[k + 1] - self.cuts[k]) for k in range(self.world)]


def shard_csr(indptr: np.ndarray, indices: np.ndarray, data: Optional[np.ndarray], num_cols: int,
              world: int, rank: int) -> RowShard:
    """The rank's row block under the nnz-balanced partition (deterministic: every rank computes
    the same cuts from the same matrix)."""
    indptr = np.ascontiguousarray(indptr, dtype=np.int32)
    cuts = fmt.row_partition(indptr, world)
    r0, r1 = int(cuts[rank]), int(cuts[rank + 1])
    p0, p1 = int(indptr[r0]), int(indptr[r1])
    return RowShard(rank, world, r0, r1, int(num_cols),
                    (indptr[r0:r1 + 1] - indptr[r0]).astype(np.int32),
                    np.ascontiguousarray(indices[p0:p1], dtype=np.int32),
                    None if data is None else np.ascontiguousarray(data[p0:p1]), cuts)


def shard_edges(shard: RowShard, full_indptr: np.ndarray) -> List[int]:
    """Stored entries per rank (sizes of the per-rank pieces of an edge-indexed output)."""
    return [int(full_indptr[shard.cuts[k + 1]] - full_indptr[shard.cuts[k]]) for k in range(shard.world)]


def broadcast_dense(x: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
    """Replicates the dense operand (in place) from ``src``."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(x, src=src, group=group)
    return x


def all_gather_blocks(local: torch.Tensor, sizes: Sequence[int], out: Optional[torch.Tensor] = None,
                      group=None) -> torch.Tensor:
    """Concatenation over ranks of 1-D blocks of unequal length ``sizes[k]`` (in elements).
    ``out``, when given, must be 1-D of length ``sum(sizes)``; the result is written there."""
    total = int(sum(sizes))
    if out is None:
        out = torch.empty(total, dtype=local.dtype, device=local.device)
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        out.copy_(local)
        return out
    rank = dist.get_rank(group)
    if local.numel() != sizes[rank]:
        raise ValueError(f"rank {rank}: local block has {local.numel()} elements, expected {sizes[rank]}")
    pieces = list(torch.split(out, [int(s) for s in sizes]))
    world = dist.get_world_size(group)
    biggest = int(max(sizes))
    if local.is_cuda and biggest * world == total:  # equal blocks: gather straight into place
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    if local.is_cuda:
        # Unequal blocks on GPUs: every rank sends its block to every other rank and receives
        # theirs straight into place, all in ONE batched group of point-to-point operations
        # (NCCL runs them concurrently over NVLink; nothing is staged or padded).
        pieces[rank].copy_(local)
        to_global = (lambda k: dist.get_global_rank(group, k)) if group is not None else (lambda k: k)
        p2p = []
        for k in range(world):
            if k == rank:
                continue
            if sizes[rank] > 0:
                p2p.append(dist.P2POp(dist.isend, pieces[rank], to_global(k), group))
            if sizes[k] > 0:
                p2p.append(dist.P2POp(dist.irecv, pieces[k], to_global(k), group))
        for req in (dist.batch_isend_irecv(p2p) if p2p else []):
            req.wait()
        return out
    # Otherwise an all-gather of unequal blocks is one broadcast per block (the library all-gather
    # wants equal sizes on some backends); the broadcasts are issued together and waited for together.
    pieces[rank].copy_(local)
    works = [dist.broadcast(pieces[k], src=dist.get_global_rank(group, k) if group is not None else k,
                            group=group, async_op=True)
             for k in range(world) if sizes[k] > 0]
    for w in works:
        w.wait()
    return out


def all_gather_rows(local: torch.Tensor, rows_per_rank: Sequence[int], feat: int,
                    out: Optional[torch.Tensor] = None, group=None) -> torch.Tensor:
    """All-gather of row blocks ``[rows_k * feat]`` into the full ``[sum(rows) * feat]`` output."""
    return all_gather_blocks(local, [int(r) * feat for r in rows_per_rank], out=out, group=group)


@dataclass
class BsrShard:
    """Block rows [row0, row1) of a BSR matrix with its own zero-based block indptr."""
    rank: int
    world: int
    row0: int
    row1: int
    indptr: np.ndarray   # int32 [row1 - row0 + 1]
    indices: np.ndarray  # int32 [stored blocks of the shard]
    data: np.ndarray     # [stored blocks of the shard, blk, blk]
    cuts: np.ndarray     # int64 [world + 1]


def shard_bsr(indptr: np.ndarray, indices: np.ndarray, data: np.ndarray, world: int, rank: int) -> BsrShard:
    """The rank's block rows under a partition balanced by stored blocks (the dense operand and
    the block column space stay whole)."""
    indptr = np.ascontiguousarray(indptr, dtype=np.int32)
    cuts = fmt.row_partition(indptr, world)
    r0, r1 = int(cuts[rank]), int(cuts[rank + 1])
    p0, p1 = int(indptr[r0]), int(indptr[r1])
    return BsrShard(rank, world, r0, r1, (indptr[r0:r1 + 1] - indptr[r0]).astype(np.int32),
                    np.ascontiguousarray(indices[p0:p1], dtype=np.int32), np.ascontiguousarray(data[p0:p1]), cuts)


@dataclass
class RgmsShard:
    """The part of an RGMS operand (CSF over relation / destination row / source) whose
    destination rows lie in [row0, row1); destination ids are re-based to the shard."""
    rank: int
    world: int
    row0: int
    row1: int
    indptr_i: np.ndarray   # int32 [num_rels + 1]
    indices_i: np.ndarray  # int32 [nnz_i of the shard], destination row - row0
    indptr_j: np.ndarray   # int32 [nnz_i of the shard + 1]
    indices_j: np.ndarray  # int32 [edges of the shard]
    data: np.ndarray       # float32 [edges of the shard]
    cuts: np.ndarray       # int64 [world + 1] over destination rows

    @property
    def num_rows(self) -> int:
        return self.row1 - self.row0


def rgms_row_cuts(indices_i: np.ndarray, indptr_j: np.ndarray, num_rows: int, world: int) -> np.ndarray:
    """Cut points over the destination rows with balanced numbers of edges: one writer per output
    row, so no reduction across GPUs is needed."""
    per_entry = np.diff(np.asarray(indptr_j, dtype=np.int64))
    per_row = np.bincount(np.asarray(indices_i, dtype=np.int64), weights=per_entry, minlength=num_rows)
    prefix = np.concatenate([[0], np.cumsum(per_row)]).astype(np.int32)
    return fmt.row_partition(prefix, world)


def shard_rgms(indptr_i: np.ndarray, indices_i: np.ndarray, indptr_j: np.ndarray, indices_j: np.ndarray,
               data: np.ndarray, num_rows: int, world: int, rank: int) -> RgmsShard:
    """The rank's destination-row block of an RGMS operand.  Inside a relation the destination
    rows are ascending, so the block is one contiguous run of level-0 entries per relation; the
    order of relations and of the entries of a row is kept, hence the same summation order."""
    indptr_i = np.asarray(indptr_i, dtype=np.int64)
    indices_i = np.asarray(indices_i, dtype=np.int64)
    indptr_j = np.asarray(indptr_j, dtype=np.int64)
    cuts = rgms_row_cuts(indices_i, indptr_j, num_rows, world)
    lo, hi = int(cuts[rank]), int(cuts[rank + 1])
    keep = (indices_i >= lo) & (indices_i < hi)
    num_rels = len(indptr_i) - 1
    rel_of = np.repeat(np.arange(num_rels), np.diff(indptr_i))
    new_indptr_i = np.concatenate([[0], np.cumsum(np.bincount(rel_of[keep], minlength=num_rels))])
    starts, ends = indptr_j[:-1][keep], indptr_j[1:][keep]
    lens = ends - starts
    new_indptr_j = np.concatenate([[0], np.cumsum(lens)])
    # positions of the kept edges: for every kept level-0 entry the run [start, end)
    edge_pos = np.repeat(starts - new_indptr_j[:-1], lens) + np.arange(int(new_indptr_j[-1]))
    return RgmsShard(rank, world, lo, hi, new_indptr_i.astype(np.int32),
                     (indices_i[keep] - lo).astype(np.int32), new_indptr_j.astype(np.int32),
                     np.ascontiguousarray(np.asarray(indices_j)[edge_pos], dtype=np.int32),
                     np.ascontiguousarray(np.asarray(data)[edge_pos], dtype=np.float32), cuts)
