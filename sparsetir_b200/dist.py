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
    # An all-gather of unequal blocks is one broadcast per block (the library all-gather wants
    # equal sizes on some backends); the broadcasts are issued together and waited for together.
    pieces = list(torch.split(out, [int(s) for s in sizes]))
    pieces[rank].copy_(local)
    world = dist.get_world_size(group)
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
