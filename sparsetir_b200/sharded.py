"""Row-sharded operators on the GPUs of one box: shard -> replicate -> run -> gather.

The reference is single-GPU; this layer is new.  Every operator of the path is independent per
output row, so rank k of N holds a contiguous block of rows of the sparse operand with a balanced
share of the stored entries (``dist.shard_*``), the whole dense operand, and computes the output
rows (or per-position outputs) of its block with the single-GPU entry points.  The classes below
package that: construction shards and uploads the structure (every rank passes the SAME whole
matrix), ``run`` launches the shard's kernels, ``gather`` all-gathers the output blocks over NCCL
into the full result on every rank, optionally in row chunks so that the gather of chunk k
overlaps the kernels of chunk k + 1.  Into a buffer from ``peer_empty`` the gather is done by
direct writes into the other GPUs' memory over NVLink — by the operator's own kernel where it has
a form that stores to peers (hyb SpMM, SDDMM), by one scatter kernel, or by one copy-engine
transfer per peer — otherwise by NCCL.
``replicate_rows`` is the other collective of the path: every rank contributes an equal block of
rows of the dense operand.

A collective that fails (a peer that is gone, a timeout of the process group) raises
``ShardError`` — the counterpart, in this layer, of the -1 an entry point returns.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from . import dist as sdist
from . import format as fmt
from . import ops


class ShardError(RuntimeError):
    """A collective of the sharded layer failed (time-out, lost peer, mismatched sizes)."""


def _world(group=None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def guarded(what: str, fn: Callable, *args, **kwargs):
    """Runs a collective; any failure of the backend becomes a ShardError that names the step."""
    try:
        return fn(*args, **kwargs)
    except (ValueError, TypeError):
        raise
    except Exception as e:  # RuntimeError, DistBackendError, DistNetworkError ...
        raise ShardError(f"{what} failed on rank {_rank()}: {e}") from e


def row_block(num_rows: int, world: int) -> int:
    """Rows per rank of the equal-block layout used to replicate a dense operand: every rank owns
    ``row_block`` rows (the last ones may own fewer real rows; the buffer is padded)."""
    return -(-int(num_rows) // int(world))


def replicate_rows(local_rows: torch.Tensor, full: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of EQUAL row blocks: ``local_rows`` is this rank's ``[row_block * feat]`` piece,
    ``full`` the ``[world * row_block * feat]`` buffer that holds the whole (padded) operand
    afterwards.  One NCCL all-gather, in place."""
    world = _world(group)
    if world == 1:
        if full.data_ptr() != local_rows.data_ptr():
            full[:local_rows.numel()].copy_(local_rows)
        return full
    if full.numel() != world * local_rows.numel():
        raise ValueError("replicate_rows: full must hold world equal blocks")
    guarded("replicate_rows (all-gather of the dense operand)", dist.all_gather_into_tensor,
            full, local_rows.contiguous(), group=group)
    return full


class PeerOutput:
    """An output buffer that every GPU of the group can write into: ``tensor`` is this rank's
    buffer, ``peers[k]`` the same buffer of rank k mapped into this process (NVLink peer memory,
    torch symmetric memory).  Allocated collectively by ``peer_empty``."""

    def __init__(self, tensor: torch.Tensor, peers: List[torch.Tensor], handle):
        self.tensor, self.peers, self.handle = tensor, peers, handle

    def numel(self) -> int:
        return self.tensor.numel()


def peer_empty(numel: int, dtype: torch.dtype, device: torch.device, group=None):
    """Collective: a ``[numel]`` buffer on every rank, each mapped on all the others.  Returns a
    PeerOutput, or a plain tensor when the group has one rank, the device is not a GPU, or this
    torch build has no symmetric memory (the gathers then go through NCCL)."""
    world = _world(group)
    if world == 1 or device.type != "cuda":
        return torch.empty(numel, dtype=dtype, device=device)
    try:
        import torch.distributed._symmetric_memory as symm
        t = symm.empty(numel, dtype=dtype, device=device)
        handle = symm.rendezvous(t, group if group is not None else dist.group.WORLD)
        peers = [handle.get_buffer(k, (numel,), dtype) for k in range(world)]
        return PeerOutput(t, peers, handle)
    except Exception as e:  # no symmetric memory here: NCCL path
        import warnings
        warnings.warn(f"peer memory unavailable ({e!r}); output all-gathers will use NCCL")
        return torch.empty(numel, dtype=dtype, device=device)


def local_tensor(out) -> torch.Tensor:
    return out.tensor if isinstance(out, PeerOutput) else out


_TRANSPORT_DEFAULT = {
    # measured on NVSwitch (2 and 4 B200s), step ending with the output whole on every rank:
    "hyb_spmm": "fused",   # 0.56 against 0.68 ms (2 GPUs), 0.96 against 1.22 ms (4 GPUs) for copy engines
    "sddmm": "copy",       # long gather-bound kernels: copy engines overlap them without SM time
    "bsrmm": "scatter",    # blocks of a few MB: one kernel costs 46 us where three transfers cost 117
    "rgms": "scatter",
}


def _peer_transport(op: str = "hyb_spmm") -> str:
    """How an operator's blocks reach the peers' buffers: ``fused`` (hyb SpMM and SDDMM: the
    kernel that finishes an output row stores it to every peer itself), ``scatter`` (one kernel
    after the call reads the block once and stores it to every peer) or ``copy`` (one copy-engine
    transfer per peer after the call).  ``SPARSETIR_PEER_TRANSPORT`` overrides the per-operator
    default; operators without a fused form take ``scatter`` for ``fused``."""
    v = os.environ.get("SPARSETIR_PEER_TRANSPORT", _TRANSPORT_DEFAULT[op]).lower()
    if v not in ("fused", "scatter", "copy"):
        raise ValueError(f"SPARSETIR_PEER_TRANSPORT={v!r}: expected 'fused', 'scatter' or 'copy'")
    if v == "fused" and op not in ("hyb_spmm", "sddmm"):
        v = "scatter"
    return v


def peer_transport_note(op: str = "hyb_spmm") -> str:
    """One line for reports: what moves the operator's blocks into the peers' buffers."""
    return {"fused": "the kernel that finishes an output row stores it into the peers' buffers itself",
            "scatter": "one kernel after the call reads the block once and stores it to every peer",
            "copy": "one copy-engine transfer per peer after the call"}[_peer_transport(op)] + \
        "; peer memory from torch symmetric memory, completion by a one-element all-reduce"


class _Gatherer:
    """All-gather of per-rank output blocks, issued on side streams so that it overlaps whatever
    the caller launches next.

    Into a PeerOutput every rank WRITES its block straight into the other ranks' buffers over
    NVLink: with one kernel of this library that reads the block once and stores it to every peer
    (``scatter``), or with one copy-engine transfer per peer, all peers at once (``copy``; no SM
    time, so it overlaps long kernels) — see ``_peer_transport``.  ``wait()`` then joins the side
    streams and meets the other ranks in a one-element NCCL all-reduce: when it completes on a
    rank, every peer's writes into that rank have completed (a rank enters the all-reduce only
    after its own).  Operators whose kernels store into the peers themselves (``fused``) only mark
    the gatherer pending, so that ``wait()`` runs the same completion step.
    Into a plain tensor the blocks go through NCCL (one group of broadcasts for unequal blocks)."""

    def __init__(self, device: torch.device, op: str = "hyb_spmm"):
        self.device = device
        self.op = op
        self.stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self.peer_streams: List = []
        self.pending: List = []
        self.p2p_pending = False
        self._token = None

    def gather(self, local: torch.Tensor, sizes: Sequence[int], out, offsets: Sequence[int],
               group=None, transport: Optional[str] = None) -> None:
        """Blocks of ``sizes[k]`` elements, rank k's going to ``out[offsets[k]:offsets[k]+sizes[k]]``
        on every rank; runs after everything queued so far on the current stream.  ``transport``
        ('scatter' or 'copy') overrides the operator's default for this block."""
        world, rank = _world(group), _rank(group)
        mine = local_tensor(out)[int(offsets[rank]):int(offsets[rank]) + int(sizes[rank])]
        if local.numel() != sizes[rank]:
            raise ValueError(f"rank {rank}: local block has {local.numel()} elements, expected {sizes[rank]}")
        if world == 1:
            if mine.data_ptr() != local.data_ptr():
                mine.copy_(local)
            return
        if isinstance(out, PeerOutput):
            if not self.peer_streams:
                # high priority: a transfer queued behind chunk k starts as soon as chunk k ends,
                # ahead of the blocks of chunk k+1's kernels that are already waiting for SMs
                self.peer_streams = [torch.cuda.Stream(device=self.device, priority=-1) for _ in range(world)]
            if mine.data_ptr() != local.data_ptr():
                mine.copy_(local)
            if local.numel() > 0:
                ready = torch.cuda.Event()
                ready.record()
                lo, hi = int(offsets[rank]), int(offsets[rank]) + int(sizes[rank])
                order = [(rank + step) % world for step in range(1, world)]  # every rank starts with another peer
                if (transport or _peer_transport(self.op)) in ("scatter", "fused"):
                    # one kernel: the block is read once and stored to every peer
                    from . import _lib as L
                    src = local.contiguous()
                    dst = (ctypes.c_void_p * len(order))(
                        *[out.peers[k].data_ptr() + lo * out.peers[k].element_size() for k in order])
                    s = self.peer_streams[rank]
                    s.wait_event(ready)
                    src.record_stream(s)
                    if L.load().sparsetir_peer_scatter(self.device.index, ctypes.c_void_p(s.cuda_stream),
                                                       ctypes.c_void_p(src.data_ptr()),
                                                       src.numel() * src.element_size(), len(order), dst) != 0:
                        raise ShardError(f"rank {rank}: peer scatter failed: {L.last_error()}")
                else:
                    for k in order:  # one copy-engine transfer per peer
                        s = self.peer_streams[k]
                        with torch.cuda.stream(s):
                            s.wait_event(ready)
                            out.peers[k][lo:hi].copy_(local, non_blocking=True)
            self.p2p_pending = True
            return
        pieces = [out[int(o):int(o) + int(s)] for o, s in zip(offsets, sizes)]
        if self.stream is None or min(int(s) for s in sizes) == 0:
            # CPU ranks (gloo) and degenerate cuts: the broadcast-based path of the base layer
            tmp = guarded("all-gather of the output blocks", sdist.all_gather_blocks, local, sizes, group=group)
            for p, t in zip(pieces, torch.split(tmp, [int(s) for s in sizes])):
                if p.data_ptr() != t.data_ptr():
                    p.copy_(t)
            return
        done = torch.cuda.Event()
        done.record()
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(done)
            # unequal blocks straight into place: NCCL runs them as one group of broadcasts
            work = guarded("all-gather of the output blocks", dist.all_gather, pieces, local,
                           group=group, async_op=True)
        self.pending.append(work)

    def wait(self, group=None) -> None:
        """Makes the current stream wait for every gather issued so far (and, for peer writes,
        for the other ranks' writes into this rank's buffer)."""
        for w in self.pending:
            guarded("all-gather of the output blocks", w.wait)
        self.pending.clear()
        if self.p2p_pending:
            cur = torch.cuda.current_stream(self.device)
            for s in self.peer_streams:
                cur.wait_stream(s)
            if self._token is None:
                self._token = torch.zeros(1, device=self.device)
            guarded("completion of the peer writes (all-reduce)", dist.all_reduce, self._token, group=group)
            self.p2p_pending = False


def _dev(a, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


class ShardedHybSpmm:
    """Y = A X with A decomposed into the hyb format shard by shard."""

    def __init__(self, indptr, indices, data, num_cols: int, buckets: Sequence[int], parts: int = 1,
                 device: Optional[torch.device] = None, group=None):
        self.group, self.world, self.rank = group, _world(group), _rank(group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.num_rows_total = len(indptr) - 1
        self.num_cols = int(num_cols)
        self.shard = sdist.shard_csr(indptr, indices, data, num_cols, self.world, self.rank)
        rows, cols, mask, vals, _ = fmt.column_part_hyb(self.shard.num_rows, num_cols, self.shard.indptr,
                                                       self.shard.indices, parts, list(buckets),
                                                       data=self.shard.data)
        self.buckets = [(_dev(vals[p][b], self.device), _dev(rows[p][b], self.device), _dev(cols[p][b], self.device))
                        for p in range(parts) for b in range(len(buckets))]
        from . import _lib as L
        self.flags = (L.HYB_REARM | L.HYB_ALL_ATOMIC) if parts > 1 else 0
        self.rows_per_rank = self.shard.rows_per_rank()
        self.row_offsets = [int(c) for c in self.shard.cuts[:-1]]
        self.referenced_cols = int(np.unique(self.shard.indices).size)
        self._gatherer = _Gatherer(self.device, "hyb_spmm")

    def prepare(self, x: torch.Tensor, y_local: torch.Tensor, feat: int) -> ops.PreparedCall:
        """The shard's call: ``x`` is the whole dense operand ``[num_cols * feat]`` on this GPU,
        ``y_local`` the ``[shard rows * feat]`` output block (zero-filled once by the caller)."""
        return ops.hyb_spmm.prepare(*ops.hyb_args(x, y_local, self.buckets, feat, self.flags))

    def prepare_gathered(self, x: torch.Tensor, out, feat: int) -> Callable[[], None]:
        """The shard's call that leaves its rows in ``out [num_rows_total * feat]`` on EVERY rank
        (``out`` from ``peer_empty``, or a plain tensor); ``wait()`` after it orders later work
        behind the other ranks' rows.  With peer memory and the 'fused' transport the SpMM kernel
        itself stores each finished row into every peer's buffer (``hyb_spmm_peers``): no copy
        follows the kernel.  Otherwise the kernel writes this rank's rows and a gather follows.
        As with any collective into a reused buffer: a rank may run the call again only when every
        rank is done reading the previous result (a ``wait()``, or any other collective, after the
        reads)."""
        lo = self.row_offsets[self.rank] * feat
        n = self.rows_per_rank[self.rank] * feat
        mine = local_tensor(out)[lo:lo + n]
        if isinstance(out, PeerOutput) and self.world > 1 and self.flags == 0 and _peer_transport() == "fused":
            order = [(self.rank + step) % self.world for step in range(1, self.world)]
            peer_c = [out.peers[k].data_ptr() + lo * out.peers[k].element_size() for k in order]
            fused_call = ops.hyb_spmm_peers.prepare(*ops.hyb_args(x, mine, self.buckets, feat, 0, peer_c=peer_c))
            plain_call = self.prepare(x, mine, feat)
            gatherer = self._gatherer
            state = {"fused": True}

            def run_fused() -> None:
                if state["fused"]:
                    try:
                        fused_call()
                        gatherer.p2p_pending = True  # the peers' rows arrive with THEIR kernels: wait() meets them
                        return
                    except ops.SparseTIRError:
                        # shapes the one-writer kernel does not take (refused before any launch):
                        # from now on the plain call followed by a transfer
                        state["fused"] = False
                plain_call()
                self.gather(mine, feat, out)

            return run_fused
        call = self.prepare(x, mine, feat)

        def run_then_gather() -> None:
            call()
            self.gather(mine, feat, out)

        return run_then_gather

    def gather(self, y_local: torch.Tensor, feat: int, out) -> None:
        """Queues the all-gather of the output rows into ``out [num_rows_total * feat]`` (a tensor,
        or a PeerOutput from ``peer_empty``) behind the work queued so far; ``wait()`` orders later
        work after it."""
        self._gatherer.gather(y_local, [r * feat for r in self.rows_per_rank], out,
                              [o * feat for o in self.row_offsets], self.group)

    def wait(self) -> None:
        self._gatherer.wait(self.group)


class _ChunkCalls(list):
    """The prepared calls of a shard's chunks; ``fused`` says that the kernels themselves store
    into the peers' buffers, so that no transfer follows them."""
    fused = False
    transport: Optional[str] = None  # 'scatter' / 'copy' chosen for these calls, None = the default


class ShardedSddmm:
    """out[p] = scale[p] * <A[row(p)], B[col(p)]> over the stored positions of the shard's rows,
    the rows cut into ``chunks`` pieces (balanced by stored positions) so that the all-gather of
    one piece overlaps the kernels of the next."""

    def __init__(self, indptr, indices, scale, num_cols: int, chunks: int = 4,
                 device: Optional[torch.device] = None, group=None):
        self.group, self.world, self.rank = group, _world(group), _rank(group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        on_device = isinstance(indptr, torch.Tensor)
        ip_host = indptr.cpu().numpy() if on_device else np.ascontiguousarray(indptr, dtype=np.int32)
        self.num_rows_total, self.num_cols = len(ip_host) - 1, int(num_cols)
        self.nnz_total = int(ip_host[-1])
        cuts = fmt.row_partition(ip_host, self.world)
        self.cuts = cuts
        self.row0, self.row1 = int(cuts[self.rank]), int(cuts[self.rank + 1])
        chunks = max(1, int(chunks)) if self.world > 1 else 1
        # every rank needs every rank's chunk boundaries (sizes and offsets of the gathered pieces)
        self.chunk_sizes: List[List[int]] = [[] for _ in range(chunks)]
        self.chunk_offsets: List[List[int]] = [[] for _ in range(chunks)]
        my_rows: List[int] = []
        for k in range(self.world):
            r0, r1 = int(cuts[k]), int(cuts[k + 1])
            sub = fmt.row_partition((ip_host[r0:r1 + 1] - ip_host[r0]).astype(np.int32), chunks)
            for c in range(chunks):
                a, b = r0 + int(sub[c]), r0 + int(sub[c + 1])
                self.chunk_sizes[c].append(int(ip_host[b] - ip_host[a]))
                self.chunk_offsets[c].append(int(ip_host[a]))
            if k == self.rank:
                my_rows = [r0 + int(s) for s in sub]
        self.chunk_rows = my_rows  # chunks + 1 global row numbers
        to_dev = (lambda t: t.to(self.device)) if on_device else (lambda a: _dev(a, self.device))
        self._ip, self._ix, self._scale = [], [], []
        for c in range(chunks):
            a, b = my_rows[c], my_rows[c + 1]
            p0, p1 = int(ip_host[a]), int(ip_host[b])
            self._ip.append(_dev((ip_host[a:b + 1] - ip_host[a]).astype(np.int32), self.device))
            self._ix.append(to_dev(indices[p0:p1]).contiguous())
            self._scale.append(None if scale is None else to_dev(scale[p0:p1]).contiguous())
        self.chunks = chunks
        self._gatherer = _Gatherer(self.device, "sddmm")

    def prepare(self, a: torch.Tensor, b: torch.Tensor, out_full, feat: int) -> List[ops.PreparedCall]:
        """One call per chunk: ``a`` is the whole row-side operand ``[num_rows_total * feat]`` (only
        the shard's rows are read), ``b`` the replicated column-side operand, ``out_full`` the
        ``[nnz_total]`` result (a tensor or a PeerOutput); each chunk writes its own range of it."""
        # with peer memory and the 'fused' transport the kernel stores every finished position
        # into the peers' buffers itself (sddmm_peers): run() then queues no transfer
        fused = (isinstance(out_full, PeerOutput) and self.world > 1 and _peer_transport("sddmm") == "fused"
                 and feat % 32 == 0 and a.data_ptr() % 32 == 0 and b.data_ptr() % 32 == 0)
        order = [(self.rank + step) % self.world for step in range(1, self.world)]
        peers = out_full.peers if fused else None
        calls = _ChunkCalls()
        calls.fused = fused
        if "SPARSETIR_PEER_TRANSPORT" not in os.environ and self.world > 1:
            # Copy engines hide a chunk's transfer behind the next chunk's kernels; when the
            # transfer is more than twice as long as those kernels there is little to hide behind
            # and the scatter kernel's lower fixed cost wins (4 GPUs, F = 32: 0.83 against 1.00 ms).
            # Estimates per stored position: 4 (N-1) bytes over ~660 GB/s of NVLink against
            # 4 F bytes of gathered row over ~15 TB/s of L2-to-SM rate.
            transfer = 4.0 * (self.world - 1) / 660e9
            kernels = 4.0 * feat / 15e12
            calls.transport = "scatter" if transfer > 2.0 * kernels else "copy"
        out_full = local_tensor(out_full)
        for c in range(self.chunks):
            r0, r1 = self.chunk_rows[c], self.chunk_rows[c + 1]
            off, size = self.chunk_offsets[c][self.rank], self.chunk_sizes[c][self.rank]
            args = [a[r0 * feat:r1 * feat], b, out_full[off:off + size], self._ip[c], self._ix[c]]
            if fused:
                args += [peers[k].data_ptr() + off * peers[k].element_size() for k in order]
            if self._scale[c] is not None:
                args.append(self._scale[c])
            fn = ops.sddmm_peers if fused else ops.sddmm
            calls.append(fn.prepare(*args) if size > 0 else None)
        return calls

    def run(self, calls: List, out_full=None) -> None:
        """Launches the chunks in order; with ``out_full`` (the buffer given to ``prepare``) every
        chunk's all-gather is queued right behind its kernels (call ``wait()`` before reading other
        ranks' parts)."""
        for c, call in enumerate(calls):
            if call is not None:
                call()
            if out_full is not None and self.world > 1 and getattr(calls, "fused", False):
                self._gatherer.p2p_pending = True  # the rows of the others arrive with THEIR kernels
            elif out_full is not None and self.world > 1:
                off, size = self.chunk_offsets[c][self.rank], self.chunk_sizes[c][self.rank]
                self._gatherer.gather(local_tensor(out_full)[off:off + size], self.chunk_sizes[c], out_full,
                                      self.chunk_offsets[c], self.group, getattr(calls, "transport", None))

    def wait(self) -> None:
        self._gatherer.wait(self.group)


class ShardedBsrmm:
    """C = A B for a BSR matrix cut into block rows balanced by stored blocks."""

    def __init__(self, indptr, indices, blocks, num_block_cols: int, blk: int,
                 device: Optional[torch.device] = None, group=None):
        self.group, self.world, self.rank = group, _world(group), _rank(group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.blk, self.num_block_cols = int(blk), int(num_block_cols)
        self.shard = sdist.shard_bsr(indptr, indices, blocks, self.world, self.rank)
        self.block_rows_total = len(indptr) - 1
        self.block_rows = self.shard.row1 - self.shard.row0
        self.nnzb = len(self.shard.indices)
        self._a = _dev(self.shard.data.reshape(-1), self.device)
        self._ip, self._ix = _dev(self.shard.indptr, self.device), _dev(self.shard.indices, self.device)
        self.rows_per_rank = [int(self.shard.cuts[k + 1] - self.shard.cuts[k]) * self.blk for k in range(self.world)]
        self.row_offsets = [int(c) * self.blk for c in self.shard.cuts[:-1]]
        self._gatherer = _Gatherer(self.device, "bsrmm")

    def prepare(self, b: torch.Tensor, c_local: torch.Tensor, feat: int) -> Optional[ops.PreparedCall]:
        if self.block_rows == 0:
            return None
        return ops.bsrmm.prepare(self._a, b, c_local, self._ip, self._ix, self.block_rows,
                                 self.num_block_cols, self.nnzb, self.blk, feat)

    def gather(self, c_local: torch.Tensor, feat: int, out) -> None:
        self._gatherer.gather(c_local, [r * feat for r in self.rows_per_rank], out,
                              [o * feat for o in self.row_offsets], self.group)

    def wait(self) -> None:
        self._gatherer.wait(self.group)


class ShardedRgms:
    """Y = sum_r A_r X W_r cut by destination rows (balanced by edges): one writer per output row,
    no reduction across GPUs."""

    def __init__(self, indptr_i, indices_i, indptr_j, indices_j, data, num_rows: int, num_cols: int,
                 device: Optional[torch.device] = None, group=None):
        self.group, self.world, self.rank = group, _world(group), _rank(group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.num_rows_total, self.num_cols = int(num_rows), int(num_cols)
        self.shard = sdist.shard_rgms(indptr_i, indices_i, indptr_j, indices_j, data, num_rows,
                                      self.world, self.rank)
        s = self.shard
        self._arrays = [_dev(v, self.device) for v in (s.data, s.indptr_i, s.indices_i, s.indptr_j, s.indices_j)]
        self.rows_per_rank = [int(s.cuts[k + 1] - s.cuts[k]) for k in range(self.world)]
        self.row_offsets = [int(c) for c in s.cuts[:-1]]
        self._gatherer = _Gatherer(self.device, "rgms")

    def prepare(self, w: torch.Tensor, x: torch.Tensor, y_local: torch.Tensor) -> Optional[ops.PreparedCall]:
        """``y_local [shard rows * feat]`` is accumulated into (zero-fill it first)."""
        if self.shard.num_rows == 0 or len(self.shard.indices_i) == 0:
            return None
        a, ip_i, ix_i, ip_j, ix_j = self._arrays
        return ops.rgms.prepare(a, w, x, y_local, ip_i, ix_i, ip_j, ix_j)

    def gather(self, y_local: torch.Tensor, feat: int, out) -> None:
        self._gatherer.gather(y_local, [r * feat for r in self.rows_per_rank], out,
                              [o * feat for o in self.row_offsets], self.group)

    def wait(self) -> None:
        self._gatherer.wait(self.group)
