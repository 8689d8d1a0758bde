"""Sharding of the contraction kernels across the GPUs of one box (one process per GPU).

The reference is single-device (``DEFAULT_NUM_DEVICES = 1``, cuda-async/src/device_context.rs:31);
this module adds the two partitions the kernels admit without any data-path exchange:

* GEMM: split N.  Rank r owns the weight columns ``B[:, n0:n1]`` (or rows of the K-major weight
  ``B[n0:n1, :]``) and computes ``C[:, n0:n1] = A . B_r`` from a replicated ``A``.
* Attention: split the (batch x head) problems; Q, K, V, O slabs are contiguous per problem.

A collective (NCCL all-gather over NVLink) runs only when the caller asks for a replicated result.
Column shards of a row-major matrix are strided, so the gather lands in a ``[world, M, N/world]``
staging buffer and one local copy re-lays it out as ``[M, N]``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def split_range(total: int, world: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """Contiguous share ``[start, stop)`` of ``total`` items for ``rank``; every boundary is a
    multiple of ``align`` (scale-block or tile alignment) and earlier ranks take the remainder."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} / world {world}")
    if total % align != 0:
        raise ValueError(f"total {total} is not a multiple of the alignment {align}")
    units = total // align
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    stop = start + base + (1 if rank < extra else 0)
    return start * align, stop * align


def shard_columns(b: torch.Tensor, world: int, rank: int, align: int = 8) -> torch.Tensor:
    """This rank's column block of a ``[K, N]`` weight, made contiguous (done once at set-up)."""
    n0, n1 = split_range(b.shape[1], world, rank, align)
    return b[:, n0:n1].contiguous()


def shard_rows(b: torch.Tensor, world: int, rank: int, align: int = 8) -> torch.Tensor:
    """This rank's row block of a K-major ``[N, K]`` weight."""
    n0, n1 = split_range(b.shape[0], world, rank, align)
    return b[n0:n1].contiguous()


def shard_problems(x: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """This rank's slab of the leading (batch x head) axis of a ``[BH, S, D]`` tensor."""
    p0, p1 = split_range(x.shape[0], world, rank, 1)
    return x[p0:p1]


def all_gather_columns(c_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None
                       ) -> torch.Tensor:
    """Reassembles ``C[M, N]`` from equal-width column shards on every rank."""
    world = dist.get_world_size(group)
    if world == 1:
        return c_local
    m, n_local = c_local.shape
    staging = torch.empty((world * m, n_local), dtype=c_local.dtype, device=c_local.device)
    dist.all_gather_into_tensor(staging, c_local.contiguous(), group=group)
    return staging.view(world, m, n_local).permute(1, 0, 2).reshape(m, world * n_local)


def all_gather_problems(o_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None
                        ) -> torch.Tensor:
    """Reassembles ``O[BH, S, D]`` from equal (batch x head) slabs on every rank."""
    world = dist.get_world_size(group)
    if world == 1:
        return o_local
    out = torch.empty((world * o_local.shape[0],) + tuple(o_local.shape[1:]), dtype=o_local.dtype,
                      device=o_local.device)
    dist.all_gather_into_tensor(out, o_local.contiguous(), group=group)
    return out


def all_gather_rows(a_full: torch.Tensor, rank_rows: torch.Tensor, group: Optional[dist.ProcessGroup] = None
                    ) -> torch.Tensor:
    """Completes ``a_full[M, K]`` on every rank from equal row slabs (rank r holds rows ``[r M/G, (r+1) M/G)``).
    Row slabs of a row-major matrix are contiguous, so the gather writes ``a_full`` directly; ``rank_rows`` may be
    the rank's own slab of ``a_full`` (gather in place)."""
    world = dist.get_world_size(group)
    if world == 1:
        if rank_rows.data_ptr() != a_full.data_ptr():
            a_full.copy_(rank_rows)
        return a_full
    if a_full.shape[0] != world * rank_rows.shape[0] or not a_full.is_contiguous():
        raise ValueError("all_gather_rows: a_full must be contiguous with world x the rank's rows")
    dist.all_gather_into_tensor(a_full, rank_rows, group=group)
    return a_full


def chunk_block_rows(rank: int, world: int, m: int, chunks: int, j: int) -> Tuple[int, int]:
    """Global rows ``[start, stop)`` of A (and C) that block ``rank`` of row chunk ``j`` holds when every rank's M/G
    rows are cut into ``chunks`` equal parts: the chunk-major layout of :class:`ShardedHostGemm`."""
    slab = m // world
    sub = slab // chunks
    return rank * slab + j * sub, rank * slab + (j + 1) * sub


class ShardedHostGemm:
    """C[:, n0:n1] = A . B[:, n0:n1] for operands that live in HOST memory, on the ranks of one box.

    The activation matrix A is needed whole by every rank, but it crosses PCIe only once: rank r uploads rows
    ``[r M/G, (r+1) M/G)`` from its pinned host slab and NCCL all-gathers over NVLink complete A in every rank's HBM.
    The step is a pipeline over ``chunks`` row chunks: the rank's weight columns (B shard) go up first, then chunk j of
    its A rows; as soon as a chunk is up it is all-gathered, multiplied (`b200tile_gemm`, weight-column split: no
    data-path collective) and its C rows travel back while the next chunk is still coming in.  With eight ranks
    copying at once the host side is the bottleneck of such a step (a 16.8 MB upload takes 0.5-0.7 ms and the same
    download 0.9-1.4 ms on the boxes this was measured on), so overlapping the two directions is what shortens it.

    In HBM, A and C are kept chunk-major (``[chunks][G x rows per chunk][.]``): chunk j holds rows
    ``r M/G + j sub + i`` of every rank r, so that a gathered chunk is one contiguous matrix."""

    def __init__(self, m: int, n_local: int, k: int, dtype: str = "bf16", group: Optional[dist.ProcessGroup] = None,
                 chunks: int = 0):
        from . import _lib
        from .tensor import _NAME_TO_TORCH
        self._lib = _lib.load()
        self._check = _lib.check
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if m % self.world:
            raise ValueError("ShardedHostGemm: M must be a multiple of the number of ranks")
        self.m, self.n, self.k, self.dtype = m, n_local, k, dtype
        slab = m // self.world
        if chunks <= 0:   # as many as leave at least 128 rows per rank and chunk
            chunks = next((c for c in (4, 2) if slab % c == 0 and slab // c >= 128), 1)
        if slab % chunks:
            raise ValueError("ShardedHostGemm: the rank's rows must divide into the chunks")
        self.chunks, self.sub = chunks, slab // chunks
        td = _NAME_TO_TORCH[dtype]
        dev = torch.device("cuda", torch.cuda.current_device())
        self.a_dev = torch.empty((chunks, self.world * self.sub, k), dtype=td, device=dev)
        self.b_dev = torch.empty((k, n_local), dtype=td, device=dev)
        self.c_dev = torch.empty((chunks, self.world * self.sub, n_local), dtype=td, device=dev)
        self.rows = (self.rank * slab, (self.rank + 1) * slab)
        self.in_stream, self.out_stream = torch.cuda.Stream(), torch.cuda.Stream()

    def __call__(self, a_rows_host: torch.Tensor, b_host: torch.Tensor, c_host: torch.Tensor,
                 stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """``a_rows_host``: this rank's M/G rows of A (pinned); ``b_host``: its [K, N/G] weight columns (pinned);
        ``c_host`` [M, N/G] is complete once ``stream`` has been synchronised."""
        s = stream or torch.cuda.current_stream()
        g, sub = self.world, self.sub
        s_in, s_out = self.in_stream, self.out_stream
        s_in.wait_stream(s)                                # earlier work on s may still read the device buffers
        s_out.wait_stream(s)
        ups = []
        with torch.cuda.stream(s_in):                      # one upload queue: B, then the chunks of A in order
            self.b_dev.copy_(b_host, non_blocking=True)
            for j in range(self.chunks):
                self.a_dev[j, self.rank * sub:(self.rank + 1) * sub].copy_(a_rows_host[j * sub:(j + 1) * sub],
                                                                           non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
                ups.append(ev)
        with torch.cuda.stream(s):
            for j in range(self.chunks):
                s.wait_event(ups[j])
                if g > 1:
                    dist.all_gather_into_tensor(self.a_dev[j], self.a_dev[j, self.rank * sub:(self.rank + 1) * sub],
                                                group=self.group)
                self._check(self._lib.b200tile_gemm(self.dtype.encode(), 0, self.a_dev[j].data_ptr(),
                                                    self.b_dev.data_ptr(), self.c_dev[j].data_ptr(), 1, g * sub, self.n,
                                                    self.k, self.k, self.n, self.n, 0, 0, 0, 0, -1, 0, 0, s.cuda_stream))
                done = torch.cuda.Event()
                done.record(s)
                s_out.wait_event(done)
                with torch.cuda.stream(s_out):
                    for r in range(g):
                        g0, g1 = chunk_block_rows(r, g, self.m, self.chunks, j)
                        c_host[g0:g1].copy_(self.c_dev[j, r * sub:(r + 1) * sub], non_blocking=True)
            s.wait_stream(s_in)                            # synchronising s covers every copy of the call
            s.wait_stream(s_out)
        return c_host


def max_over_ranks(ms: float, device: torch.device, group: Optional[dist.ProcessGroup] = None
                   ) -> float:
    """Device-timed duration reduced with MAX over ranks (the job time of a sharded step)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
