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


def max_over_ranks(ms: float, device: torch.device, group: Optional[dist.ProcessGroup] = None
                   ) -> float:
    """Device-timed duration reduced with MAX over ranks (the job time of a sharded step)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
