"""Column (N) sharding of the quantized matmuls across the GPUs of one node.

The reference has no multi-GPU code.  Output columns are independent - C[:, n0:n1] needs all
of A but only B[:, n0:n1] - so each rank owns a contiguous [K, N/g] slab of the weights
(pre-sharded once, like column-parallel layers), calls the same single-GPU `solve` on it
and writes its own slab of C.  No data-path collective is needed; an all-gather of C over
NCCL/NVLink is optional.  One process per GPU (torch.distributed).
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from . import ops

SLAB_ALIGN = 128  # keeps every slab a whole number of MMA tile columns / TMA boxes


def slab_width(N: int, world: int, align: int = SLAB_ALIGN) -> int:
    """Width of every rank's column slab (the last ranks' may be cut short or empty)."""
    if N <= 0 or world <= 0:
        raise ValueError("N and world must be positive")
    per = -(-N // world)
    return -(-per // align) * align


def column_slab(N: int, world: int, rank: int, align: int = SLAB_ALIGN) -> tuple[int, int]:
    """[n0, n1) owned by `rank`."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    w = slab_width(N, world, align)
    n0 = min(N, rank * w)
    return n0, min(N, n0 + w)


def shard_columns(B: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """The rank's [K, n1-n0] slab of a row-major [K, N] weight, as its own contiguous matrix."""
    n0, n1 = column_slab(B.shape[1], world, rank)
    return B[:, n0:n1].contiguous()


def shard_rows(W: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """For the W4A16 layout (w_q [N, K/2], scales [N, K/G]) output columns are weight rows."""
    n0, n1 = column_slab(W.shape[0], world, rank)
    return W[n0:n1].contiguous()


def all_gather_columns(C_slab: torch.Tensor, N: int, group=None) -> torch.Tensor:
    """Assemble the full row-major [M, N] output from every rank's column slab.

    all_gather delivers [world, M, w]; the slabs are then interleaved back into rows.  Slabs
    are padded to the common width so the collective is a single equal-size all-gather."""
    world = dist.get_world_size(group)
    M = C_slab.shape[0]
    w = slab_width(N, world)
    if C_slab.shape[1] != w:
        padded = C_slab.new_zeros((M, w))
        padded[:, : C_slab.shape[1]] = C_slab
        C_slab = padded
    gathered = C_slab.new_empty((world * M, w))  # rank-major concatenation along dim 0
    dist.all_gather_into_tensor(gathered, C_slab.contiguous(), group=group)
    return gathered.view(world, M, w).permute(1, 0, 2).reshape(M, world * w)[:, :N].contiguous()


def mm_int8_sharded(A: torch.Tensor, B_slab: torch.Tensor, N: int, scale_A: float, scale_B: float,
                    scale_C: float, zero_point_A: int, zero_point_B: int, zero_point_C: int,
                    gather: bool = False, group=None,
                    solver: Callable[..., torch.Tensor] | None = None) -> torch.Tensor:
    """Rank-local slab of C (or, with gather=True, the whole C on every rank).

    `B_slab` is this rank's `shard_columns` of the weights; A is replicated.  `solver` is
    the single-GPU operator (default: the CUDA mm_int8)."""
    solver = solver or ops.mm_int8
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    n0, n1 = column_slab(N, world, rank)
    if B_slab.shape[1] != n1 - n0:
        raise ValueError(f"rank {rank}: slab has {B_slab.shape[1]} columns, expected {n1 - n0}")
    if n1 > n0:
        C_slab = solver(A, B_slab, scale_A, scale_B, scale_C, zero_point_A, zero_point_B,
                        zero_point_C)
    else:
        C_slab = A.new_empty((A.shape[0], 0), dtype=torch.int8)
    return all_gather_columns(C_slab, N, group) if gather else C_slab


def mm_int4_sharded(x: torch.Tensor, w_q_slab: torch.Tensor, scales_slab: torch.Tensor, N: int,
                    group_size: int, gather: bool = False, group=None,
                    solver: Callable[..., torch.Tensor] | None = None) -> torch.Tensor:
    solver = solver or ops.mm_int4
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    n0, n1 = column_slab(N, world, rank)
    if w_q_slab.shape[0] != n1 - n0:
        raise ValueError(f"rank {rank}: slab has {w_q_slab.shape[0]} rows, expected {n1 - n0}")
    if n1 > n0:
        y_slab = solver(x, w_q_slab, scales_slab, group_size)
    else:
        y_slab = x.new_empty((x.shape[0], 0))
    return all_gather_columns(y_slab, N, group) if gather else y_slab
