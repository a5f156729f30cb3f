"""Column (N) sharding of the quantized matmuls across the GPUs of one node.

The reference has no multi-GPU code.  Output columns are independent - C[:, n0:n1] needs all
of A but only B[:, n0:n1] - so each rank owns a contiguous [K, N/g] slab of the weights
(pre-sharded once, like column-parallel layers), calls the same single-GPU `solve` on it
and writes its own slab of C.  No data-path collective is needed; an all-gather of C over
NCCL/NVLink is optional.  One process per GPU (torch.distributed).
"""
from __future__ import annotations

import ctypes
from typing import Callable

import torch
import torch.distributed as dist

from . import _lib, ops

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


def mm_int4a8_sharded(A: torch.Tensor, w_q_slab: torch.Tensor, N: int, scale_A: float, scale_B: float,
                      scale_C: float, zero_point_A: int, zero_point_B: int, zero_point_C: int,
                      gather: bool = False, group=None,
                      solver: Callable[..., torch.Tensor] | None = None) -> torch.Tensor:
    """W4A8: output columns are rows of w_q [N, K/2], so a rank's slab is `shard_rows(w_q)`."""
    solver = solver or ops.mm_int4a8
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    n0, n1 = column_slab(N, world, rank)
    if w_q_slab.shape[0] != n1 - n0:
        raise ValueError(f"rank {rank}: slab has {w_q_slab.shape[0]} rows, expected {n1 - n0}")
    if n1 > n0:
        C_slab = solver(A, w_q_slab, scale_A, scale_B, scale_C, zero_point_A, zero_point_B,
                        zero_point_C)
    else:
        C_slab = A.new_empty((A.shape[0], 0), dtype=torch.int8)
    return all_gather_columns(C_slab, N, group) if gather else C_slab


def upload_replicated_rows(host: torch.Tensor, dev: torch.Tensor, group=None) -> torch.Tensor:
    """Fill the replicated device matrix `dev` [M, K] on every rank from identical HOST copies
    `host` [M, K] (pinned for full speed) with each rank carrying only 1/world of the rows over
    its own PCIe link: rank r uploads rows [r*M/g, (r+1)*M/g) and an NCCL all-gather over
    NVLink delivers every rank's rows to all.  The whole job then moves M*K bytes
    host->device once, as a single GPU would, instead of once per rank.  Needs M % world == 0
    (otherwise every rank uploads everything).  Asynchronous on the current stream."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    M = host.shape[0]
    if world == 1 or M % world != 0:
        dev.copy_(host, non_blocking=True)
        return dev
    rank = dist.get_rank(group)
    rows = M // world
    mine = torch.empty((rows,) + tuple(dev.shape[1:]), dtype=dev.dtype, device=dev.device)
    mine.copy_(host[rank * rows:(rank + 1) * rows], non_blocking=True)
    dist.all_gather_into_tensor(dev.view(world * rows, *dev.shape[1:]), mine, group=group)
    return dev


class GatheredOutput:
    """The full row-major C [M, N] of a column-sharded matmul, one copy per GPU of the node,
    allocated from torch symmetric memory so that every rank can store into every copy.

    `mm_int8_allgather` writes this rank's column slab into all copies from inside the matmul's
    epilogue (peer stores over NVLink); after `wait()` every rank's `tensor` holds the whole C.
    No NCCL collective moves data."""

    def __init__(self, M: int, N: int, device: torch.device, group=None, multicast: bool | None = None):
        """`multicast`: use the NVLink multicast (NVLS) mapping of the allocation when the
        platform offers one, so that whole row segments leave each GPU once and NVSwitch
        replicates them (default: yes unless TEXO_NO_MULTICAST=1); without it every copy is
        written with its own peer store."""
        import os

        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 GPUs")
        self.M, self.N = M, N
        self.tensor = symm_mem.empty((M, N), dtype=torch.int8, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        # the tensor may sit at an offset inside the symmetric allocation
        offset = int(self.tensor.data_ptr()) - int(self.handle.buffer_ptrs[self.rank])
        ptrs = [int(p) + offset for p in self.handle.buffer_ptrs]
        self._ptr_array = (ctypes.c_void_p * self.world)(*ptrs)
        if multicast is None:
            multicast = os.environ.get("TEXO_NO_MULTICAST", "0") != "1"
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.multicast_ptr = mc + offset if (multicast and mc and self.world > 1) else 0

    def wait(self) -> None:
        """All ranks' stores into every copy are complete and visible after this returns on
        the current stream (call it on every rank)."""
        self.handle.barrier()


def mm_int8_allgather(A: torch.Tensor, B_slab: torch.Tensor, out: GatheredOutput, scale_A: float,
                      scale_B: float, scale_C: float, zero_point_A: int, zero_point_B: int,
                      zero_point_C: int) -> torch.Tensor:
    """Column-sharded mm_int8 with the gather fused into the kernel: returns out.tensor, complete
    on every rank once out.wait() has run."""
    n0, n1 = column_slab(out.N, out.world, out.rank)
    if tuple(B_slab.shape) != (A.shape[1], n1 - n0) or A.shape[0] != out.M:
        raise ValueError(f"rank {out.rank}: operands do not match the gathered output")
    if not (A.is_cuda and B_slab.is_cuda and A.dtype == torch.int8 and B_slab.dtype == torch.int8
            and A.is_contiguous() and B_slab.is_contiguous()):
        raise ValueError("A and B_slab must be contiguous CUDA int8 tensors")
    if n1 > n0:
        lib = _lib.load()
        with torch.cuda.device(A.device), ops._DefaultStreamOrder(A.device):
            rc = lib.texo_mm_int8_solve_allgather_multicast(
                A.data_ptr(), B_slab.data_ptr(), ctypes.cast(out._ptr_array, ctypes.c_void_p),
                out.multicast_ptr or None, out.world, out.M, n1 - n0, A.shape[1], out.N, n0,
                scale_A, scale_B, scale_C, zero_point_A, zero_point_B, zero_point_C)
        if rc != 0:
            raise RuntimeError("texo_mm_int8_solve_allgather rejected its arguments")
    return out.tensor
