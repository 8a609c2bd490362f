"""Host-side sharding helpers for the two paths that shard naturally (one process per GPU):

* a large GEMM split along N -- every rank holds all of W and a contiguous block of X rows and
  produces D[:, n0:n1]; the optional output all-gather lands in a [world][M][N/world] buffer
  (contiguous per rank, no strided copy), from which ``assemble_columns`` gives the [M][N] view;
* whole-network inference split along the batch -- no collective at all.

Works with any torch.distributed backend (NCCL over NVLink on GPUs, gloo on CPU in the tests).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """Contiguous [begin, end) of ``total`` items for ``rank``; block sizes are multiples of
    ``multiple`` (except possibly the last rank's) and differ by at most one multiple."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad world / rank")
    units = (total + multiple - 1) // multiple
    base, extra = divmod(units, world)
    begin_u = rank * base + min(rank, extra)
    end_u = begin_u + base + (1 if rank < extra else 0)
    return min(begin_u * multiple, total), min(end_u * multiple, total)


def allgather_columns(local: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather equal-sized column blocks D[:, n0:n1] (shape [M, n]) into [world][M][n]."""
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    # the flat [world*M][n] view is what every backend accepts for the concatenated output
    dist.all_gather_into_tensor(out.view((world * local.shape[0],) + tuple(local.shape[1:])), local.contiguous(),
                                group=group)
    return out


def assemble_columns(gathered: torch.Tensor) -> torch.Tensor:
    """[world][M][n] -> [M][world*n] (a copy; the gathered layout itself needs none)."""
    world, M, n = gathered.shape
    return gathered.permute(1, 0, 2).reshape(M, world * n)


def max_over_ranks(value: float, device, group=None) -> float:
    """Largest ``value`` over the ranks (step times are reported as the slowest rank's)."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t[0])


class SymmetricGather:
    """A [world][M][n] int32 buffer allocated as symmetric memory (the same buffer, peer-mapped, on
    every rank) for the fused all-gather: a rank's GEMM writes its column block into slot ``rank``
    of its own buffer and -- through ``peer_destinations()`` handed to the epilogue as
    ``peer_out`` -- into slot ``rank`` of every other rank's buffer, with plain stores over NVLink
    from the kernel that computes the tile.  ``barrier()`` orders the ranks before anyone reads.
    """

    def __init__(self, M: int, n: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.buffer = symm_mem.empty((self.world, M, n), dtype=torch.int32, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self.slot_bytes = M * n * 4

    def local_slot(self) -> torch.Tensor:
        return self.buffer[self.rank]

    def peer_destinations(self) -> list:
        """Device addresses of slot ``rank`` in every other rank's buffer."""
        ptrs = list(self.handle.buffer_ptrs)
        return [int(ptrs[r]) + self.rank * self.slot_bytes for r in range(self.world) if r != self.rank]

    def barrier(self) -> None:
        self.handle.barrier()
