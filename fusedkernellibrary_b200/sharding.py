"""Plane sharding across the GPUs of one box.

Every output plane depends only on its own descriptor and one source image (the reference
indexes opData[thread.z] and nothing else, operation_model/batch_operations.h:153-160), so a
batch splits by plane with no exchange step.  One process drives one GPU; a rank builds and
launches a plan over its own planes only.
"""
from __future__ import annotations


def plane_range(n_planes: int, world: int, rank: int, available=None) -> tuple[int, int]:
    """Contiguous [first, first+count) of rank `rank` (the library's fkb_assign_planes): sizes differ by at
    most one plane, and the ranges of ranks 0..world-1 tile [0, n_planes) in order, so that each rank's
    outputs form one contiguous slab of a consolidated tensor.  Ranks whose `available` entry is false get
    no planes; theirs go to the others."""
    if world <= 0 or not (0 <= rank < world) or n_planes < 0:
        raise ValueError("bad sharding arguments")
    from . import abi
    return abi.assign_planes(n_planes, world, available)[rank]


def interleaved_planes(n_planes: int, world: int, rank: int) -> list[int]:
    """Planes rank, rank+world, ...: with source image = plane index mod n_images this keeps only
    n_images / world distinct images on a GPU when world divides n_images."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad sharding arguments")
    return list(range(rank, n_planes, world))


def max_over_ranks(value: float) -> float:
    """Largest `value` of any rank (the timing rule for every multi-GPU number); identity when no
    process group is initialised."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
