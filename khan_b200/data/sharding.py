"""Molecule sharding for data-parallel featurization.

Molecules are independent in every op of the path (each loop of the reference is bounded by one
molecule's atom range, ``gpu_featurizer/kernel_cpu.cpp:425-431``), so N GPUs each take a
contiguous range of molecules and run ``ani_sort`` + ``featurize`` + ``featurize_grad`` on their own
shard with no communication -- exactly what each tower of the reference does with the batch it
dequeues (``khan/training/trainer_multi_tower.py:296-320``).
"""
from __future__ import annotations

import numpy as np

from .synthetic import Batch


def shard_bounds(mol_atom_counts, world_size: int):
    """Contiguous molecule ranges ``[(start, stop), ...]``, one per rank, balanced by atom count
    (the cost of a molecule grows with its size).  Every molecule lands in exactly one range;
    ranges may be empty when there are fewer molecules than ranks."""
    counts = np.asarray(mol_atom_counts, dtype=np.int64)
    n = counts.shape[0]
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    prefix = np.concatenate([[0], np.cumsum(counts)])
    total = int(prefix[-1])
    cuts = [0]
    for r in range(1, world_size):
        target = total * r / world_size
        cut = int(np.searchsorted(prefix, target, side="left"))
        cuts.append(min(max(cut, cuts[-1]), n))
    cuts.append(n)
    return [(cuts[r], cuts[r + 1]) for r in range(world_size)]


def shard_batch(batch: Batch, rank: int, world_size: int) -> Batch:
    """The molecules of ``batch`` that belong to ``rank``, as an independent batch."""
    start, stop = shard_bounds(batch.mol_atom_counts, world_size)[rank]
    return batch.slice_mols(start, stop)


def max_over_ranks(value: float, group=None) -> float:
    """Maximum of a per-rank scalar (a step time); identity without a process group."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def sum_over_ranks(value: float, group=None) -> float:
    """Sum of a per-rank scalar (units processed); identity without a process group."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t.item())
