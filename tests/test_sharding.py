"""Data-parallel host logic: molecule sharding and the max-over-ranks reduction, exercised with
two gloo ranks on the CPU.  The shards are featurized with the CPU oracle (this is a test) and
must reassemble to exactly the single-process result."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT
from khan_b200.data import sharding, synthetic as syn


def test_shard_bounds_cover_everything_once():
    rng = np.random.default_rng(0)
    for n_mols in (0, 1, 2, 7, 64, 1000):
        counts = rng.integers(1, 27, n_mols)
        for world in (1, 2, 3, 8):
            bounds = sharding.shard_bounds(counts, world)
            assert len(bounds) == world
            assert bounds[0][0] == 0 and bounds[-1][1] == n_mols
            for (a0, a1), (b0, b1) in zip(bounds, bounds[1:]):
                assert a1 == b0 and a0 <= a1
            if n_mols >= 8 * world:
                atoms = [counts[s:e].sum() for s, e in bounds]
                assert max(atoms) - min(atoms) <= 2 * counts.max()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    batch = syn.config1(n_mols=48)
    shard = sharding.shard_batch(batch, rank, world)
    si, gi, ac = oracle.ani_sort(shard.atomic_numbers)   # each rank sorts its own shard
    x, y, z = shard.coords(np.float64)
    feats = oracle.featurize(x, y, z, shard.atomic_numbers, shard.mol_offsets,
                             shard.mol_atom_counts, si, ac)
    rows = np.concatenate([f.reshape(-1, 384) for f in feats])[gi]   # back to atom order
    np.save(os.path.join(out_dir, f"rows{rank}.npy"), rows)
    # step-time reduction used by the benchmark: max over ranks, units summed over ranks
    t = sharding.max_over_ranks(10.0 + rank)
    units = sharding.sum_over_ranks(float(shard.n_atoms))
    np.save(os.path.join(out_dir, f"red{rank}.npy"), np.array([t, units]))
    dist.destroy_process_group()


def test_two_gloo_ranks_reassemble_the_single_process_result(tmp_path, oracle_mod):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    batch = syn.config1(n_mols=48)
    si, gi, ac = oracle_mod.ani_sort(batch.atomic_numbers)
    x, y, z = batch.coords(np.float64)
    feats = oracle_mod.featurize(x, y, z, batch.atomic_numbers, batch.mol_offsets,
                                 batch.mol_atom_counts, si, ac)
    full = np.concatenate([f.reshape(-1, 384) for f in feats])[gi]
    parts = np.concatenate([np.load(tmp_path / f"rows{r}.npy") for r in range(world)])
    np.testing.assert_array_equal(parts, full)
    for r in range(world):
        t, units = np.load(tmp_path / f"red{r}.npy")
        assert t == 11.0 and units == batch.n_atoms
