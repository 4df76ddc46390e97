"""Weight-gradient averaging across data-parallel ranks, with two gloo ranks on the CPU: after the
all-reduce every rank holds the mean gradient, so identical replicas stay identical."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from khan_b200.model import activations, nn
    from khan_b200.training.trainer_multi_tower import average_gradients
    model = nn.MoleculeNN(precision=torch.float64, activation_fn=activations.gaussian, device="cpu",
                          seed=7, init="he")                     # same seed: identical replicas
    acs = np.array([20, 9, 4, 3])
    gen = torch.Generator().manual_seed(100 + rank)              # different data per rank
    feats = torch.rand((int(acs.sum()), 384), dtype=torch.float64, generator=gen)
    loss = (model.atom_energies_sorted(feats, acs) ** 2).mean()
    loss.backward()
    local = torch.cat([p.grad.reshape(-1) for p in model.get_parameters()]).clone()
    average_gradients(model.get_parameters())
    avg = torch.cat([p.grad.reshape(-1) for p in model.get_parameters()])
    # the flat-buffer form (what FlatNadam hands over): the buffer itself is reduced in place
    flat = local.clone()
    average_gradients([], flat_grads=flat)
    np.save(os.path.join(out_dir, f"flat{rank}.npy"), flat.numpy())
    np.save(os.path.join(out_dir, f"local{rank}.npy"), local.numpy())
    np.save(os.path.join(out_dir, f"avg{rank}.npy"), avg.numpy())
    dist.destroy_process_group()


def test_two_ranks_end_up_with_the_mean_gradient(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    local = [np.load(tmp_path / f"local{r}.npy") for r in range(world)]
    avg = [np.load(tmp_path / f"avg{r}.npy") for r in range(world)]
    assert local[0].shape == (296452,)
    assert np.abs(local[0] - local[1]).max() > 0
    np.testing.assert_allclose(avg[0], (local[0] + local[1]) / 2, rtol=1e-12, atol=1e-15)
    np.testing.assert_array_equal(avg[0], avg[1])
    flat = [np.load(tmp_path / f"flat{r}.npy") for r in range(world)]
    np.testing.assert_array_equal(flat[0], avg[0])
    np.testing.assert_array_equal(flat[1], avg[0])
