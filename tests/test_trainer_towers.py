"""One tower per process: the trainer refuses several CUDA devices in one process before it touches
any of them (the reference builds one graph per tower in one process,
khan/training/trainer_multi_tower.py:253-259,290-419; here several GPUs are one rank each), and
the launch helpers refuse a tensor that lives on another device than the launching one."""
import pytest
import torch

from khan_b200 import TrainerMultiGPU, TrainerMultiTower, _lib


def test_two_towers_in_one_process_are_refused_with_directions():
    with pytest.raises(NotImplementedError, match="one process per GPU"):
        TrainerMultiTower(None, ["cuda:0", "cuda:1"])
    with pytest.raises(NotImplementedError, match="torchrun"):
        TrainerMultiGPU(None, n_gpus=2)


def test_same_device_check_names_the_offender():
    a = torch.zeros(3)
    _lib.same_device("cpu", a, None, a)
    with pytest.raises(ValueError, match="launching GPU"):
        _lib.same_device(torch.device("cuda", 1), a, where="unit test")
