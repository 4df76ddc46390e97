"""Activation functions of the atomic networks (``khan/model/activations.py:62-74`` of the
reference), as torch functions, with the ids the fused CUDA kernel uses."""
import torch


def celu(a, alpha: float = 0.1):
    return torch.where(a >= 0, a, alpha * (torch.exp(torch.clamp(a, max=0.0) / alpha) - 1.0))


def normal(a, mean: float = 0.0, std: float = 1.0):
    return torch.exp(-((a - mean) / std) ** 2 / 2.0)


def gaussian(a):
    return torch.exp(-a * a)


def softplus(a, shift: float = 0.69314718056):
    return torch.nn.functional.softplus(a) - shift


KERNEL_ID = {celu: 0, gaussian: 1, normal: 2, softplus: 3}


def get_fn_by_name(name: str):
    return {"celu": celu, "normal": normal, "gaussian": gaussian, "softplus": softplus}[name]


def get_all_fn_names():
    return ["celu", "normal", "gaussian", "softplus"]
