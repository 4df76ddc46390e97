"""The ``ani_mod`` op surface on torch tensors.

The reference loads ``ani.so`` with ``tf.load_op_library`` and calls
``ani_mod.ani_sort / featurize / featurize_grad / featurize_grad_inverse``
(``khan/training/trainer_multi_tower.py:123-127,305-320,23-91``).  This module exposes the same
op names with the same argument order, on CUDA tensors, each forwarding to one C-ABI entry
point of ``libani_b200.so`` on torch's current stream.  Outputs are allocated here, exactly
as the reference's op shells allocate them from the host-side ``acs``
(``gpu_featurizer/ani_op.cpp:52-73``).

torch is used for device memory and streams only; there is no fallback implementation.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib

FEATURE_SIZE = 384
feature_size = FEATURE_SIZE  # the `feature_size` attr the trainer reads back from the op


def _suffix(t: torch.Tensor) -> str:
    if t.dtype == torch.float32:
        return "f32"
    if t.dtype == torch.float64:
        return "f64"
    raise TypeError(f"featurize supports float32 and float64, got {t.dtype}")


def _dev(t: torch.Tensor, dtype=None, name: str = "tensor") -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (khan_b200 has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def _p(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr() if t is not None and t.numel() else 0)


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def host_counts(acs) -> np.ndarray:
    """``acs`` as a host int32[4] array (a device tensor costs one synchronising copy)."""
    if isinstance(acs, torch.Tensor):
        acs = acs.detach().cpu().numpy()
    out = np.ascontiguousarray(np.asarray(acs, dtype=np.int32).reshape(4))
    return out


def _acs_ptr(acs: np.ndarray):
    return acs.ctypes.data_as(_lib.c_int_p)


def ani_sort(atomic_numbers: torch.Tensor):
    """AniSort: returns ``(scatter_idxs, gather_idxs, atom_counts)`` as int32 CUDA tensors."""
    a = _dev(atomic_numbers, torch.int32, "atomic_numbers")
    n = a.numel()
    with torch.cuda.device(a.device):
        scatter = torch.empty(n, dtype=torch.int32, device=a.device)
        gather = torch.empty(n, dtype=torch.int32, device=a.device)
        counts = torch.empty(4, dtype=torch.int32, device=a.device)
        _lib.check(_lib.lib().ani_sort(_p(a), n, _p(scatter), _p(gather), _p(counts), _stream()),
                   "ani_sort")
    return scatter, gather, counts


def _common(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs):
    xs = _dev(xs, None, "xs")
    dt = xs.dtype
    ys, zs = _dev(ys, dt, "ys"), _dev(zs, dt, "zs")
    a = _dev(atomic_numbers, torch.int32, "atomic_numbers")
    mo = _dev(mol_offsets, torch.int32, "mol_offsets")
    mac = _dev(mol_atom_counts, torch.int32, "mol_atom_counts")
    si = _dev(scatter_idxs, torch.int32, "scatter_idxs")
    return xs, ys, zs, a, mo, mac, si


def featurize_into(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs,
                   acs_host: np.ndarray, out: torch.Tensor):
    """Featurize into a caller-owned ``[n_atoms, 384]`` buffer laid out H rows, C rows, N rows,
    O rows (the element-sorted order ``gather_idxs`` indexes).  No allocation, no sync."""
    xs, ys, zs, a, mo, mac, si = _common(xs, ys, zs, atomic_numbers, mol_offsets,
                                         mol_atom_counts, scatter_idxs)
    suf = _suffix(xs)
    starts = np.concatenate([[0], np.cumsum(acs_host)])[:4] * FEATURE_SIZE
    flat = out.view(-1)
    ptrs = [ctypes.c_void_p(flat.data_ptr() + int(s) * flat.element_size()) for s in starts]
    with torch.cuda.device(xs.device):
        fn = getattr(_lib.lib(), "ani_featurize_" + suf)
        _lib.check(fn(_p(xs), _p(ys), _p(zs), _p(a), _p(mo), _p(mac), mo.numel(), _p(si), *ptrs,
                      _acs_ptr(acs_host), _stream()), "ani_featurize_" + suf)
    return out


def featurize(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs, acs):
    """Featurize: returns four flat tensors ``h, c, n, o`` of ``acs[t] * 384`` values
    (views of one allocation; reshape each to ``(-1, 384)`` as the reference trainer does,
    ``khan/training/trainer_multi_tower.py:324-327``)."""
    acs_host = host_counts(acs)
    n_atoms = int(acs_host.sum())
    out = torch.empty((n_atoms, FEATURE_SIZE), dtype=xs.dtype, device=xs.device)
    featurize_into(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs,
                   acs_host, out)
    flat = out.view(-1)
    ends = np.cumsum(acs_host) * FEATURE_SIZE
    starts = ends - acs_host * FEATURE_SIZE
    return tuple(flat[int(s):int(e)] for s, e in zip(starts, ends))


def featurize_grad(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs, acs,
                   h_grads, c_grads, n_grads, o_grads):
    """FeaturizeGrad: returns ``x_grads, y_grads, z_grads`` (``[n_atoms]`` each).

    The arrays start as zeros, so an atom that no molecule range covers gets a zero gradient, as
    in the reference (gpu_featurizer/functor_op_cpu.cpp:70-72); the C entry point itself writes
    only the atoms of the molecules it is given."""
    xs, ys, zs, a, mo, mac, si = _common(xs, ys, zs, atomic_numbers, mol_offsets,
                                         mol_atom_counts, scatter_idxs)
    suf = _suffix(xs)
    acs_host = host_counts(acs)
    n_atoms = int(acs_host.sum())
    gs = []
    for t, g in enumerate((h_grads, c_grads, n_grads, o_grads)):
        g = _dev(g, xs.dtype, "grads").view(-1)
        if g.numel() != int(acs_host[t]) * FEATURE_SIZE:
            raise ValueError(f"upstream gradient {t} has {g.numel()} values, expected "
                             f"{int(acs_host[t]) * FEATURE_SIZE}")
        gs.append(g)
    with torch.cuda.device(xs.device):
        outs = torch.zeros((3, n_atoms), dtype=xs.dtype, device=xs.device)
        fn = getattr(_lib.lib(), "ani_featurize_grad_" + suf)
        _lib.check(fn(_p(xs), _p(ys), _p(zs), _p(a), _p(mo), _p(mac), mo.numel(), _p(si),
                      *[_p(g) for g in gs], _p(outs[0]), _p(outs[1]), _p(outs[2]),
                      _acs_ptr(acs_host), _stream()), "ani_featurize_grad_" + suf)
    return outs[0], outs[1], outs[2]


def featurize_grad_inverse(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs,
                           acs, x_grads, y_grads, z_grads):
    """FeaturizeGradInverse: Jacobian-vector product; returns four flat tensors like
    :func:`featurize` (the transpose of :func:`featurize_grad`)."""
    xs, ys, zs, a, mo, mac, si = _common(xs, ys, zs, atomic_numbers, mol_offsets,
                                         mol_atom_counts, scatter_idxs)
    suf = _suffix(xs)
    acs_host = host_counts(acs)
    n_atoms = int(acs_host.sum())
    vs = [_dev(v, xs.dtype, "grads").view(-1) for v in (x_grads, y_grads, z_grads)]
    for v in vs:
        if v.numel() != n_atoms:
            raise ValueError(f"coordinate vector has {v.numel()} values, expected {n_atoms}")
    out = torch.empty((n_atoms, FEATURE_SIZE), dtype=xs.dtype, device=xs.device)
    flat = out.view(-1)
    ends = np.cumsum(acs_host) * FEATURE_SIZE
    starts = ends - acs_host * FEATURE_SIZE
    ptrs = [ctypes.c_void_p(flat.data_ptr() + int(s) * flat.element_size()) for s in starts]
    with torch.cuda.device(xs.device):
        fn = getattr(_lib.lib(), "ani_featurize_grad_inverse_" + suf)
        _lib.check(fn(_p(xs), _p(ys), _p(zs), _p(a), _p(mo), _p(mac), mo.numel(), _p(si),
                      *[_p(v) for v in vs], *ptrs, _acs_ptr(acs_host), _stream()),
                   "ani_featurize_grad_inverse_" + suf)
    return tuple(flat[int(s):int(e)] for s, e in zip(starts, ends))


def featurize_sorted(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs, acs):
    """Featurize into one ``[n_atoms, 384]`` tensor laid out H rows, C rows, N rows, O rows (the
    order ``gather_idxs`` indexes; the four outputs of :func:`featurize` are its slices)."""
    acs_host = host_counts(acs)
    out = torch.empty((int(acs_host.sum()), FEATURE_SIZE), dtype=xs.dtype, device=xs.device)
    return featurize_into(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs,
                          acs_host, out)


def _split(buf, acs_host):
    flat = buf.reshape(-1)
    ends = np.cumsum(acs_host) * FEATURE_SIZE
    starts = ends - acs_host * FEATURE_SIZE
    return [flat[int(s):int(e)] for s, e in zip(starts, ends)]


class _FeaturizeSorted(torch.autograd.Function):
    """Featurize with the gradient wiring of the reference trainer: d/d(x, y, z) through
    FeaturizeGrad (``khan/training/trainer_multi_tower.py:23-52``) and, one level up, through
    FeaturizeGradInverse (``:64-91``)."""

    @staticmethod
    def forward(ctx, xs, ys, zs, a, mo, mac, si, acs):
        acs = host_counts(acs)
        ctx.save_for_backward(xs, ys, zs, a, mo, mac, si)
        ctx.acs = acs
        return featurize_sorted(xs, ys, zs, a, mo, mac, si, acs)

    @staticmethod
    def backward(ctx, grad_buf):
        xs, ys, zs, a, mo, mac, si = ctx.saved_tensors
        gx, gy, gz = _FeaturizeGradSorted.apply(xs, ys, zs, a, mo, mac, si, ctx.acs, grad_buf)
        return gx, gy, gz, None, None, None, None, None


class _FeaturizeGradSorted(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xs, ys, zs, a, mo, mac, si, acs, grad_buf):
        ctx.save_for_backward(xs, ys, zs, a, mo, mac, si)
        ctx.acs = acs
        return featurize_grad(xs, ys, zs, a, mo, mac, si, acs, *_split(grad_buf.contiguous(), acs))

    @staticmethod
    def backward(ctx, vx, vy, vz):
        xs, ys, zs, a, mo, mac, si = ctx.saved_tensors
        vx, vy, vz = (v if v is not None else torch.zeros_like(xs) for v in (vx, vy, vz))
        parts = featurize_grad_inverse(xs, ys, zs, a, mo, mac, si, ctx.acs, vx, vy, vz)
        # the four parts are consecutive slices of one buffer; gradients with respect to the
        # coordinates themselves (third-order terms) are not provided, as in the reference
        # (it returns None for the first eight inputs)
        n = int(ctx.acs.sum())
        buf = torch.cat(parts).view(n, FEATURE_SIZE) if n else parts[0].view(0, FEATURE_SIZE)
        return (None,) * 8 + (buf,)


def featurize_sorted_autograd(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts,
                              scatter_idxs, acs):
    """:func:`featurize_sorted` that torch.autograd can differentiate with respect to xs, ys, zs."""
    return _FeaturizeSorted.apply(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts,
                                  scatter_idxs, acs)


def featurize_autograd(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs, acs):
    """:func:`featurize` (four flat outputs) that torch.autograd can differentiate."""
    acs_host = host_counts(acs)
    buf = featurize_sorted_autograd(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts,
                                    scatter_idxs, acs_host)
    return tuple(_split(buf, acs_host))


def ani_charge(xs, ys, zs, qs, mol_offsets, mol_atom_counts):
    """``ani_mod.ani_charge`` (gpu_featurizer/ani_charges.cpp:45-113): damped Coulomb energy of
    every molecule from per-atom partial charges ``qs``; returns ``[n_mols]``."""
    xs = _dev(xs, name="xs")
    suf = _suffix(xs)
    ys, zs, qs = _dev(ys, xs.dtype, "ys"), _dev(zs, xs.dtype, "zs"), _dev(qs, xs.dtype, "qs")
    mo, mac = _dev(mol_offsets, torch.int32, "mol_offsets"), _dev(mol_atom_counts, torch.int32, "mol_atom_counts")
    out = torch.empty(mo.numel(), dtype=xs.dtype, device=xs.device)
    with torch.cuda.device(xs.device):
        _lib.check(getattr(_lib.lib(), "ani_charge_" + suf)(
            _p(xs), _p(ys), _p(zs), _p(qs), _p(mo), _p(mac), mo.numel(), xs.numel(), _p(out), _stream()),
            "ani_charge_" + suf)
    return out


def ani_charge_grad(xs, ys, zs, qs, mol_offsets, mol_atom_counts, grads):
    """``ani_mod.ani_charge_grad`` (gpu_featurizer/ani_charges.cpp:123-214): gradient with respect
    to the charges given ``grads = dL/d(charge_energies)``; returns ``[n_atoms]``."""
    xs = _dev(xs, name="xs")
    suf = _suffix(xs)
    ys, zs, qs = _dev(ys, xs.dtype, "ys"), _dev(zs, xs.dtype, "zs"), _dev(qs, xs.dtype, "qs")
    grads = _dev(grads, xs.dtype, "grads")
    mo, mac = _dev(mol_offsets, torch.int32, "mol_offsets"), _dev(mol_atom_counts, torch.int32, "mol_atom_counts")
    if grads.numel() != mo.numel():
        raise ValueError("grads must hold one value per molecule")
    out = torch.empty(xs.numel(), dtype=xs.dtype, device=xs.device)
    with torch.cuda.device(xs.device):
        _lib.check(getattr(_lib.lib(), "ani_charge_grad_" + suf)(
            _p(xs), _p(ys), _p(zs), _p(qs), _p(mo), _p(mac), mo.numel(), xs.numel(), _p(grads), _p(out),
            _stream()), "ani_charge_grad_" + suf)
    return out


class _AniCharge(torch.autograd.Function):
    """ani_charge with the gradient the reference registers for it: with respect to the
    charges only (khan/training/trainer_multi_tower.py:94-120)."""

    @staticmethod
    def forward(ctx, xs, ys, zs, qs, mo, mac):
        ctx.save_for_backward(xs, ys, zs, qs, mo, mac)
        return ani_charge(xs, ys, zs, qs, mo, mac)

    @staticmethod
    def backward(ctx, grads):
        xs, ys, zs, qs, mo, mac = ctx.saved_tensors
        return None, None, None, ani_charge_grad(xs, ys, zs, qs, mo, mac, grads.contiguous()), None, None


def ani_charge_autograd(xs, ys, zs, qs, mol_offsets, mol_atom_counts):
    """ani_charge that torch.autograd can differentiate with respect to ``qs``."""
    return _AniCharge.apply(xs, ys, zs, qs, mol_offsets, mol_atom_counts)


def device_status() -> int:
    """Synchronise the current stream and return (and clear) the device status word."""
    return int(_lib.lib().ani_device_status(_stream()))


def check_device_status(where: str = "ani kernels") -> None:
    _lib.check(device_status(), where)
