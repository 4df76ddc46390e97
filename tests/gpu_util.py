"""Helpers for the GPU parity tests: run a Batch through the ani_mod ops (which call the C ABI)."""
import numpy as np
import torch

from khan_b200 import ani_mod

DEV = "cuda:0"


def to_dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV)


def gpu_sort(atomic_numbers):
    si, gi, ac = ani_mod.ani_sort(to_dev(atomic_numbers.astype(np.int32)))
    return si.cpu().numpy(), gi.cpu().numpy(), ac.cpu().numpy()


def batch_tensors(batch, dt):
    x, y, z = batch.coords(dt)
    return (to_dev(x), to_dev(y), to_dev(z), to_dev(batch.atomic_numbers), to_dev(batch.mol_offsets),
            to_dev(batch.mol_atom_counts))


def gpu_featurize(batch, dt, si=None, ac=None):
    x, y, z, a, mo, mac = batch_tensors(batch, dt)
    if si is None:
        si_t, gi_t, ac_t = ani_mod.ani_sort(a)
        ac = ac_t.cpu().numpy()
    else:
        si_t = to_dev(si)
    feats = ani_mod.featurize(x, y, z, a, mo, mac, si_t, ac)
    ani_mod.check_device_status("featurize")
    return [f.cpu().numpy() for f in feats]


def gpu_featurize_grad(batch, dt, up, si=None, ac=None):
    x, y, z, a, mo, mac = batch_tensors(batch, dt)
    if si is None:
        si_t, gi_t, ac_t = ani_mod.ani_sort(a)
        ac = ac_t.cpu().numpy()
    else:
        si_t = to_dev(si)
    g = [to_dev(u.astype(dt)) for u in up]
    out = ani_mod.featurize_grad(x, y, z, a, mo, mac, si_t, ac, *g)
    ani_mod.check_device_status("featurize_grad")
    return [o.cpu().numpy() for o in out]
