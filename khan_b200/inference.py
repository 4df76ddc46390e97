"""Energies and forces of staged batches through the C ABI only (no autograd):

    ani_sort -> featurize -> atomic networks (forward) -> molecule sums (ani_molecule_energy)
             -> atomic networks (backward to the features, dE_mol/dE_atom = 1) -> featurize_grad

which is what the reference evaluates for ``predict`` + ``coordinate_gradients``
(``khan/training/trainer_multi_tower.py:580-614,655-678``: ``tf.gradients(tower_pred, [x, y, z])``),
with every buffer pre-allocated so that a pass can be captured into a CUDA graph.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from .model import activations
from .staged import FEATURE_SIZE, StagedBatch


def _ptr(t: torch.Tensor, offset_elems: int = 0):
    return ctypes.c_void_p(t.data_ptr() + offset_elems * t.element_size())


class EnergyForces:
    """Pre-allocated evaluator for one model (float32, the fused 384-128-128-64-1 networks)."""

    def __init__(self, model, n_atoms: int, n_mols: int, device="cuda:0"):
        if not model.fused:
            raise ValueError("EnergyForces needs the fused float32 384-128-128-64-1 networks")
        self.model = model
        self.device = torch.device(device)
        _lib.same_device(self.device, *model.get_parameters(), where="EnergyForces")
        self.act_id = activations.KERNEL_ID[model.activation_fn]
        self.split = bool(model.split_precision)
        f32 = dict(dtype=torch.float32, device=self.device)
        self.energy_sorted = torch.empty(n_atoms, **f32)
        self.ones = torch.ones(n_atoms, **f32)
        self.acts = [torch.empty((n_atoms, w), **f32) for w in (128, 128, 64)]
        self.dacts = [torch.empty((n_atoms, w), **f32) for w in (128, 128, 64)]
        self.dzs = [torch.empty((n_atoms, w), **f32) for w in (128, 128, 64)]
        self.mol_energy = torch.zeros(n_mols, **f32)
        self.n_atoms_cap, self.n_mols_cap = n_atoms, n_mols

    def _weights(self, t: int):
        ann = self.model.anns[t]
        return [w.detach() for w in ann.Ws], [b.detach() for b in ann.bs]

    def run(self, sb: StagedBatch, stream: ctypes.c_void_p | None = None, pack: bool = True,
            forces: bool = True) -> None:
        """One pass over the batch staged in ``sb``.  Afterwards ``self.mol_energy[:sb.n_mols]``
        holds the molecule energies and ``sb.grads[:, :sb.n_atoms]`` dE/dx, dE/dy, dE/dz (forces are
        their negatives).  ``pack=False`` skips the refresh of the pre-packed weights: for a caller
        that packed them (``model.pack_weights``) after the last change of the weights, e.g. once
        before a series of passes that run side by side on several streams.  ``forces=False`` stops
        after the molecule energies (``predict``)."""
        if sb.n_atoms > self.n_atoms_cap or sb.n_mols > self.n_mols_cap or sb.dtype != torch.float32:
            raise ValueError("batch does not fit this evaluator")
        _lib.same_device(self.device, sb.features, sb.x, where="EnergyForces.run")
        if stream is None:
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        lib = _lib.lib()
        n, acs = sb.n_atoms, sb.acs_host
        starts = np.concatenate([[0], np.cumsum(acs)])
        sb.run_sort(stream)
        sb.run_featurize(stream)
        fwd, bwd = _lib.MlpArgs(), _lib.MlpBackwardArgs()
        packed = self.model.pack_weights(stream) if pack else self.model.packed_weights()
        for t in range(4):
            if acs[t] == 0:
                continue
            s = int(starts[t])
            (w1, w2, w3, w4), (b1, b2, b3, b4) = self._weights(t)
            fwd.features[t] = _ptr(sb.features, s * FEATURE_SIZE)
            fwd.w1[t], fwd.w2[t], fwd.w3[t], fwd.w4[t] = _ptr(w1), _ptr(w2), _ptr(w3), _ptr(w4)
            fwd.b1[t], fwd.b2[t], fwd.b3[t], fwd.b4[t] = _ptr(b1), _ptr(b2), _ptr(b3), _ptr(b4)
            fwd.energy[t] = _ptr(self.energy_sorted, s)
            if packed is not None:
                fwd.packed[t] = bwd.packed[t] = _ptr(packed[t])
            fwd.act1[t], fwd.act2[t], fwd.act3[t] = (_ptr(a, s * a.shape[1]) for a in self.acts)
            fwd.dact1[t], fwd.dact2[t], fwd.dact3[t] = (_ptr(d, s * d.shape[1]) for d in self.dacts)
            bwd.grad_energy[t] = _ptr(self.ones, s)
            bwd.w1[t], bwd.w2[t], bwd.w3[t], bwd.w4[t] = _ptr(w1), _ptr(w2), _ptr(w3), _ptr(w4)
            bwd.dact1[t], bwd.dact2[t], bwd.dact3[t] = (_ptr(d, s * d.shape[1]) for d in self.dacts)
            bwd.dz1[t], bwd.dz2[t], bwd.dz3[t] = (_ptr(z, s * z.shape[1]) for z in self.dzs)
            bwd.grad_features[t] = _ptr(sb.upstream, s * FEATURE_SIZE)   # the upstream of featurize_grad
        _lib.check(lib.ani_mlp_forward_f32(ctypes.byref(fwd), sb._acs_ptr, self.act_id, int(self.split), stream),
                   "ani_mlp_forward_f32")
        _lib.check(lib.ani_molecule_energy_f32(_ptr(self.energy_sorted), _ptr(sb.gather), _ptr(sb.mol_offsets),
                                               _ptr(sb.mol_counts), sb.n_mols, n, None, 0.0,
                                               _ptr(self.mol_energy), None, None, stream), "ani_molecule_energy_f32")
        if not forces:
            return
        _lib.check(lib.ani_mlp_backward_f32(ctypes.byref(bwd), sb._acs_ptr, int(self.split), stream),
                   "ani_mlp_backward_f32")
        sb.run_featurize_grad(stream)

    KERNELS_PER_PASS = 7   # weight packing (unless pack=False), sort, featurize, mlp forward, molecule sums, mlp backward, featurize_grad
