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

    def _pass_args(self, sb: StagedBatch):
        """The argument block of ``ani_network_pass_f32``: everything that does not change from batch to batch
        is filled once (and again when the model's weights have moved), the batch's own fields per call."""
        first = self.model.anns[0].Ws[0]
        packed = self.model.packed_weights()
        key = (first.data_ptr(), None if packed is None else packed.data_ptr())
        if getattr(self, "_pa_key", None) != key:
            a = _lib.PassArgs()
            a.activation, a.split_precision = self.act_id, int(self.split)
            a.energy_sorted, a.grad_energy_sorted = self.energy_sorted.data_ptr(), self.ones.data_ptr()
            for name, bufs in (("act", self.acts), ("dact", self.dacts), ("dz", self.dzs)):
                for k, t in enumerate(bufs):
                    setattr(a, f"{name}{k + 1}", t.data_ptr())
            a.mol_energy = self.mol_energy.data_ptr()
            for t in range(4):
                (w1, w2, w3, w4), (b1, b2, b3, b4) = self._weights(t)
                for name, v in (("w1", w1), ("w2", w2), ("w3", w3), ("w4", w4), ("b1", b1), ("b2", b2), ("b3", b3),
                                ("b4", b4)):
                    getattr(a, name)[t] = v.data_ptr()
                if packed is not None:
                    a.packed[t] = packed[t].data_ptr()
            self._pa, self._pa_key = a, key
        a = self._pa
        a.n_atoms, a.n_mols, a.acs_host = sb.n_atoms, sb.n_mols, sb.acs_host.ctypes.data
        a.xs, a.ys, a.zs = sb.x.data_ptr(), sb.y.data_ptr(), sb.z.data_ptr()
        a.atomic_numbers, a.mol_offsets, a.mol_atom_counts = (sb.types.data_ptr(), sb.mol_offsets.data_ptr(),
                                                              sb.mol_counts.data_ptr())
        a.scatter_idxs, a.gather_idxs, a.atom_counts = sb.scatter.data_ptr(), sb.gather.data_ptr(), sb.counts.data_ptr()
        a.features, a.feature_grads = sb.features.data_ptr(), sb.upstream.data_ptr()
        g, cap, esz = sb.grads.data_ptr(), sb.n_atoms_cap, sb.grads.element_size()
        a.x_grads, a.y_grads, a.z_grads = g, g + cap * esz, g + 2 * cap * esz
        return a

    def featurize(self, sb: StagedBatch, stream: ctypes.c_void_p | None = None) -> None:
        """Sort + featurize of the batch staged in ``sb`` only (one C-ABI call): they need nothing but the
        coordinates, so a caller may run them for the NEXT batch on another stream beside the network kernels
        of this one and then call ``run(..., featurized=True)``."""
        if sb.n_atoms > self.n_atoms_cap or sb.n_mols > self.n_mols_cap or sb.dtype != torch.float32:
            raise ValueError("batch does not fit this evaluator")
        _lib.same_device(self.device, sb.features, sb.x, where="EnergyForces.featurize")
        if stream is None:
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        a = self._pass_args(sb)
        a.phases = _lib.PASS_FEATURIZE
        _lib.check(_lib.lib().ani_network_pass_f32(ctypes.byref(a), stream), "ani_network_pass_f32")

    def run(self, sb: StagedBatch, stream: ctypes.c_void_p | None = None, pack: bool = True,
            forces: bool = True, featurized: bool = False) -> None:
        """One pass over the batch staged in ``sb`` -- one C-ABI call (``ani_network_pass_f32``).  Afterwards
        ``self.mol_energy[:sb.n_mols]`` holds the molecule energies and ``sb.grads[:, :sb.n_atoms]`` dE/dx,
        dE/dy, dE/dz (forces are their negatives).  ``pack=False`` skips the refresh of the pre-packed
        weights: for a caller that packed them (``model.pack_weights``) after the last change of the
        weights, e.g. once before a series of passes that run side by side on several streams.
        ``forces=False`` stops after the molecule energies (``predict``); ``featurized=True`` leaves sort +
        featurize out (``featurize`` has run for this batch)."""
        if sb.n_atoms > self.n_atoms_cap or sb.n_mols > self.n_mols_cap or sb.dtype != torch.float32:
            raise ValueError("batch does not fit this evaluator")
        _lib.same_device(self.device, sb.features, sb.x, where="EnergyForces.run")
        if stream is None:
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        if self.model.packed_weights() is None:
            self.model.pack_weights(stream)          # allocates the packed copy (first use)
            pack = False
        a = self._pass_args(sb)
        a.phases = ((_lib.PASS_PACK if pack else 0) | (0 if featurized else _lib.PASS_FEATURIZE) | _lib.PASS_FORWARD
                    | _lib.PASS_ENERGY | ((_lib.PASS_BACKWARD | _lib.PASS_COORD_GRAD) if forces else 0))
        _lib.check(_lib.lib().ani_network_pass_f32(ctypes.byref(a), stream), "ani_network_pass_f32")

    KERNELS_PER_PASS = 7   # weight packing (unless pack=False), sort, featurize, mlp forward, molecule sums, mlp backward, featurize_grad
