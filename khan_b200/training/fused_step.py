"""``FusedTrainStep``: one data-parallel training step on the C ABI only, no autograd.

    ani_sort -> featurize -> networks forward -> molecule energies + MSE gradient
             -> networks backward (to the features) -> weight gradients (added into the flat buffer)
             -> [all-reduce of the flat gradient buffer  ||  featurize_grad (coordinate gradients)]
             -> fused clip + Nadam + moving average

This is the energy-fitting step of the reference (``khan/training/trainer_multi_tower.py:295-427``
with the mean-squared-error loss of the benchmark configuration) with every buffer pre-allocated,
so that the two compute phases can be captured into CUDA graphs, and with the one exchange of the
step -- the gradient all-reduce -- issued right after the weight gradients, where it overlaps the
coordinate-gradient kernel.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _lib
from ..model import activations
from ..staged import FEATURE_SIZE, StagedBatch
from .optim import FlatNadam
from .trainer_multi_tower import average_gradients


def _ptr(t: torch.Tensor, offset_elems: int = 0):
    return ctypes.c_void_p(t.data_ptr() + offset_elems * t.element_size())


class FusedTrainStep:
    def __init__(self, model, optimizer: FlatNadam, n_atoms: int, n_mols: int, device="cuda:0"):
        if not model.fused:
            raise ValueError("FusedTrainStep needs the fused float32 384-128-128-64-1 networks")
        self.model, self.optimizer = model, optimizer
        self.device = torch.device(device)
        self.act_id = activations.KERNEL_ID[model.activation_fn]
        self.split = bool(model.split_precision)
        f32 = dict(dtype=torch.float32, device=self.device)
        self.energy_sorted = torch.empty(n_atoms, **f32)
        self.grad_energy_sorted = torch.zeros(n_atoms, **f32)
        self.acts = [torch.empty((n_atoms, w), **f32) for w in (128, 128, 64)]
        self.dacts = [torch.empty((n_atoms, w), **f32) for w in (128, 128, 64)]
        self.dzs = [torch.empty((n_atoms, w), **f32) for w in (128, 128, 64)]
        self.mol_energy = torch.zeros(n_mols, **f32)
        self.l2s = torch.zeros(n_mols, **f32)
        self.n_atoms_cap, self.n_mols_cap = n_atoms, n_mols
        for ann in model.anns:       # the weight gradients are added straight into the flat buffer
            for p in list(ann.Ws) + list(ann.bs):
                if p.grad is None or p.grad.data_ptr() % 4:
                    raise ValueError("parameters must have gradient buffers (FlatNadam provides them)")

    def forward_backward(self, sb: StagedBatch, labels: torch.Tensor, stream=None, feature_grad: bool = True) -> None:
        """Everything up to the weight gradients.  Afterwards ``self.l2s[:n_mols]`` holds the squared
        errors, the flat gradient buffer the weight gradients of this batch (it is zeroed here
        first) and, unless ``feature_grad`` is False (energy-only training: the three products
        towards the features are skipped), ``sb.upstream`` dLoss/dfeatures."""
        if sb.n_atoms > self.n_atoms_cap or sb.n_mols > self.n_mols_cap or sb.dtype != torch.float32:
            raise ValueError("batch does not fit this step")
        if stream is None:
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        lib = _lib.lib()
        n, acs = sb.n_atoms, sb.acs_host
        starts = np.concatenate([[0], np.cumsum(acs)])
        sb.run_sort(stream)
        sb.run_featurize(stream)
        fwd, bwd, wg = _lib.MlpArgs(), _lib.MlpBackwardArgs(), _lib.MlpWeightGradArgs()
        packed = self.model.pack_weights(stream)
        for t in range(4):
            if acs[t] == 0:
                continue
            s = int(starts[t])
            ann = self.model.anns[t]
            (w1, w2, w3, w4), (b1, b2, b3, b4) = ann.Ws, ann.bs
            fwd.features[t] = wg.features[t] = _ptr(sb.features, s * FEATURE_SIZE)
            fwd.w1[t] = bwd.w1[t] = _ptr(w1.data)
            fwd.w2[t] = bwd.w2[t] = _ptr(w2.data)
            fwd.w3[t] = bwd.w3[t] = _ptr(w3.data)
            fwd.w4[t] = bwd.w4[t] = _ptr(w4.data)
            fwd.b1[t], fwd.b2[t], fwd.b3[t], fwd.b4[t] = _ptr(b1.data), _ptr(b2.data), _ptr(b3.data), _ptr(b4.data)
            fwd.energy[t] = _ptr(self.energy_sorted, s)
            if packed is not None:
                fwd.packed[t] = bwd.packed[t] = _ptr(packed[t])
            fwd.act1[t], fwd.act2[t], fwd.act3[t] = (_ptr(a, s * a.shape[1]) for a in self.acts)
            wg.act1[t], wg.act2[t], wg.act3[t] = fwd.act1[t], fwd.act2[t], fwd.act3[t]
            fwd.dact1[t], fwd.dact2[t], fwd.dact3[t] = (_ptr(d, s * d.shape[1]) for d in self.dacts)
            bwd.dact1[t], bwd.dact2[t], bwd.dact3[t] = fwd.dact1[t], fwd.dact2[t], fwd.dact3[t]
            bwd.grad_energy[t] = wg.grad_energy[t] = _ptr(self.grad_energy_sorted, s)
            bwd.dz1[t], bwd.dz2[t], bwd.dz3[t] = (_ptr(z, s * z.shape[1]) for z in self.dzs)
            wg.dz1[t], wg.dz2[t], wg.dz3[t] = bwd.dz1[t], bwd.dz2[t], bwd.dz3[t]
            bwd.grad_features[t] = _ptr(sb.upstream, s * FEATURE_SIZE) if feature_grad else None
            wg.dw1[t], wg.dw2[t], wg.dw3[t], wg.dw4[t] = _ptr(w1.grad), _ptr(w2.grad), _ptr(w3.grad), _ptr(w4.grad)
            wg.db1[t], wg.db2[t], wg.db3[t], wg.db4[t] = _ptr(b1.grad), _ptr(b2.grad), _ptr(b3.grad), _ptr(b4.grad)
        _lib.check(lib.ani_mlp_forward_f32(ctypes.byref(fwd), sb._acs_ptr, self.act_id, int(self.split), stream),
                   "ani_mlp_forward_f32")
        _lib.check(lib.ani_molecule_energy_f32(_ptr(self.energy_sorted), _ptr(sb.gather), _ptr(sb.mol_offsets),
                                               _ptr(sb.mol_counts), sb.n_mols, n, _ptr(labels),
                                               1.0 / max(sb.n_mols, 1), _ptr(self.mol_energy), _ptr(self.l2s),
                                               _ptr(self.grad_energy_sorted), stream), "ani_molecule_energy_f32")
        _lib.check(lib.ani_mlp_backward_f32(ctypes.byref(bwd), sb._acs_ptr, int(self.split), stream),
                   "ani_mlp_backward_f32")
        self.optimizer.flat_grads.zero_()
        _lib.check(lib.ani_mlp_weight_grad_f32(ctypes.byref(wg), sb._acs_ptr, int(self.split), stream),
                   "ani_mlp_weight_grad_f32")

    def coordinate_gradient(self, sb: StagedBatch, stream=None) -> None:
        """dLoss/dx, dy, dz into ``sb.grads`` (featurize_grad with ``sb.upstream`` as its upstream)."""
        if stream is None:
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        sb.run_featurize_grad(stream)

    def step(self, sb: StagedBatch, labels: torch.Tensor) -> None:
        """The whole step, eagerly, on the current stream (no overlap)."""
        self.forward_backward(sb, labels)
        average_gradients(self.model.get_parameters(), self.optimizer.flat_grads)
        self.coordinate_gradient(sb)
        self.optimizer.step()

    KERNELS = 12   # weight packing, sort, featurize, mlp fwd, molecule energy, mlp bwd, memset, wgrad, zero3, featurize_grad, sumsq, nadam
