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
        # every pointer of a launch must belong to the launching GPU (no peer access is ever enabled)
        _lib.same_device(self.device, *model.get_parameters(), optimizer.flat_params, optimizer.flat_grads,
                         where="FusedTrainStep")
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
        self._args_key = self._args = None
        for ann in model.anns:       # the weight gradients are added straight into the flat buffer
            for p in list(ann.Ws) + list(ann.bs):
                if p.grad is None or p.grad.data_ptr() % 4:
                    raise ValueError("parameters must have gradient buffers (FlatNadam provides them)")

    def _check(self, sb: StagedBatch) -> None:
        if sb.n_atoms > self.n_atoms_cap or sb.n_mols > self.n_mols_cap or sb.dtype != torch.float32:
            raise ValueError("batch does not fit this step")
        _lib.same_device(self.device, sb.features, sb.x, where="FusedTrainStep")

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _network_args(self, sb: StagedBatch, feature_grad: bool, packed=None):
        """The three argument blocks of the atomic-network kernels for this batch (the blocks of
        the last batch are kept: a step asks for them twice)."""
        acs = sb.acs_host
        w_first = self.model.anns[0].Ws[0]
        key = (id(sb), int(acs[0]), int(acs[1]), int(acs[2]), int(acs[3]), feature_grad,
               None if packed is None else packed.data_ptr(), w_first.data_ptr(), w_first.grad.data_ptr(),
               sb.features.data_ptr(), sb.upstream.data_ptr())
        if self._args_key == key:
            return self._args
        starts = np.concatenate([[0], np.cumsum(acs)])
        fwd, bwd, wg = _lib.MlpArgs(), _lib.MlpBackwardArgs(), _lib.MlpWeightGradArgs()
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
        self._args_key, self._args = key, (fwd, bwd, wg)
        return self._args

    # The step in four phases, each on the CURRENT stream of the device.  ``featurize`` of a batch
    # depends on nothing but its coordinates, so a caller may run it for the NEXT batch beside the
    # network kernels of this one; ``coordinate_gradient`` and ``weight_gradients`` both depend on
    # ``networks`` only and may run side by side (see StepPipeline).

    def featurize(self, sb: StagedBatch) -> None:
        """ani_sort + featurize: ``sb.features`` (element-sorted rows) and the sort indices."""
        self._check(sb)
        stream = self._stream()
        sb.run_sort(stream)
        sb.run_featurize(stream)

    def featurize_pass(self, sb: StagedBatch) -> None:
        """The same as ``featurize`` through the one-call entry point (one argument block, one call)."""
        self._check(sb)
        a = self._pass_args(sb)
        a.phases = _lib.PASS_FEATURIZE
        _lib.check(_lib.lib().ani_network_pass_f32(ctypes.byref(a), self._stream()), "ani_network_pass_f32")

    def networks(self, sb: StagedBatch, labels: torch.Tensor, feature_grad: bool = True) -> None:
        """Weight packing, networks forward, molecule energies + MSE gradient, networks backward.
        Afterwards ``self.l2s[:n_mols]`` holds the squared errors, the dz buffers the layer
        gradients and, unless ``feature_grad`` is False (energy-only training: the three products
        towards the features are skipped), ``sb.upstream`` dLoss/dfeatures."""
        self._check(sb)
        stream = self._stream()
        lib = _lib.lib()
        fwd, bwd, _ = self._network_args(sb, feature_grad, self.model.pack_weights(stream))
        _lib.check(lib.ani_mlp_forward_f32(ctypes.byref(fwd), sb._acs_ptr, self.act_id, int(self.split), stream),
                   "ani_mlp_forward_f32")
        _lib.check(lib.ani_molecule_energy_f32(_ptr(self.energy_sorted), _ptr(sb.gather), _ptr(sb.mol_offsets),
                                               _ptr(sb.mol_counts), sb.n_mols, sb.n_atoms, _ptr(labels),
                                               1.0 / max(sb.n_mols, 1), _ptr(self.mol_energy), _ptr(self.l2s),
                                               _ptr(self.grad_energy_sorted), stream), "ani_molecule_energy_f32")
        _lib.check(lib.ani_mlp_backward_f32(ctypes.byref(bwd), sb._acs_ptr, int(self.split), stream),
                   "ani_mlp_backward_f32")

    def weight_gradients(self, sb: StagedBatch) -> None:
        """Zeroes the flat gradient buffer and adds the weight gradients of this batch to it."""
        stream = self._stream()
        if self._args_key is not None and self._args_key[0] == id(sb) and self._args_key[1:5] == tuple(int(c) for c in sb.acs_host):
            wg = self._args[2]          # the blocks networks() built for this batch
        else:
            wg = self._network_args(sb, True)[2]
        self.optimizer.flat_grads.zero_()
        _lib.check(_lib.lib().ani_mlp_weight_grad_f32(ctypes.byref(wg), sb._acs_ptr, int(self.split), stream),
                   "ani_mlp_weight_grad_f32")

    def _pass_args(self, sb: StagedBatch):
        """Argument block of ``ani_network_pass_f32``; the fields that do not depend on the batch are filled
        once (and again when the weights or their gradient buffers have moved)."""
        first = self.model.anns[0].Ws[0]
        packed = self.model.packed_weights()
        key = (first.data_ptr(), first.grad.data_ptr(), None if packed is None else packed.data_ptr())
        if getattr(self, "_pa_key", None) != key:
            a = _lib.PassArgs()
            a.activation, a.split_precision = self.act_id, int(self.split)
            a.energy_sorted, a.grad_energy_sorted = self.energy_sorted.data_ptr(), self.grad_energy_sorted.data_ptr()
            for name, bufs in (("act", self.acts), ("dact", self.dacts), ("dz", self.dzs)):
                for k, t in enumerate(bufs):
                    setattr(a, f"{name}{k + 1}", t.data_ptr())
            a.mol_energy, a.l2s = self.mol_energy.data_ptr(), self.l2s.data_ptr()
            for t, ann in enumerate(self.model.anns):
                for k, (w, b) in enumerate(zip(ann.Ws, ann.bs)):
                    getattr(a, f"w{k + 1}")[t], getattr(a, f"b{k + 1}")[t] = w.data_ptr(), b.data_ptr()
                    getattr(a, f"dw{k + 1}")[t], getattr(a, f"db{k + 1}")[t] = w.grad.data_ptr(), b.grad.data_ptr()
                if packed is not None:
                    a.packed[t] = packed[t].data_ptr()
            a.zero_ptr = self.optimizer.flat_grads.data_ptr()
            a.zero_bytes = self.optimizer.flat_grads.numel() * 4
            self._pa, self._pa_key = a, key
        a = self._pa
        a.n_atoms, a.n_mols, a.acs_host = sb.n_atoms, sb.n_mols, sb.acs_host.ctypes.data
        a.xs, a.ys, a.zs = sb.x.data_ptr(), sb.y.data_ptr(), sb.z.data_ptr()
        a.atomic_numbers, a.mol_offsets, a.mol_atom_counts = (sb.types.data_ptr(), sb.mol_offsets.data_ptr(),
                                                              sb.mol_counts.data_ptr())
        a.scatter_idxs, a.gather_idxs, a.atom_counts = sb.scatter.data_ptr(), sb.gather.data_ptr(), sb.counts.data_ptr()
        a.features = sb.features.data_ptr()
        return a

    def forward_backward(self, sb: StagedBatch, labels: torch.Tensor, feature_grad: bool = True,
                         featurized: bool = False) -> None:
        """Everything up to the weight gradients, in order on the current stream: weight packing, sort,
        featurize, networks forward, molecule energies + MSE gradient, networks backward, zero + weight
        gradients -- one C-ABI call (``ani_network_pass_f32``).  ``featurized``: sort + featurize of this
        batch have been done already (``featurize``, say on another stream beside the previous batch's
        networks) and are left out."""
        self._check(sb)
        stream = self._stream()
        if self.model.packed_weights() is None:
            self.model.pack_weights(stream)          # allocates the packed copy (first use)
        a = self._pass_args(sb)
        a.feature_grads = sb.upstream.data_ptr() if feature_grad else None
        a.labels, a.grad_scale = labels.data_ptr(), 1.0 / max(sb.n_mols, 1)
        a.phases = (_lib.PASS_PACK | (0 if featurized else _lib.PASS_FEATURIZE) | _lib.PASS_FORWARD | _lib.PASS_ENERGY
                    | _lib.PASS_BACKWARD | _lib.PASS_WEIGHT_GRAD)
        _lib.check(_lib.lib().ani_network_pass_f32(ctypes.byref(a), stream), "ani_network_pass_f32")
        self._args_key = None      # the per-phase argument blocks (networks / weight_gradients) are stale now

    def coordinate_gradient(self, sb: StagedBatch) -> None:
        """dLoss/dx, dy, dz into ``sb.grads`` (featurize_grad with ``sb.upstream`` as its upstream)."""
        sb.run_featurize_grad(self._stream())

    def step(self, sb: StagedBatch, labels: torch.Tensor) -> None:
        """The whole step, eagerly, on the current stream (no overlap)."""
        self.forward_backward(sb, labels)
        average_gradients(self.model.get_parameters(), self.optimizer.flat_grads)
        self.coordinate_gradient(sb)
        self.optimizer.step()

    KERNELS = 11   # weight packing, sort, featurize, mlp fwd, molecule energy, mlp bwd, memset, wgrad, featurize_grad, sumsq, nadam


class StepPipeline:
    """Training steps over a pool of resident batches with the independent kernels side by side:

        feature stream    sort + featurize of batch b+1      (needs only its coordinates)
        main stream       networks(b) -> weight gradients(b) -> [all-reduce] -> update
        gradient stream                  coordinate gradient(b)          (needs networks(b) only)

    The network kernels run one 128-atom tile per SM on about three quarters of the SMs, and a
    featurizer CTA fits beside a network CTA, so the side streams use what the network kernels
    leave free (measured on a 1024-molecule batch: networks + featurize 119 us side by side against
    131 us in sequence) and the step needs no launch boundary between its phases.  The sequence of
    weights is the one of the serial step: featurize does not read the weights, and each update
    still waits for everything of its own batch.

    ``prime()`` featurizes batch 0; ``run(k)`` then performs step k on batch ``k % len(staged)``
    and featurizes the batch after it.  With ``graphs`` the phases are captured once per batch
    (one graph per step on a single GPU, and with ``peer`` -- a ``PeerAllReduce`` -- on several: the mean
    of the gradients over the ranks is then a kernel of the library inside the graph; with a library
    all-reduce the collective stays outside the graphs, between the graph that ends with the weight
    gradients and the graph of the update).
    """

    def __init__(self, step: FusedTrainStep, staged, labels, allreduce: bool = False, graphs: bool = True,
                 peer=None):
        if len(staged) < 2 or len(staged) != len(labels):
            raise ValueError("StepPipeline needs at least two resident batches and one label vector per batch")
        self.step, self.staged, self.labels = step, list(staged), list(labels)
        self.allreduce = bool(allreduce)
        # a PeerAllReduce: the mean over the ranks is one kernel of the library and the step stays ONE graph
        self.peer = peer if allreduce else None
        self.nb = len(self.staged)
        dev = step.device
        self.feature_stream = torch.cuda.Stream(device=dev)
        self.gradient_stream = torch.cuda.Stream(device=dev)
        self._whole = self._update = None
        if graphs:
            self._capture()

    def _issue(self, b: int, update: bool) -> None:
        """One step on the current stream with its two side branches forked and joined."""
        step = self.step
        cur = torch.cuda.current_stream(step.device)
        self.feature_stream.wait_stream(cur)
        with torch.cuda.stream(self.feature_stream):
            step.featurize(self.staged[(b + 1) % self.nb])
        step.networks(self.staged[b], self.labels[b])
        # the featurizer joins here: letting it run on into the gradient kernels was measured slower
        cur.wait_stream(self.feature_stream)
        self.gradient_stream.wait_stream(cur)
        with torch.cuda.stream(self.gradient_stream):
            step.coordinate_gradient(self.staged[b])
        step.weight_gradients(self.staged[b])
        if update:       # single GPU, or the mean over the ranks as a kernel of this library
            if self.peer is not None:
                self.peer.mean_(step.optimizer.flat_grads)
            step.optimizer.step()
        cur.wait_stream(self.gradient_stream)

    @staticmethod
    def _graph_of(fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g

    def _capture(self) -> None:
        with torch.cuda.device(self.step.device):
            whole = not self.allreduce or self.peer is not None
            self._whole = [self._graph_of(lambda b=b: self._issue(b, whole)) for b in range(self.nb)]
            if not whole:
                self._update = self._graph_of(self.step.optimizer.step)

    def prime(self) -> None:
        self.step.featurize(self.staged[0])

    def run(self, k: int) -> None:
        b = k % self.nb
        step = self.step
        whole = not self.allreduce or self.peer is not None
        if self._whole is not None:
            self._whole[b].replay()
        else:
            self._issue(b, whole)
        if whole:
            return
        # Several ranks: the collective sits between the weight gradients and the update with nothing
        # beside it.  (Measured on two GPUs: starting the coordinate gradient here instead, under the
        # all-reduce, is slower -- presumably its persistent grid fills every SM and the collective's
        # kernel waits behind it.)
        average_gradients(step.model.get_parameters(), step.optimizer.flat_grads)
        if self._update is not None:
            self._update.replay()
        else:
            step.optimizer.step()
