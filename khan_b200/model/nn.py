"""Atomic and molecular networks: the model side of khan (``khan/model/nn.py`` of the reference).

``AtomNN`` is one dense stack per element, ``A = act(A W + b)`` with a linear last layer of width
one; ``MoleculeNN`` holds one ``AtomNN`` per element, evaluates each on the feature rows of its
element and brings the atomic energies back to atom order with ``gather_idxs``
(``khan/model/nn.py:39-67,165-172``).  Parameters keep the reference's shapes and names
(``W`` is ``(in, out)``, names like ``near_W_H_384x128_l1``) so that its ``.npz`` checkpoints map
one to one.

For float32 and the architecture 384-128-128-64-1 the forward pass of all four networks is one
fused tensor-core kernel (``ani_mlp_forward_f32``); its backward pass and every other
architecture or precision use torch's dense GEMMs on the GPU.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _lib
from . import activations

FUSED_LAYERS = (384, 128, 128, 64, 1)
TYPE_MAP = ["H", "C", "N", "O"]


class AtomNN:
    """Dense stack for the atoms of one element."""

    def __init__(self, layer_sizes, precision=torch.float32, activation_fn=activations.celu,
                 atom_type: str = "", prefix: str = "", device="cuda", generator=None,
                 init: str = "reference"):
        assert precision in (torch.float32, torch.float64)
        assert layer_sizes[-1] == 1
        self.layer_sizes = tuple(int(v) for v in layer_sizes)
        self.precision = precision
        self.activation_fn = activation_fn
        self.atom_type = atom_type
        self.Ws, self.bs, self.names = [], [], []
        for idx in range(1, len(layer_sizes)):
            x, y = layer_sizes[idx - 1], layer_sizes[idx]
            # reference: N(0, sqrt(2 / (x + y))), khan/model/nn.py:45-59; "he": N(0, sqrt(2 / x))
            std = (2.0 / (x + y)) ** 0.5 if init == "reference" else (2.0 / x) ** 0.5
            w = torch.randn((x, y), dtype=torch.float64, generator=generator) * std
            name = "_" + atom_type + "_" + str(x) + "x" + str(y) + "_l" + str(idx)
            self.Ws.append(w.to(precision).to(device).requires_grad_(True))
            self.bs.append(torch.zeros(y, dtype=precision, device=device, requires_grad=True))
            self.names.append((prefix + "W" + name, prefix + "b" + name))

    def get_parameters(self):
        return self.Ws + self.bs

    def named_parameters(self):
        out = {}
        for (wn, bn), w, b in zip(self.names, self.Ws, self.bs):
            out[wn + ":0"] = w
            out[bn + ":0"] = b
        return out

    def atom_energies(self, features: torch.Tensor) -> torch.Tensor:
        """Energies ``(n,)`` of the feature rows ``(n, layer_sizes[0])`` (dense torch path)."""
        a = features
        last = len(self.Ws) - 1
        for k, (w, b) in enumerate(zip(self.Ws, self.bs)):
            a = a @ w + b
            if k != last:
                a = self.activation_fn(a)
        return a.reshape(-1)


def _dense_energies(features, acs, act_fn, params):
    """The four networks in plain differentiable torch ops (element-sorted rows in and out)."""
    starts = np.concatenate([[0], np.cumsum(acs)])
    parts = []
    for t in range(4):
        a = features[int(starts[t]):int(starts[t + 1])]
        w1, b1, w2, b2, w3, b3, w4, b4 = params[8 * t: 8 * t + 8]
        a = act_fn(a @ w1 + b1)
        a = act_fn(a @ w2 + b2)
        a = act_fn(a @ w3 + b3)
        parts.append((a @ w4 + b4).reshape(-1))
    return torch.cat(parts)


class _FusedMlp(torch.autograd.Function):
    """The four atomic networks on the tensor-core kernels: one launch forward
    (``ani_mlp_forward_f32``), one launch for the backward pass along the activations
    (``ani_mlp_backward_f32``: dz1, dz2, dz3 and the feature gradient); the weight gradients are
    the plain products ``A_{l-1}^T dz_l`` over the atoms of each element.  When the backward pass
    itself has to be differentiated (force training, ``create_graph=True``) it is evaluated in
    dense differentiable torch ops instead."""

    @staticmethod
    def forward(ctx, features, acs, act_id, split, act_and_packed, *params):
        act_fn, packed = act_and_packed
        # params: for each of the 4 elements W1,b1,W2,b2,W3,b3,W4,b4 (reference shapes, W = (in, out))
        n = features.shape[0]
        dev = features.device
        _lib.same_device(dev, *params, packed, where="atomic networks (forward)")
        starts = np.concatenate([[0], np.cumsum(acs)])
        f32 = dict(dtype=torch.float32, device=dev)
        energy = torch.empty(n, **f32)
        acts = [torch.empty((n, 128), **f32), torch.empty((n, 128), **f32), torch.empty((n, 64), **f32)]
        dacts = [torch.empty((n, 128), **f32), torch.empty((n, 128), **f32), torch.empty((n, 64), **f32)]
        args = _lib.MlpArgs()
        keep = []
        for t in range(4):
            w1, b1, w2, b2, w3, b3, w4, b4 = params[8 * t: 8 * t + 8]
            tr = [w1.detach().contiguous(), w2.detach().contiguous(), w3.detach().contiguous(),
                  w4.detach().reshape(-1).contiguous()]      # no copies: the kernel reads [in][out]
            keep.extend(tr)
            s = int(starts[t])
            cnt = int(acs[t])

            def ptr(tensor, offset=0, live=cnt > 0):
                return ctypes.c_void_p(tensor.data_ptr() + offset * tensor.element_size()) if live else None

            args.features[t] = ptr(features, s * 384)
            args.w1[t], args.w2[t], args.w3[t], args.w4[t] = (ptr(x) for x in tr)
            args.b1[t], args.b2[t], args.b3[t], args.b4[t] = (ptr(b.detach()) for b in (b1, b2, b3, b4))
            args.energy[t] = ptr(energy, s)
            args.act1[t], args.act2[t], args.act3[t] = (ptr(a, s * a.shape[1]) for a in acts)
            args.dact1[t], args.dact2[t], args.dact3[t] = (ptr(d, s * d.shape[1]) for d in dacts)
            args.packed[t] = ptr(packed[t]) if packed is not None else None
        acs_arr = np.ascontiguousarray(np.asarray(acs, dtype=np.int32))
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().ani_mlp_forward_f32(ctypes.byref(args), acs_arr.ctypes.data_as(_lib.c_int_p),
                                                      int(act_id), int(split) & 1, stream),
                       "ani_mlp_forward_f32")
        ctx.save_for_backward(features, *acts, *dacts, *params)
        ctx.acs, ctx.act_fn, ctx.split, ctx.accumulate = acs_arr, act_fn, bool(int(split) & 1), bool(int(split) & 2)
        ctx.packed = packed      # the weights do not change between this pass and its backward pass
        return energy

    @staticmethod
    def backward(ctx, grad_energy):
        features, a1, a2, a3, d1, d2, d3, *params = ctx.saved_tensors
        acs, act_fn = ctx.acs, ctx.act_fn
        if torch.is_grad_enabled():
            # double backward: everything from differentiable ops so that the second derivative
            # through the activation is kept
            with torch.enable_grad():
                inputs = [features] + list(params)
                wanted = [k for k, need in enumerate([ctx.needs_input_grad[0]] + list(ctx.needs_input_grad[5:])) if need]
                energy = _dense_energies(features, acs, act_fn, params)
                got = torch.autograd.grad(energy, [inputs[k] for k in wanted], grad_energy, create_graph=True,
                                          allow_unused=True)
            out = [None] * len(inputs)
            for k, g in zip(wanted, got):
                out[k] = g
            return (out[0], None, None, None, None, *out[1:])
        n = features.shape[0]
        dev = features.device
        starts = np.concatenate([[0], np.cumsum(acs)])
        f32 = dict(dtype=torch.float32, device=dev)
        dz1, dz2, dz3 = torch.empty((n, 128), **f32), torch.empty((n, 128), **f32), torch.empty((n, 64), **f32)
        grad_feat = torch.empty_like(features) if ctx.needs_input_grad[0] else None
        g = grad_energy.contiguous()
        args = _lib.MlpBackwardArgs()
        keep = []
        for t in range(4):
            s, cnt = int(starts[t]), int(acs[t])
            w1, _, w2, _, w3, _, w4, _ = params[8 * t: 8 * t + 8]
            ws = [w1.detach().contiguous(), w2.detach().contiguous(), w3.detach().contiguous(),
                  w4.detach().reshape(-1).contiguous()]
            keep.extend(ws)

            def ptr(tensor, offset=0, live=cnt > 0):
                return ctypes.c_void_p(tensor.data_ptr() + offset * tensor.element_size()) if live else None

            args.grad_energy[t] = ptr(g, s)
            args.w1[t], args.w2[t], args.w3[t], args.w4[t] = (ptr(x) for x in ws)
            args.dact1[t], args.dact2[t], args.dact3[t] = ptr(d1, s * 128), ptr(d2, s * 128), ptr(d3, s * 64)
            args.dz1[t], args.dz2[t], args.dz3[t] = ptr(dz1, s * 128), ptr(dz2, s * 128), ptr(dz3, s * 64)
            args.grad_features[t] = ptr(grad_feat, s * 384) if grad_feat is not None else None
            args.packed[t] = ptr(ctx.packed[t]) if ctx.packed is not None else None
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().ani_mlp_backward_f32(ctypes.byref(args), acs.ctypes.data_as(_lib.c_int_p),
                                                       int(ctx.split), stream), "ani_mlp_backward_f32")
        # weight and bias gradients: one more launch.  With `accumulate_into_grad` set on the model
        # (only valid when gradients are obtained with .backward(), as the trainer does) and a
        # gradient buffer on every parameter (the flat optimiser provides them) the kernel adds
        # into those buffers directly and None is returned, which is what autograd's own
        # accumulation would do with 32 separate additions; otherwise the gradients are slices
        # of one zero-filled buffer and are returned.
        sizes = [384 * 128, 128, 128 * 128, 128, 128 * 64, 64, 64, 4]   # the last slot holds b4 (1 value): keeps every slice 16-byte aligned
        per_elem = sum(sizes)
        direct = ctx.accumulate and all(p.grad is not None and p.grad.is_contiguous() and p.grad.dtype == torch.float32
                     and p.grad.data_ptr() % 16 == 0 for p in params)
        wbuf = None if direct else torch.zeros(4 * per_elem, **f32)
        wargs = _lib.MlpWeightGradArgs()
        grads = [None] * len(params)
        for t in range(4):
            s, e = int(starts[t]), int(starts[t + 1])
            cnt = e - s

            def ptr(tensor, offset=0, live=cnt > 0):
                return ctypes.c_void_p(tensor.data_ptr() + offset * tensor.element_size()) if live else None

            wargs.features[t], wargs.act1[t], wargs.act2[t] = ptr(features, s * 384), ptr(a1, s * 128), ptr(a2, s * 128)
            wargs.act3[t], wargs.grad_energy[t] = ptr(a3, s * 64), ptr(g, s)
            wargs.dz1[t], wargs.dz2[t], wargs.dz3[t] = ptr(dz1, s * 128), ptr(dz2, s * 128), ptr(dz3, s * 64)
            if direct:
                outs = [ptr(p.grad) for p in params[8 * t: 8 * t + 8]]
            else:
                offs = np.concatenate([[0], np.cumsum(sizes)]) + t * per_elem
                outs = [ptr(wbuf, int(o)) for o in offs[:8]]
                if cnt > 0:
                    grads[8 * t: 8 * t + 8] = [
                        wbuf[int(offs[k]):int(offs[k]) + params[8 * t + k].numel()].view(params[8 * t + k].shape)
                        for k in range(8)]
            (wargs.dw1[t], wargs.db1[t], wargs.dw2[t], wargs.db2[t], wargs.dw3[t], wargs.db3[t],
             wargs.dw4[t], wargs.db4[t]) = outs
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().ani_mlp_weight_grad_f32(ctypes.byref(wargs), acs.ctypes.data_as(_lib.c_int_p),
                                                          int(ctx.split), stream), "ani_mlp_weight_grad_f32")
        return (grad_feat, None, None, None, None, *grads)


class _GatherRows(torch.autograd.Function):
    """``x[idx]`` whose backward is one scatter-add (torch's own index backward sorts the
    indices first: five launches instead of two)."""

    @staticmethod
    def forward(ctx, x, idx):
        ctx.save_for_backward(idx)
        ctx.n = x.shape[0]
        return x[idx]

    @staticmethod
    def backward(ctx, grad):
        (idx,) = ctx.saved_tensors
        out = torch.zeros((ctx.n,) + tuple(grad.shape[1:]), dtype=grad.dtype, device=grad.device)
        return out.index_add_(0, idx, grad), None


class MoleculeNN:
    """One :class:`AtomNN` per element plus the gather back to atom order."""

    def __init__(self, type_map=TYPE_MAP, layer_sizes=FUSED_LAYERS, precision=torch.float32,
                 activation_fn=activations.celu, prefix: str = "near_", device="cuda", seed=None,
                 init: str = "reference", split_precision: bool = True):
        gen = torch.Generator().manual_seed(seed) if seed is not None else None
        self.type_map = list(type_map)
        self.layer_sizes = tuple(layer_sizes)
        self.precision = precision
        self.activation_fn = activation_fn
        self.split_precision = split_precision
        self.accumulate_into_grad = False   # see _FusedMlp.backward; set by trainers that call .backward()
        self.anns = [AtomNN(layer_sizes, precision, activation_fn, atom_type=t, prefix=prefix,
                            device=device, generator=gen, init=init) for t in self.type_map]

    def get_parameters(self):
        out = []
        for a in self.anns:
            out.extend(a.get_parameters())
        return out

    def named_parameters(self):
        out = {}
        for a in self.anns:
            out.update(a.named_parameters())
        return out

    def pack_weights(self, stream=None):
        """Refreshes the pre-packed copy of W1, W2, W3 of the four networks (``ani_mlp_pack_weights_f32``:
        one small launch) and returns it, ``[4, ani_mlp_packed_bytes()]`` bytes on the parameters' device.
        The tensor-core kernels that are given it fetch their weight chunks with one bulk copy each;
        it has to be refreshed whenever the weights changed, so the callers do it once per pass."""
        dev = self.anns[0].Ws[0].device
        if getattr(self, "_packed", None) is None or self._packed.device != dev:
            self._packed = torch.empty((4, int(_lib.lib().ani_mlp_packed_bytes())), dtype=torch.uint8, device=dev)
        args = _lib.MlpPackArgs()
        for t, ann in enumerate(self.anns):
            w1, w2, w3 = (w.detach() for w in ann.Ws[:3])
            if not (w1.is_contiguous() and w2.is_contiguous() and w3.is_contiguous()):
                return None
            args.w1[t], args.w2[t], args.w3[t] = w1.data_ptr(), w2.data_ptr(), w3.data_ptr()
            args.packed[t] = self._packed[t].data_ptr()
        if stream is None:
            stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().ani_mlp_pack_weights_f32(ctypes.byref(args), stream), "ani_mlp_pack_weights_f32")
        return self._packed

    def packed_weights(self):
        """The pre-packed copy as ``pack_weights`` last wrote it (None before the first call)."""
        return getattr(self, "_packed", None)

    @property
    def fused(self) -> bool:
        return (self.precision == torch.float32 and self.layer_sizes == FUSED_LAYERS
                and len(self.anns) == 4 and self.activation_fn in activations.KERNEL_ID)

    def atom_energies_sorted(self, features: torch.Tensor, acs) -> torch.Tensor:
        """Energies in element-sorted order from the ``[n_atoms, F]`` feature buffer laid out H
        rows, C rows, N rows, O rows."""
        acs = np.asarray(acs, dtype=np.int64)
        if self.fused and features.is_cuda:
            params = []
            for a in self.anns:
                for w, b in zip(a.Ws, a.bs):
                    params.extend([w, b])
            flags = (1 if self.split_precision else 0) | (2 if self.accumulate_into_grad else 0)
            _lib.same_device(features.device, self.anns[0].Ws[0], where="MoleculeNN.atom_energies_sorted")
            packed = self.pack_weights()
            return _FusedMlp.apply(features, acs, activations.KERNEL_ID[self.activation_fn],
                                   flags, (self.activation_fn, packed), *params)
        starts = np.concatenate([[0], np.cumsum(acs)])
        parts = [ann.atom_energies(features[int(starts[t]):int(starts[t + 1])])
                 for t, ann in enumerate(self.anns)]
        return torch.cat(parts)

    def atom_outputs(self, features: torch.Tensor, acs, gather_idxs: torch.Tensor) -> torch.Tensor:
        """Atomic energies in atom order (``tf.gather(tf.concat(...), gather_idxs)``,
        khan/model/nn.py:171-172)."""
        return _GatherRows.apply(self.atom_energies_sorted(features, acs), gather_idxs.long())
