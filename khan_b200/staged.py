"""A batch staged on one GPU with every buffer of the hot path pre-allocated, so that one pass
(ani_sort -> featurize -> featurize_grad) issues C-ABI calls only: no allocation, no host
synchronisation, nothing that cannot be captured into a CUDA graph.

The reference runs the same three ops per tower per batch
(``khan/training/trainer_multi_tower.py:295-320`` forward, ``:23-52`` gradient); there the sort
runs on the host and the gradient op on the CPU.  Here all three run on the device, and the
per-element atom counts that size the outputs are taken from the host copy of the element ids
(one ``bincount`` while the batch is being assembled), so no device-to-host copy sits between
the sort and the featurizer.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib

FEATURE_SIZE = 384


def _ptr(t: torch.Tensor, offset_elems: int = 0) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr() + offset_elems * t.element_size())


class StagedBatch:
    """Device buffers for one batch: inputs, sort outputs, features, upstream, gradients."""

    def __init__(self, n_atoms: int, n_mols: int, dtype=torch.float32, device="cuda:0"):
        self.device = torch.device(device)
        self.dtype = dtype
        self.suffix = "f32" if dtype == torch.float32 else "f64"
        self.n_atoms_cap, self.n_mols_cap = n_atoms, n_mols
        self.n_atoms, self.n_mols = n_atoms, n_mols
        d, i32 = self.device, torch.int32
        self.xyz = torch.empty((3, n_atoms), dtype=dtype, device=d)
        self.x, self.y, self.z = self.xyz[0], self.xyz[1], self.xyz[2]   # what the kernels read
        self.types = torch.empty(n_atoms, dtype=i32, device=d)
        self.mol_offsets = torch.empty(n_mols, dtype=i32, device=d)
        self.mol_counts = torch.empty(n_mols, dtype=i32, device=d)
        self._own_inputs = (self.x, self.y, self.z, self.types, self.mol_offsets, self.mol_counts)
        self.scatter = torch.empty(n_atoms, dtype=i32, device=d)
        self.gather = torch.empty(n_atoms, dtype=i32, device=d)
        self.counts = torch.empty(4, dtype=i32, device=d)
        self.features = torch.empty((n_atoms, FEATURE_SIZE), dtype=dtype, device=d)
        self.upstream = torch.empty((n_atoms, FEATURE_SIZE), dtype=dtype, device=d)
        self.grads = torch.empty((3, n_atoms), dtype=dtype, device=d)
        self.acs_host = np.zeros(4, np.int32)
        self._acs_ptr = self.acs_host.ctypes.data_as(_lib.c_int_p)

    # -- host -> device --------------------------------------------------------------------
    def set_shape(self, n_atoms: int, n_mols: int, acs_host) -> None:
        if n_atoms > self.n_atoms_cap or n_mols > self.n_mols_cap:
            raise ValueError("batch larger than the staged capacity")
        self.n_atoms, self.n_mols = int(n_atoms), int(n_mols)
        self.acs_host[:] = acs_host
        if int(self.acs_host.sum()) != self.n_atoms:
            raise ValueError("atom counts do not add up to n_atoms")

    def adopt(self, fed) -> None:
        """Uses the device tensors of a fed batch (``khan_b200.data.feeder.FedBatch``) as the inputs of
        the next passes, without copying them; the sort / feature / gradient buffers stay this
        object's own.  The fed batch must stay alive until those passes have been enqueued."""
        if fed.x.dtype != self.dtype:
            raise ValueError("precision of the fed batch does not match")
        self.set_shape(fed.n_atoms, fed.n_mols, fed.acs)
        self.x, self.y, self.z = fed.x, fed.y, fed.z
        self.types, self.mol_offsets, self.mol_counts = fed.types, fed.mol_offsets, fed.mol_counts

    def upload(self, host: "HostBatch", non_blocking: bool = True, with_upstream: bool = True) -> int:
        """Copies one pinned host batch in; returns the bytes moved."""
        self.x, self.y, self.z, self.types, self.mol_offsets, self.mol_counts = self._own_inputs
        self.set_shape(host.n_atoms, host.n_mols, host.acs)
        n, m = self.n_atoms, self.n_mols
        for r in range(3):   # row by row: each copy is one contiguous range on both sides
            self.xyz[r, :n].copy_(host.xyz[r, :n], non_blocking=non_blocking)
        self.types[:n].copy_(host.types[:n], non_blocking=non_blocking)
        self.mol_offsets[:m].copy_(host.mol_offsets[:m], non_blocking=non_blocking)
        self.mol_counts[:m].copy_(host.mol_counts[:m], non_blocking=non_blocking)
        moved = n * (3 * self.xyz.element_size() + 4) + m * 8
        if with_upstream:
            self.upstream[:n].copy_(host.upstream[:n], non_blocking=non_blocking)
            moved += n * FEATURE_SIZE * self.upstream.element_size()
        return moved

    def download(self, features_host: torch.Tensor, grads_host: torch.Tensor, non_blocking: bool = True) -> int:
        """Copies the feature rows and the coordinate gradients of the current batch into
        (pinned) host tensors of shape [>= n_atoms, 384] and [3, >= n_atoms]; returns the
        bytes moved.  Every copy is one contiguous range on both sides, so none of them falls
        back to a staged, host-blocking transfer."""
        n = self.n_atoms
        features_host[:n].copy_(self.features[:n], non_blocking=non_blocking)
        for r in range(3):
            grads_host[r, :n].copy_(self.grads[r, :n], non_blocking=non_blocking)
        return n * (FEATURE_SIZE + 3) * self.features.element_size()

    # -- the hot path ----------------------------------------------------------------------
    def _element_ptrs(self, buf: torch.Tensor):
        starts = np.concatenate([[0], np.cumsum(self.acs_host)])[:4]
        return [_ptr(buf, int(s) * FEATURE_SIZE) for s in starts]

    def run_sort(self, stream: ctypes.c_void_p) -> None:
        _lib.check(_lib.lib().ani_sort(_ptr(self.types), self.n_atoms, _ptr(self.scatter),
                                       _ptr(self.gather), _ptr(self.counts), stream), "ani_sort")

    def run_featurize(self, stream: ctypes.c_void_p) -> None:
        fn = getattr(_lib.lib(), "ani_featurize_" + self.suffix)
        _lib.check(fn(_ptr(self.x), _ptr(self.y), _ptr(self.z), _ptr(self.types),
                      _ptr(self.mol_offsets), _ptr(self.mol_counts), self.n_mols, _ptr(self.scatter),
                      *self._element_ptrs(self.features), self._acs_ptr, stream),
                   "ani_featurize_" + self.suffix)

    def run_featurize_grad(self, stream: ctypes.c_void_p) -> None:
        fn = getattr(_lib.lib(), "ani_featurize_grad_" + self.suffix)
        cap = self.n_atoms_cap
        _lib.check(fn(_ptr(self.x), _ptr(self.y), _ptr(self.z), _ptr(self.types),
                      _ptr(self.mol_offsets), _ptr(self.mol_counts), self.n_mols, _ptr(self.scatter),
                      *self._element_ptrs(self.upstream), _ptr(self.grads), _ptr(self.grads, cap),
                      _ptr(self.grads, 2 * cap), self._acs_ptr, stream),
                   "ani_featurize_grad_" + self.suffix)

    def run_step(self, stream: ctypes.c_void_p | None = None) -> None:
        """One pass of the hot path: sort, forward, coordinate gradient (``kernels_per_step()`` launches)."""
        if stream is None:
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        self.run_sort(stream)
        self.run_featurize(stream)
        self.run_featurize_grad(stream)

    KERNELS_PER_STEP = 3  # sort, featurize, featurize_grad (batches of small molecules)

    def kernels_per_step(self) -> int:
        """Kernel launches of ``run_step`` for the current batch: 3 for a batch of small molecules (mean
        size <= 24 atoms, the rule of the library's dispatch), else 4 -- the gradient kernel for large
        molecules accumulates with atomics and is preceded by a zero fill of its outputs."""
        return 3 if self.n_mols > 0 and self.n_atoms <= 24 * self.n_mols else 4


class HostBatch:
    """One batch in pinned host memory, in the layout StagedBatch.upload expects."""

    def __init__(self, batch, upstream=None, dtype=torch.float32, pin: bool = True):
        np_dt = np.float32 if dtype == torch.float32 else np.float64
        self.n_atoms, self.n_mols = batch.n_atoms, batch.n_mols
        self.acs = np.bincount(batch.atomic_numbers, minlength=4).astype(np.int32)

        def pinned(a):
            t = torch.from_numpy(np.ascontiguousarray(a))
            return t.pin_memory() if pin and torch.cuda.is_available() else t

        self.xyz = pinned(np.stack(batch.coords(np_dt)))
        self.types = pinned(batch.atomic_numbers.astype(np.int32))
        self.mol_offsets = pinned(batch.mol_offsets.astype(np.int32))
        self.mol_counts = pinned(batch.mol_atom_counts.astype(np.int32))
        if upstream is None:
            self.upstream = None
        else:
            flat = np.concatenate([np.asarray(u, dtype=np_dt).reshape(-1, FEATURE_SIZE) for u in upstream])
            self.upstream = pinned(flat)
