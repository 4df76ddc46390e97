"""``RawDataset``: the unfeaturized dataset type of khan (``khan/data/dataset.py:6-183`` of the
reference), with the same constructor and methods."""
from __future__ import annotations

import math

import numpy as np


class RawDataset:
    """A collection of molecules, each an ``(n, 4)`` array ``[type, x, y, z]`` with compacted
    element ids (H 0, C 1, N 2, O 3), optional per-molecule targets ``all_ys`` and optional
    per-molecule ``(n, 3)`` forces ``all_grads``."""

    def __init__(self, all_Xs, all_ys=None, all_grads=None):
        if all_ys is not None:
            assert len(all_Xs) == len(all_ys)
        if all_grads is not None:
            assert len(all_Xs) == len(all_grads)
        self.all_Xs = all_Xs
        self.all_ys = all_ys
        self.all_grads = all_grads

    def num_mols(self) -> int:
        return len(self.all_Xs)

    def num_batches(self, batch_size: int) -> int:
        return math.ceil(self.num_mols() / batch_size)

    def iterate(self, batch_size: int, shuffle: bool, fuzz=None):
        """Yields ``(mol_Xs, mol_ids, mol_yts, mol_grads)`` per batch exactly as the reference does
        (``khan/data/dataset.py:144-183``): concatenated ``(N, 4)`` atoms, per-atom molecule index
        inside the batch, targets (or None) and concatenated forces (or None).  The last batch is
        not padded.  ``fuzz`` adds uniform noise in ``[-fuzz, fuzz]`` to the coordinates."""
        perm = np.arange(len(self.all_Xs))
        if shuffle:
            np.random.shuffle(perm)
        for batch_idx in range(self.num_batches(batch_size)):
            picks = perm[batch_idx * batch_size: min((batch_idx + 1) * batch_size, len(self.all_Xs))]
            mols = [self.all_Xs[p] for p in picks]
            counts = np.fromiter((len(m) for m in mols), dtype=np.int64, count=len(mols))
            mol_Xs = np.concatenate(mols, axis=0)  # a copy: safe to modify
            mol_ids = np.repeat(np.arange(len(mols)), counts)
            if fuzz is not None:
                # x of all atoms, then y, then z: the order in which the reference consumes numpy's
                # stream (khan/data/dataset.py:166-169), so a seed gives the same perturbed batch
                mol_Xs[:, 1:4] += np.random.uniform(-fuzz, fuzz, (3, mol_Xs.shape[0])).T
            mol_yts = [self.all_ys[p] for p in picks] if self.all_ys is not None else None
            mol_grads = (np.concatenate([self.all_grads[p] for p in picks], axis=0)
                         if self.all_grads is not None else None)
            yield mol_Xs, mol_ids, mol_yts, mol_grads
