"""Seeded synthetic molecule batches with the shape statistics of the ANI-1 GDB sets.

The reference trains on ANI-1 GDB8 conformations (loaded by ``data_loaders.py:37-46`` of the
reference through ``khan/data/pyanitools.py``); that data set is not available offline, so
these generators stand in for it.  Nothing here reproduces an item of the real data set: the
molecules are random walks, not chemistry.

Every generator returns a :class:`Batch` whose arrays are laid out exactly as
``RawDataset.iterate`` + the trainer's graph feed them to the ops
(``khan/training/trainer_multi_tower.py:295-320`` of the reference): structure-of-arrays
coordinates, compacted element ids H0 C1 N2 O3, and per-molecule offsets / atom counts.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

VALENCE = {1: 4, 2: 3, 3: 2}  # compacted ids: C, N, O


@dataclass
class Batch:
    """One batch of molecules in the op-level layout (float64 master copy)."""

    xs: np.ndarray  # float64[N]
    ys: np.ndarray
    zs: np.ndarray
    atomic_numbers: np.ndarray  # int32[N], 0..3
    mol_offsets: np.ndarray  # int32[M]
    mol_atom_counts: np.ndarray  # int32[M]

    @property
    def n_atoms(self) -> int:
        return int(self.atomic_numbers.shape[0])

    @property
    def n_mols(self) -> int:
        return int(self.mol_atom_counts.shape[0])

    def coords(self, dtype):
        return (self.xs.astype(dtype), self.ys.astype(dtype), self.zs.astype(dtype))

    def molecules(self):
        """List of (n, 4) ``[type, x, y, z]`` arrays: the input format of ``RawDataset``."""
        out = []
        for off, cnt in zip(self.mol_offsets, self.mol_atom_counts):
            sl = slice(int(off), int(off + cnt))
            out.append(np.stack([self.atomic_numbers[sl].astype(np.float64), self.xs[sl],
                                 self.ys[sl], self.zs[sl]], axis=1))
        return out

    def slice_mols(self, start: int, stop: int) -> "Batch":
        """Molecules ``[start, stop)`` as an independent batch (offsets rebased to 0)."""
        cnt = self.mol_atom_counts[start:stop]
        if cnt.shape[0] == 0:
            z = np.zeros(0)
            return Batch(z, z.copy(), z.copy(), np.zeros(0, np.int32), np.zeros(0, np.int32),
                         np.zeros(0, np.int32))
        a0 = int(self.mol_offsets[start])
        a1 = int(self.mol_offsets[stop - 1] + self.mol_atom_counts[stop - 1])
        off = (self.mol_offsets[start:stop] - a0).astype(np.int32)
        return Batch(self.xs[a0:a1].copy(), self.ys[a0:a1].copy(), self.zs[a0:a1].copy(),
                     self.atomic_numbers[a0:a1].copy(), off, cnt.copy())


def _unit(rng) -> np.ndarray:
    v = rng.normal(size=3)
    return v / np.linalg.norm(v)


def _walk_molecule(rng, n_heavy: int):
    """Self-avoiding random walk of heavy atoms with hydrogens filling the valences."""
    types = rng.choice(np.array([1, 2, 3]), size=n_heavy, p=[0.72, 0.14, 0.14])
    pos = np.zeros((n_heavy, 3))
    for k in range(1, n_heavy):
        for _ in range(200):
            bond = rng.uniform(1.38, 1.54)
            if k == 1:
                cand = pos[0] + bond * _unit(rng)
            else:
                back = pos[k - 2] - pos[k - 1]
                back /= np.linalg.norm(back)
                ang = np.deg2rad(rng.uniform(105.0, 120.0))
                # random direction at angle `ang` from the previous bond
                perp = np.cross(back, _unit(rng))
                while np.linalg.norm(perp) < 1e-6:
                    perp = np.cross(back, _unit(rng))
                perp /= np.linalg.norm(perp)
                cand = pos[k - 1] + bond * (np.cos(ang) * back + np.sin(ang) * perp)
            if k < 2 or np.min(np.linalg.norm(pos[: k - 1] - cand, axis=1)) > 1.9:
                break
        pos[k] = cand
    h_pos = []
    for k in range(n_heavy):
        heavy_bonds = (1 if k > 0 else 0) + (1 if k < n_heavy - 1 else 0)
        for _ in range(max(0, VALENCE[int(types[k])] - heavy_bonds)):
            h_pos.append(pos[k] + rng.uniform(1.0, 1.1) * _unit(rng))
    all_types = np.concatenate([types, np.zeros(len(h_pos), dtype=types.dtype)])
    all_pos = np.concatenate([pos, np.array(h_pos).reshape(-1, 3)], axis=0)
    return all_types.astype(np.int32), all_pos


def _assemble(mols) -> Batch:
    counts = np.array([t.shape[0] for t, _ in mols], dtype=np.int32)
    offsets = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int32) if len(mols) else \
        np.zeros(0, np.int32)
    types = np.concatenate([t for t, _ in mols]).astype(np.int32) if len(mols) else np.zeros(0, np.int32)
    pos = np.concatenate([p for _, p in mols], axis=0) if len(mols) else np.zeros((0, 3))
    return Batch(np.ascontiguousarray(pos[:, 0]), np.ascontiguousarray(pos[:, 1]),
                 np.ascontiguousarray(pos[:, 2]), types, offsets, counts)


def gdb_like_batch(n_mols: int, seed: int, heavy_min: int = 1, heavy_max: int = 8,
                   jitter: float = 0.0, jitter_seed: int | None = None) -> Batch:
    """GDB8-like molecules: ``heavy_min..heavy_max`` heavy atoms (uniform), C .72/N .14/O .14,
    bond U(1.38, 1.54) A, bond angle U(105, 120) deg, hydrogens at U(1.0, 1.1) A."""
    rng = np.random.default_rng(seed)
    mols = [_walk_molecule(rng, int(rng.integers(heavy_min, heavy_max + 1))) for _ in range(n_mols)]
    batch = _assemble(mols)
    if jitter > 0.0:
        jr = np.random.default_rng(seed + 10 if jitter_seed is None else jitter_seed)
        batch.xs = batch.xs + jr.normal(0.0, jitter, batch.n_atoms)
        batch.ys = batch.ys + jr.normal(0.0, jitter, batch.n_atoms)
        batch.zs = batch.zs + jr.normal(0.0, jitter, batch.n_atoms)
    return batch


def config0(seed: int = 0) -> Batch:
    """64 molecules with 3-8 heavy atoms: the CPU-runnable forward case."""
    return gdb_like_batch(64, seed, heavy_min=3, heavy_max=8)


def config1(seed: int = 1, n_mols: int = 1024) -> Batch:
    """1024 molecules with 1-8 heavy atoms and N(0, 0.05 A) coordinate jitter."""
    return gdb_like_batch(n_mols, seed, heavy_min=1, heavy_max=8, jitter=0.05, jitter_seed=seed + 10)


def upstream_grads(batch: Batch, atom_counts, seed: int = 12, dtype=np.float32):
    """dL/dAEV ~ N(0, 1) per feature, one flat buffer per element (H, C, N, O)."""
    rng = np.random.default_rng(seed)
    return [rng.normal(size=int(c) * 384).astype(dtype) for c in atom_counts]


def config4(seed: int = 4, n_mols: int = 256, n_min: int = 64, n_max: int = 256) -> Batch:
    """Large molecules: atoms uniform in a sphere at 0.1 atoms/A^3, >= 0.9 A apart,
    H .5 / C .35 / N .08 / O .07."""
    rng = np.random.default_rng(seed)
    mols = []
    for _ in range(n_mols):
        n = int(rng.integers(n_min, n_max + 1))
        radius = (3.0 * n / (4.0 * np.pi * 0.1)) ** (1.0 / 3.0)
        pos = np.zeros((n, 3))
        k = 0
        while k < n:
            cand = rng.uniform(-radius, radius, size=3)
            if cand @ cand > radius * radius:
                continue
            if k and np.min(np.sum((pos[:k] - cand) ** 2, axis=1)) < 0.81:
                continue
            pos[k] = cand
            k += 1
        types = rng.choice(np.array([0, 1, 2, 3]), size=n, p=[0.5, 0.35, 0.08, 0.07]).astype(np.int32)
        mols.append((types, pos))
    return _assemble(mols)


def kat_fixture():
    """The 11-atom, 2-molecule fixture of the reference's own tests
    (``gpu_featurizer/test_kernel.py:269-285``; also ``khan/data/dataset.py:31-47``)."""
    atom_matrix = np.array([
        [0, 1.0, 2.0, 3.0], [2, 2.0, 1.0, 4.0], [0, 0.5, 1.2, 2.3], [1, 0.3, 1.7, 3.2],
        [2, 0.6, 1.2, 1.1], [0, 14.0, 23.0, 15.0], [0, 2.0, 0.5, 0.3], [0, 2.3, 0.2, 0.4],
        [0, 2.3, 0.2, 0.4], [1, 0.3, 1.7, 3.2], [2, 0.6, 1.2, 1.1]], dtype=np.float64)
    return Batch(atom_matrix[:, 1].copy(), atom_matrix[:, 2].copy(), atom_matrix[:, 3].copy(),
                 atom_matrix[:, 0].astype(np.int32), np.array([0, 8], np.int32),
                 np.array([8, 3], np.int32))


def count_work(batch: Batch):
    """(radial pairs P, angular triplets T) of a batch, float32 distances as the float32 kernels
    see them: P = unordered pairs with r < 4.6, T = sum over atoms of C(n_ang, 2) with n_ang the
    neighbours closer than 3.1.  Used to turn a measured time into algorithmic flop/s."""
    xs, ys, zs = batch.coords(np.float32)
    pairs = 0
    triplets = 0
    for off, cnt in zip(batch.mol_offsets, batch.mol_atom_counts):
        sl = slice(int(off), int(off + cnt))
        p = np.stack([xs[sl], ys[sl], zs[sl]], axis=1)
        d = p[:, None, :] - p[None, :, :]
        r = np.sqrt((d * d).sum(-1, dtype=np.float32))
        np.fill_diagonal(r, np.inf)
        pairs += int((r < np.float32(4.6)).sum()) // 2
        n_ang = (r < np.float32(3.1)).sum(1)
        triplets += int((n_ang * (n_ang - 1) // 2).sum())
    return pairs, triplets


def batch_pool(n_batches: int, n_mols: int = 1024, seed: int = 1, pool_factor: int = 4):
    """``n_batches`` distinct config-1-like batches.  Batch 0 is exactly ``config1(seed)``; the
    others draw ``n_mols`` molecules from a pool of ``pool_factor * n_mols`` generated ones and
    apply fresh N(0, 0.05 A) jitter, which is much cheaper than generating every batch anew."""
    first = config1(seed=seed, n_mols=n_mols)
    if n_batches <= 1:
        return [first]
    pool = gdb_like_batch(pool_factor * n_mols, seed + 1000, heavy_min=1, heavy_max=8)
    mols = pool.molecules()
    rng = np.random.default_rng(seed + 2000)
    out = [first]
    for _ in range(n_batches - 1):
        pick = rng.choice(len(mols), size=n_mols, replace=False)
        chosen = [(mols[i][:, 0].astype(np.int32), mols[i][:, 1:] + rng.normal(0.0, 0.05, mols[i][:, 1:].shape))
                  for i in pick]
        out.append(_assemble(chosen))
    return out
