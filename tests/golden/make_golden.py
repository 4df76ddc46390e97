"""Regenerates the golden vectors under tests/golden/ from the REFERENCE's own CPU kernels.

Run in a checkout that has the reference sources (``make -C oracle`` builds
``oracle/_ref/libani_ref_o2.so`` from the reference's unmodified
``gpu_featurizer/kernel_cpu.cpp``):

    python tests/golden/make_golden.py

Files written (float64 unless noted):
  kat.npz      the 11-atom / 2-molecule fixture of gpu_featurizer/test_kernel.py:269-285 with the
               three sort vectors that test asserts (:310-312), reference features in float32
               and float64, and reference coordinate gradients for a seeded upstream.
  c0_head.npz  the first 5 molecules of the config-0 batch (64 GDB8-like molecules, seed 0):
               inputs, reference features (float32 and float64) and gradients.
  c0_sums.npz  per-element-buffer sums and sums of squares of the reference features of the
               whole config-0 batch (float32 and float64 runs), plus its inputs.
The float32 gradient vectors are the float64 reference evaluated on the float32-rounded inputs
and rounded to float32: the reference's own float32 gradient is non-finite on part of these
inputs (0/0 in gpu_featurizer/kernel_cpu.cpp:335-353) and is stored only as a finite mask count.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from khan_b200.data import synthetic as syn  # noqa: E402

IMPL = "ref"


def run(batch, seed_up):
    si, gi, ac = oracle.ani_sort(batch.atomic_numbers)
    out = dict(xs=batch.xs, ys=batch.ys, zs=batch.zs, atomic_numbers=batch.atomic_numbers,
               mol_offsets=batch.mol_offsets, mol_atom_counts=batch.mol_atom_counts,
               scatter_idxs=si, gather_idxs=gi, atom_counts=ac)
    args = (batch.atomic_numbers, batch.mol_offsets, batch.mol_atom_counts, si, ac)
    up = syn.upstream_grads(batch, ac, seed=seed_up, dtype=np.float64)
    for t, name in enumerate("hcno"):
        out["up_" + name] = up[t]
    for dt, tag in ((np.float32, "f32"), (np.float64, "f64")):
        x, y, z = batch.coords(dt)
        feats = oracle.featurize(x, y, z, *args, impl=IMPL)
        for t, name in enumerate("hcno"):
            out[f"feat_{name}_{tag}"] = feats[t]
        # gradient: float64 reference on the dt-rounded inputs and dt-rounded upstream
        x64, y64, z64 = (v.astype(np.float64) for v in (x, y, z))
        up_dt = [u.astype(dt).astype(np.float64) for u in up]
        g = oracle.featurize_grad(x64, y64, z64, *args, *up_dt, impl=IMPL)
        for k, name in enumerate("xyz"):
            out[f"grad_{name}_{tag}"] = g[k].astype(dt)
        if dt == np.float32:
            g32 = oracle.featurize_grad(x, y, z, *args, *[u.astype(dt) for u in up], impl=IMPL)
            out["ref_f32_grad_nonfinite_atoms"] = np.array(
                int(np.sum(~(np.isfinite(g32[0]) & np.isfinite(g32[1]) & np.isfinite(g32[2])))))
    return out


def main():
    assert oracle.available(IMPL), "build oracle/_ref first (make -C oracle)"
    np.savez_compressed(os.path.join(HERE, "kat.npz"), **run(syn.kat_fixture(), 5))
    c0 = syn.config0()
    np.savez_compressed(os.path.join(HERE, "c0_head.npz"), **run(c0.slice_mols(0, 5), 6))
    si, gi, ac = oracle.ani_sort(c0.atomic_numbers)
    sums = dict(xs=c0.xs, ys=c0.ys, zs=c0.zs, atomic_numbers=c0.atomic_numbers,
                mol_offsets=c0.mol_offsets, mol_atom_counts=c0.mol_atom_counts, atom_counts=ac)
    for dt, tag in ((np.float32, "f32"), (np.float64, "f64")):
        x, y, z = c0.coords(dt)
        feats = oracle.featurize(x, y, z, c0.atomic_numbers, c0.mol_offsets, c0.mol_atom_counts,
                                 si, ac, impl=IMPL)
        sums["sum_" + tag] = np.array([f.astype(np.float64).sum() for f in feats])
        sums["sumsq_" + tag] = np.array([(f.astype(np.float64) ** 2).sum() for f in feats])
        sums["max_" + tag] = np.array([f.max() if f.size else 0.0 for f in feats], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "c0_sums.npz"), **sums)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
