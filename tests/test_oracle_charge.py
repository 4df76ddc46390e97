"""CPU checks of the AniCharge / AniChargeGrad restatement in oracle/.

The reference holds no golden numbers for these ops: its tests check only that AniChargeGrad is
the derivative of AniCharge by finite differences, on the 11-atom fixture with a fixed charge
vector, to 2e-3 (float32, delta 1e-2) and 1e-11 (float64, delta 1e-3)
(gpu_featurizer/test_kernel.py:398-447).  The same check pins the oracle here, together with
properties of the formula itself (gpu_featurizer/ani_charges.cpp:58-71)."""
import numpy as np
import pytest

from khan_b200.data import synthetic as syn

QS = [0.3, 4.5, 2.2, 3.4, -5.6, 3.4, 1.1, 3.2, 1.0, 0.3, 2.4]   # test_kernel.py:424-436
K_E = np.float32(0.529176917)                                    # parameters.h:10
R_RC = np.float32(4.6)


def _energy_numpy(b, q):
    x, y, z = b.coords(np.float64)
    out = np.zeros(b.n_mols)
    for m, (o, n) in enumerate(zip(b.mol_offsets, b.mol_atom_counts)):
        for i in range(o, o + n):
            for j in range(i + 1, o + n):
                r = np.sqrt((x[i] - x[j]) ** 2 + (y[i] - y[j]) ** 2 + (z[i] - z[j]) ** 2)
                fc = 0.5 * np.cos(np.pi * r / float(R_RC)) + 0.5 if r <= float(R_RC) else 0.0
                out[m] += float(K_E) * q[i] * q[j] * (1 - fc) / r
    return out


@pytest.mark.parametrize("dt,delta,tol", [(np.float32, 1e-2, 2e-3), (np.float64, 1e-3, 1e-11)])
def test_gradient_error_as_the_reference_test_measures_it(oracle_mod, dt, delta, tol):
    b = syn.kat_fixture()
    x, y, z = b.coords(dt)
    q = np.array(QS, dt)
    args = (b.mol_offsets, b.mol_atom_counts)
    # tf.test.compute_gradient_error: max |analytic - numeric| over the (11 x 2) Jacobian
    numeric = np.zeros((11, 2))
    for i in range(11):
        qp, qm = q.copy(), q.copy()
        qp[i] += dt(delta)
        qm[i] -= dt(delta)
        ep = oracle_mod.ani_charge(x, y, z, qp, *args).astype(np.float64)
        em = oracle_mod.ani_charge(x, y, z, qm, *args).astype(np.float64)
        numeric[i] = (ep - em) / (2 * delta)
    analytic = np.zeros((11, 2))
    for m in range(2):
        g = np.zeros(2, dt)
        g[m] = 1
        analytic[:, m] = oracle_mod.ani_charge_grad(x, y, z, q, *args, g)
    assert np.abs(analytic - numeric).max() < tol


def test_energy_matches_the_formula(oracle_mod):
    b = syn.kat_fixture()
    x, y, z = b.coords(np.float64)
    q = np.array(QS)
    got = oracle_mod.ani_charge(x, y, z, q, b.mol_offsets, b.mol_atom_counts)
    assert np.allclose(got, _energy_numpy(b, q), rtol=1e-13, atol=0)
    got32 = oracle_mod.ani_charge(*b.coords(np.float32), q.astype(np.float32), b.mol_offsets, b.mol_atom_counts)
    assert np.allclose(got32, got, rtol=2e-6)


def test_bilinear_in_the_charges_and_zero_outside_molecules(oracle_mod):
    b = syn.config1(n_mols=12)
    x, y, z = b.coords(np.float64)
    rng = np.random.default_rng(3)
    q = rng.normal(size=b.n_atoms)
    args = (b.mol_offsets, b.mol_atom_counts)
    e1 = oracle_mod.ani_charge(x, y, z, q, *args)
    assert np.allclose(oracle_mod.ani_charge(x, y, z, 3 * q, *args), 9 * e1, rtol=1e-13)
    # Euler: sum_i q_i dE/dq_i = 2 E for a form of degree two
    g = oracle_mod.ani_charge_grad(x, y, z, q, *args, np.ones(b.n_mols))
    per_mol = np.add.reduceat(q * g, b.mol_offsets)
    assert np.allclose(per_mol, 2 * e1, rtol=1e-12, atol=1e-14)
    # leave the last molecule out of the table: its atoms get a zero gradient
    g2 = oracle_mod.ani_charge_grad(x, y, z, q, b.mol_offsets[:-1], b.mol_atom_counts[:-1], np.ones(b.n_mols - 1))
    assert np.all(g2[b.mol_offsets[-1]:] == 0) and np.array_equal(g2[:b.mol_offsets[-1]], g[:b.mol_offsets[-1]])


def test_empty_and_single_atom_molecules(oracle_mod):
    x = np.array([0.0, 1.0, 5.0])
    z = np.zeros(3)
    q = np.array([1.0, -2.0, 0.5])
    e = oracle_mod.ani_charge(x, z, z, q, np.array([0, 2, 3]), np.array([2, 1, 0]))
    assert e[1] == 0 and e[2] == 0 and e[0] != 0
    assert oracle_mod.ani_charge(x[:0], z[:0], z[:0], q[:0], np.zeros(0, np.int32), np.zeros(0, np.int32)).shape == (0,)
