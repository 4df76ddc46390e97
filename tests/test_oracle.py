"""Pins the CPU oracle: the plain-C restatement (oracle/ani_oracle.c) against the reference's
known-answer vectors and against golden outputs of the reference's own kernel_cpu.cpp."""
import numpy as np
import pytest

from conftest import normwise
from khan_b200.data import synthetic as syn

ELEMS = "hcno"


def _args(g):
    return (g["atomic_numbers"], g["mol_offsets"], g["mol_atom_counts"], g["scatter_idxs"],
            g["atom_counts"])


def test_sort_known_answer(oracle_mod):
    # gpu_featurizer/test_kernel.py:310-312 (same gather vector in khan/model/test_nn.py:95)
    b = syn.kat_fixture()
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    np.testing.assert_array_equal(ac, [6, 2, 3, 0])
    np.testing.assert_array_equal(si, [0, 0, 1, 0, 1, 2, 3, 4, 5, 1, 2])
    np.testing.assert_array_equal(gi, [0, 8, 1, 6, 9, 2, 3, 4, 5, 7, 10])


def test_sort_matches_stable_argsort(oracle_mod):
    rng = np.random.default_rng(3)
    for n in (0, 1, 7, 33, 1000):
        a = rng.integers(0, 4, n).astype(np.int32)
        si, gi, ac = oracle_mod.ani_sort(a)
        order = np.argsort(a, kind="stable")
        inv = np.empty(n, np.int64)
        inv[order] = np.arange(n)
        np.testing.assert_array_equal(gi, inv)
        np.testing.assert_array_equal(ac, np.bincount(a, minlength=4))
        starts = np.concatenate([[0], np.cumsum(ac)])[:4]
        np.testing.assert_array_equal(si, inv - starts[a] if n else inv)


def test_linearize_matches_reference_layout(oracle_mod):
    # pair order HH,HC,HN,HO,CC,CN,CO,NN,NO,OO (gpu_featurizer/kernel_cpu.cpp:9-23)
    k = 0
    for i in range(4):
        for j in range(i, 4):
            assert oracle_mod.linearize(i, j, 0, 0) == k * 32
            assert oracle_mod.linearize(j, i, 3, 2) == k * 32 + 3 * 4 + 2
            k += 1


@pytest.mark.parametrize("fixture", ["kat.npz", "c0_head.npz"])
@pytest.mark.parametrize("tag,dt", [("f32", np.float32), ("f64", np.float64)])
def test_port_forward_equals_reference_golden(oracle_mod, golden, fixture, tag, dt):
    g = golden(fixture)
    feats = oracle_mod.featurize(g["xs"].astype(dt), g["ys"].astype(dt), g["zs"].astype(dt),
                                 *_args(g), impl="port")
    for t, e in enumerate(ELEMS):
        # the port follows the reference's types operation by operation: bit-exact
        np.testing.assert_array_equal(feats[t], g[f"feat_{e}_{tag}"])


@pytest.mark.parametrize("fixture", ["kat.npz", "c0_head.npz"])
def test_port_gradient_equals_reference_golden(oracle_mod, golden, fixture):
    g = golden(fixture)
    up = [g["up_" + e] for e in ELEMS]
    out = oracle_mod.featurize_grad(g["xs"], g["ys"], g["zs"], *_args(g), *up, impl="port")
    for k, c in enumerate("xyz"):
        assert normwise(out[k], g[f"grad_{c}_f64"]) < 1e-13


def test_port_full_config0_checksums(oracle_mod, golden):
    g = golden("c0_sums.npz")
    si, gi, ac = oracle_mod.ani_sort(g["atomic_numbers"])
    np.testing.assert_array_equal(ac, g["atom_counts"])
    for tag, dt in (("f32", np.float32), ("f64", np.float64)):
        feats = oracle_mod.featurize(g["xs"].astype(dt), g["ys"].astype(dt), g["zs"].astype(dt),
                                     g["atomic_numbers"], g["mol_offsets"], g["mol_atom_counts"],
                                     si, ac, impl="port", threads=4)
        s = np.array([f.astype(np.float64).sum() for f in feats])
        s2 = np.array([(f.astype(np.float64) ** 2).sum() for f in feats])
        np.testing.assert_allclose(s, g["sum_" + tag], rtol=1e-14)
        np.testing.assert_allclose(s2, g["sumsq_" + tag], rtol=1e-14)


def test_generators_are_deterministic(golden):
    g = golden("c0_sums.npz")
    c0 = syn.config0()
    np.testing.assert_array_equal(c0.atomic_numbers, g["atomic_numbers"])
    np.testing.assert_array_equal(c0.xs, g["xs"])
    np.testing.assert_array_equal(c0.mol_offsets, g["mol_offsets"])


def test_threads_do_not_change_results(oracle_mod):
    b = syn.config1(n_mols=64)
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    x, y, z = b.coords(np.float64)
    args = (b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac)
    one = oracle_mod.featurize(x, y, z, *args, threads=1)
    four = oracle_mod.featurize(x, y, z, *args, threads=4)
    for a, c in zip(one, four):
        np.testing.assert_array_equal(a, c)


def test_gradient_is_the_transpose_of_the_jvp(oracle_mod):
    # <g, J v> == <J^T g, v> on the reference fixture (double)
    b = syn.kat_fixture()
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    rng = np.random.default_rng(0)
    g = [rng.normal(size=int(c) * 384) for c in ac]
    v = [rng.normal(size=b.n_atoms) for _ in range(3)]
    args = (b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac)
    jv = oracle_mod.featurize_grad_inverse(b.xs, b.ys, b.zs, *args, *v)
    jtg = oracle_mod.featurize_grad(b.xs, b.ys, b.zs, *args, *g)
    lhs = sum(float((a * c).sum()) for a, c in zip(g, jv))
    rhs = sum(float((a * c).sum()) for a, c in zip(jtg, v))
    assert abs(lhs - rhs) < 1e-12 * max(1.0, abs(lhs))


def test_gradient_against_finite_differences(oracle_mod):
    # same check as gpu_featurizer/test_kernel.py:463-535 (double: delta 1e-6, tol 1e-9)
    b = syn.kat_fixture()
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    args = (b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac)
    rng = np.random.default_rng(1)
    g = [rng.normal(size=int(c) * 384) for c in ac]
    grads = oracle_mod.featurize_grad(b.xs, b.ys, b.zs, *args, *g)

    def loss(x, y, z):
        f = oracle_mod.featurize(x, y, z, *args)
        return sum(float((a * c).sum()) for a, c in zip(f, g))

    delta = 1e-6
    for axis, arr in enumerate((b.xs, b.ys, b.zs)):
        for i in range(b.n_atoms):
            coords = [b.xs.copy(), b.ys.copy(), b.zs.copy()]
            coords[axis][i] += delta
            up = loss(*coords)
            coords[axis][i] -= 2 * delta
            dn = loss(*coords)
            assert abs((up - dn) / (2 * delta) - grads[axis][i]) < 1e-6


def test_reference_build_agrees_when_present(oracle_mod):
    if not oracle_mod.available("ref"):
        pytest.skip("oracle/_ref not built on this machine")
    b = syn.config1(n_mols=32)
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    args = (b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac)
    for dt in (np.float32, np.float64):
        x, y, z = b.coords(dt)
        for a, c in zip(oracle_mod.featurize(x, y, z, *args, impl="port"),
                        oracle_mod.featurize(x, y, z, *args, impl="ref")):
            np.testing.assert_array_equal(a, c)
    x, y, z = b.coords(np.float64)
    g = syn.upstream_grads(b, ac, dtype=np.float64)
    for a, c in zip(oracle_mod.featurize_grad(x, y, z, *args, *g, impl="port"),
                    oracle_mod.featurize_grad(x, y, z, *args, *g, impl="ref")):
        assert normwise(a, c) < 1e-13


def test_reference_indexing_of_grad_inverse_vanishes(oracle_mod):
    # gpu_featurizer/kernel_cpu.cpp:111,118,155,162,169 read X_grads at the central atom's element
    # id for every atom of a term; the i/j/k derivatives of a term cancel, so the result is ~0
    b = syn.kat_fixture()
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    rng = np.random.default_rng(4)
    v = [rng.normal(size=b.n_atoms) for _ in range(3)]
    args = (b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac)
    port = oracle_mod.featurize_grad_inverse(b.xs, b.ys, b.zs, *args, *v, reference_indexing=True)
    assert all(np.abs(o).max() == 0 for o in port if o.size)
    if oracle_mod.available("ref"):
        ref = oracle_mod.featurize_grad_inverse(b.xs, b.ys, b.zs, *args, *v, impl="ref")
        assert all(np.abs(o).max() < 1e-12 for o in ref if o.size)
    jvp = oracle_mod.featurize_grad_inverse(b.xs, b.ys, b.zs, *args, *v)
    assert max(np.abs(o).max() for o in jvp if o.size) > 1.0
