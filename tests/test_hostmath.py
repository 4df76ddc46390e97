"""The per-pair / per-triplet formulas the CUDA kernels use (khan_b200/csrc/ani_params.h) are
plain host+device C++.  This test compiles them with g++ into a naive loop nest and checks
them against the oracle, so an algebra mistake shows up without a GPU."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, normwise
from khan_b200.data import synthetic as syn


@pytest.fixture(scope="module")
def hostmath(tmp_path_factory):
    out = tmp_path_factory.mktemp("hostmath") / "libhostmath.so"
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-I", os.path.join(ROOT, "khan_b200", "csrc"),
           "-o", str(out), os.path.join(ROOT, "tests", "hostmath", "host_math.cpp")]
    subprocess.run(cmd, check=True)
    return ctypes.CDLL(str(out))


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


CASES = {
    "kat": lambda: syn.kat_fixture(),
    "gdb": lambda: syn.config1(n_mols=48),
    "large": lambda: syn.config4(n_mols=2, n_min=64, n_max=96),
}


@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("dt,suf,ftol,gtol", [(np.float32, "f32", 1e-5, 1e-5),
                                               (np.float64, "f64", 1e-12, 1e-12)])
def test_shared_math_matches_oracle(hostmath, oracle_mod, case, dt, suf, ftol, gtol):
    b = CASES[case]()
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    x, y, z = b.coords(dt)
    common = (b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac)
    ref = oracle_mod.featurize(x, y, z, *common)
    outs = [np.full(int(c) * 384, 7.0, dt) for c in ac]
    getattr(hostmath, "hostmath_featurize_" + suf)(
        _p(x), _p(y), _p(z), _p(b.atomic_numbers), _p(b.mol_offsets), _p(b.mol_atom_counts),
        ctypes.c_int(b.n_mols), _p(si), *[_p(o) for o in outs])
    for t in range(4):
        assert normwise(outs[t], ref[t]) < ftol

    up = syn.upstream_grads(b, ac, dtype=dt)
    # gradient reference: double oracle on the dt-rounded inputs
    gref = oracle_mod.featurize_grad(*(v.astype(np.float64) for v in (x, y, z)), *common,
                                     *[u.astype(np.float64) for u in up])
    go = [np.zeros(b.n_atoms, dt) for _ in range(3)]
    getattr(hostmath, "hostmath_featurize_grad_" + suf)(
        _p(x), _p(y), _p(z), _p(b.atomic_numbers), _p(b.mol_offsets), _p(b.mol_atom_counts),
        ctypes.c_int(b.n_mols), _p(si), *[_p(u) for u in up], *[_p(o) for o in go])
    for k in range(3):
        assert np.isfinite(go[k]).all()
        assert normwise(go[k], gref[k]) < gtol


def test_ed_harder_rmse_known_answer():
    """Two conformer groups worked by hand: group 1 true (2,1,3) / predicted (3,0,2): the lowest
    true value is the second, so the shift is +1 and the errors are (2,0,0); group 2 true
    (8,9,2,3) / predicted (7,8,4,1): shift -2, errors (-3,-3,0,-4).  The same example sits in
    khan/utils/helpers.py:71-80 of the reference."""
    import math
    from khan_b200.utils import ed_harder_rmse
    want = (math.sqrt(4 / 3) + math.sqrt((9 + 9 + 0 + 16) / 4)) / 2
    assert abs(ed_harder_rmse([[2, 1, 3], [8, 9, 2, 3]], [3, 0, 2, 7, 8, 4, 1]) - want) < 1e-15


def test_split_rows_equals_numpy_split():
    from khan_b200.training.trainer_multi_tower import _split_rows
    rng = np.random.default_rng(8)
    counts = rng.integers(0, 9, 200)
    offsets = (np.cumsum(counts) - counts).astype(np.int32)
    rows = rng.normal(size=(int(counts.sum()), 3))
    got, want = _split_rows(rows, offsets), np.split(rows, offsets[1:])
    assert len(got) == len(want) == 200
    assert all(np.array_equal(a, b) for a, b in zip(got, want))
