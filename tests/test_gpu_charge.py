"""GPU parity of AniCharge / AniChargeGrad against the CPU oracle (through ani_mod -> C ABI).

Tolerances: normwise 1e-5 (float32) and 1e-12 (float64), the same as for the featurizer.  The
float32 result is compared with the float64 oracle on the float32-rounded inputs as well, and
the reference's own finite-difference check (gpu_featurizer/test_kernel.py:398-447) is repeated
on the GPU."""
import numpy as np
import pytest

from conftest import normwise
from khan_b200.data import synthetic as syn

pytestmark = pytest.mark.gpu

TOL = {np.float32: 1e-5, np.float64: 1e-12}
CASES = {
    "kat": lambda: syn.kat_fixture(),
    "config1_part": lambda: syn.config1(n_mols=200),
    "config4_part": lambda: syn.config4(n_mols=4, n_min=64, n_max=200),
}


@pytest.fixture(scope="module")
def gpu():
    import torch
    assert torch.cuda.is_available()
    import gpu_util
    return gpu_util


def _charges(b, dt, seed=5):
    return np.random.default_rng(seed).normal(scale=0.4, size=b.n_atoms).astype(dt)


@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_energy_and_gradient_vs_oracle(gpu, oracle_mod, case, dt):
    from khan_b200 import ani_mod
    b = CASES[case]()
    q = _charges(b, dt)
    g = np.random.default_rng(6).normal(size=b.n_mols).astype(dt)
    x, y, z = b.coords(dt)
    x_t, y_t, z_t, _, mo, mac = gpu.batch_tensors(b, dt)
    e = ani_mod.ani_charge(x_t, y_t, z_t, gpu.to_dev(q), mo, mac).cpu().numpy()
    dq = ani_mod.ani_charge_grad(x_t, y_t, z_t, gpu.to_dev(q), mo, mac, gpu.to_dev(g)).cpu().numpy()
    ani_mod.check_device_status("ani_charge")
    args = (b.mol_offsets, b.mol_atom_counts)
    for ref_dt in {dt, np.float64}:
        cast = [c.astype(ref_dt) for c in (x, y, z, q)]
        e_ref = oracle_mod.ani_charge(*cast, *args)
        dq_ref = oracle_mod.ani_charge_grad(*cast, *args, g.astype(ref_dt))
        assert e.dtype == dt and e.shape == e_ref.shape and dq.shape == dq_ref.shape
        assert normwise(e, e_ref) < TOL[dt], (case, ref_dt)
        assert normwise(dq, dq_ref) < TOL[dt], (case, ref_dt)


def test_gradient_error_on_the_reference_fixture(gpu):
    import torch
    from khan_b200 import ani_mod
    b = syn.kat_fixture()
    x, y, z, _, mo, mac = gpu.batch_tensors(b, np.float64)
    q = gpu.to_dev(np.array([0.3, 4.5, 2.2, 3.4, -5.6, 3.4, 1.1, 3.2, 1.0, 0.3, 2.4]))
    q.requires_grad_(True)
    fn = lambda qq: ani_mod.ani_charge_autograd(x, y, z, qq, mo, mac)
    assert torch.autograd.gradcheck(fn, (q,), eps=1e-3, atol=1e-11, rtol=0)


def test_ragged_tables(gpu, oracle_mod):
    """Empty and one-atom molecules, a molecule left out of the table, and an empty batch."""
    import torch
    from khan_b200 import ani_mod
    b = syn.config1(n_mols=9)
    dt = np.float64
    x, y, z = b.coords(dt)
    q = _charges(b, dt)
    offs = np.concatenate([b.mol_offsets[:-1], [3, b.mol_offsets[-1]]]).astype(np.int32)   # last molecule dropped
    cnts = np.concatenate([b.mol_atom_counts[:-1], [0, 1]]).astype(np.int32)   # + an empty and a single
    g = np.arange(1, len(offs) + 1, dtype=dt)
    t = [gpu.to_dev(v) for v in (x, y, z, q)]
    e = ani_mod.ani_charge(*t, gpu.to_dev(offs), gpu.to_dev(cnts)).cpu().numpy()
    assert np.allclose(e, oracle_mod.ani_charge(x, y, z, q, offs, cnts), rtol=1e-12, atol=1e-15)
    assert e[-1] == 0 and e[-2] == 0
    # the one-atom molecule is the first atom of the dropped one: no overlap, zero gradient
    dq = ani_mod.ani_charge_grad(*t, gpu.to_dev(offs), gpu.to_dev(cnts), gpu.to_dev(g)).cpu().numpy()
    ref = oracle_mod.ani_charge_grad(x, y, z, q, offs[:-2], cnts[:-2], g[:-2])
    assert np.allclose(dq, ref, rtol=1e-12, atol=1e-15)
    assert np.all(dq[b.mol_offsets[-1]:] == 0)
    empty_f = torch.empty(0, dtype=torch.float64, device=gpu.DEV)
    empty_i = torch.empty(0, dtype=torch.int32, device=gpu.DEV)
    assert ani_mod.ani_charge(empty_f, empty_f, empty_f, empty_f, empty_i, empty_i).numel() == 0
    assert ani_mod.ani_charge_grad(empty_f, empty_f, empty_f, empty_f, empty_i, empty_i, empty_f).numel() == 0
    ani_mod.check_device_status("ani_charge")


def test_bad_molecule_table_is_reported_not_dereferenced(gpu):
    from khan_b200 import ani_mod, _lib
    b = syn.kat_fixture()
    x, y, z, _, mo, mac = gpu.batch_tensors(b, np.float32)
    q = gpu.to_dev(np.ones(b.n_atoms, np.float32))
    bad = gpu.to_dev(np.array([0, 9], np.int32))     # second molecule would run past the batch
    e = ani_mod.ani_charge(x, y, z, q, bad, gpu.to_dev(np.array([8, 5], np.int32)))
    assert ani_mod.device_status() == -6
    assert float(e[1]) == 0.0
