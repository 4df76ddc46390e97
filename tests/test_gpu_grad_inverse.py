"""GPU parity of FeaturizeGradInverse (Jacobian-vector product) and of the autograd wiring.

Reference for the numbers: the CPU oracle's J v (``oracle.featurize_grad_inverse`` with the
default indexing).  The reference's own kernel multiplies by the vector entry at the central
atom's ELEMENT id (gpu_featurizer/kernel_cpu.cpp:111-169), which makes its output vanish; that
behaviour is pinned in tests/test_oracle.py and is not what the GPU entry point computes.
Tolerances: normwise 1e-5 (float32, against the float64 oracle on the float32-rounded inputs)
and 1e-12 (float64)."""
import numpy as np
import pytest

from conftest import normwise
from khan_b200.data import synthetic as syn

pytestmark = pytest.mark.gpu

TOL = {np.float32: 1e-5, np.float64: 1e-12}
CASES = {
    "kat": lambda: syn.kat_fixture(),
    "config1_part": lambda: syn.config1(n_mols=96),
    "config4_part": lambda: syn.config4(n_mols=3, n_min=64, n_max=120),
}


@pytest.fixture(scope="module")
def gpu():
    import torch
    assert torch.cuda.is_available()
    import gpu_util
    return gpu_util


def _gpu_jvp(gpu, batch, dt, v, si, ac):
    from khan_b200 import ani_mod
    x, y, z, a, mo, mac = gpu.batch_tensors(batch, dt)
    out = ani_mod.featurize_grad_inverse(x, y, z, a, mo, mac, gpu.to_dev(si), ac,
                                         *[gpu.to_dev(c.astype(dt)) for c in v])
    ani_mod.check_device_status("featurize_grad_inverse")
    return [o.cpu().numpy() for o in out]


@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_jvp_vs_oracle(gpu, oracle_mod, case, dt):
    b = CASES[case]()
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    rng = np.random.default_rng(21)
    v = [rng.normal(size=b.n_atoms).astype(dt) for _ in range(3)]
    x, y, z = b.coords(dt)
    ref = oracle_mod.featurize_grad_inverse(*(c.astype(np.float64) for c in (x, y, z)),
                                            b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si,
                                            ac, *[c.astype(np.float64) for c in v], threads=8)
    got = _gpu_jvp(gpu, b, dt, v, si, ac)
    for t in range(4):
        assert got[t].shape == ref[t].shape
        assert normwise(got[t], ref[t]) < TOL[dt], (case, t)


def test_jvp_is_the_transpose_of_the_vjp_on_the_gpu(gpu, oracle_mod):
    b = syn.config1(n_mols=64)
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    rng = np.random.default_rng(22)
    v = [rng.normal(size=b.n_atoms) for _ in range(3)]
    g = syn.upstream_grads(b, ac, dtype=np.float64)
    jv = _gpu_jvp(gpu, b, np.float64, v, si, ac)
    jtg = gpu.gpu_featurize_grad(b, np.float64, g, si=si, ac=ac)
    lhs = sum(float((a * c).sum()) for a, c in zip(g, jv))
    rhs = sum(float((a * c).sum()) for a, c in zip(jtg, v))
    assert abs(lhs - rhs) < 1e-10 * max(1.0, abs(lhs))


def test_autograd_first_and_second_order(gpu, oracle_mod):
    import torch
    from khan_b200 import ani_mod
    b = syn.kat_fixture()
    x, y, z, a, mo, mac = gpu.batch_tensors(b, np.float64)
    x.requires_grad_(True); y.requires_grad_(True); z.requires_grad_(True)
    si, gi, ac = ani_mod.ani_sort(a)
    acs = ac.cpu().numpy()
    feats = ani_mod.featurize_autograd(x, y, z, a, mo, mac, si, acs)
    w = [torch.linspace(-1.0, 1.0, f.numel(), dtype=f.dtype, device=f.device).requires_grad_(True)
         for f in feats]
    energy = sum((f * wi).sum() for f, wi in zip(feats, w) if f.numel())
    gx, gy, gz = torch.autograd.grad(energy, [x, y, z], create_graph=True)
    direct = ani_mod.featurize_grad(x.detach(), y.detach(), z.detach(), a, mo, mac, si, acs,
                                    *[wi.detach() for wi in w])
    for got, exp in zip((gx, gy, gz), direct):
        assert torch.allclose(got, exp, rtol=0, atol=1e-12)
    # second order: d(sum of forces)/d(weights) = J . ones, through FeaturizeGradInverse
    # (the structure of gpu_featurizer/test_kernel.py:353-400)
    force_loss = gx.sum() + 2.0 * gy.sum() - gz.sum()
    dw = torch.autograd.grad(force_loss, [wi for wi, f in zip(w, feats) if f.numel()])
    ones = [np.ones(b.n_atoms), 2.0 * np.ones(b.n_atoms), -np.ones(b.n_atoms)]
    esi, egi, eac = oracle_mod.ani_sort(b.atomic_numbers)
    ref = oracle_mod.featurize_grad_inverse(b.xs, b.ys, b.zs, b.atomic_numbers, b.mol_offsets,
                                            b.mol_atom_counts, esi, eac, *ones)
    ref = [r for r in ref if r.size]
    for got, exp in zip(dw, ref):
        assert normwise(got.cpu().numpy(), exp) < 1e-9 or np.abs(exp).max() < 1e-12
