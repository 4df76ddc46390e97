"""GPU parity: the CUDA path, called through the C ABI (ani_mod -> ctypes -> libani_b200.so),
against the CPU oracle and the committed golden vectors of the reference.

Tolerances (normwise, max|a-b| <= tol * max|b| per output array):
  features   float32 1e-5 vs the float32 reference;   float64 1e-12
  gradients  float32 1e-5 vs the float64 reference evaluated on the float32-rounded inputs
             (the reference's float32 gradient is non-finite on part of realistic inputs);
             float64 1e-12
Sort indices are compared bit for bit.
"""
import numpy as np
import pytest

from conftest import normwise
from khan_b200.data import synthetic as syn

pytestmark = pytest.mark.gpu

ELEMS = "hcno"
FTOL = {np.float32: 1e-5, np.float64: 1e-12}


@pytest.fixture(scope="module")
def gpu():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import gpu_util
    return gpu_util


@pytest.fixture(scope="module")
def ref_impl(oracle_mod):
    return oracle_mod.best_impl()


# --------------------------------------------------------------------------- sort
def test_sort_known_answer(gpu):
    b = syn.kat_fixture()
    si, gi, ac = gpu.gpu_sort(b.atomic_numbers)
    np.testing.assert_array_equal(ac, [6, 2, 3, 0])
    np.testing.assert_array_equal(si, [0, 0, 1, 0, 1, 2, 3, 4, 5, 1, 2])
    np.testing.assert_array_equal(gi, [0, 8, 1, 6, 9, 2, 3, 4, 5, 7, 10])


@pytest.mark.parametrize("n", [0, 1, 31, 32, 33, 1023, 1024, 1025, 4097, 13727, 65536, 65537,
                               200001, 3000017])
def test_sort_bit_exact(gpu, oracle_mod, n):
    rng = np.random.default_rng(n)
    p = rng.dirichlet(np.ones(4)) if n % 2 else np.array([0.67, 0.24, 0.045, 0.045])
    a = rng.choice(4, size=n, p=p).astype(np.int32)
    si, gi, ac = gpu.gpu_sort(a)
    esi, egi, eac = oracle_mod.ani_sort(a)
    np.testing.assert_array_equal(ac, eac)
    np.testing.assert_array_equal(si, esi)
    np.testing.assert_array_equal(gi, egi)


def test_sort_single_element_and_sorted_inputs(gpu, oracle_mod):
    for a in (np.zeros(5000, np.int32), np.full(70000, 3, np.int32),
              np.sort(np.random.default_rng(0).integers(0, 4, 9000)).astype(np.int32),
              np.sort(np.random.default_rng(1).integers(0, 4, 9000))[::-1].astype(np.int32)):
        si, gi, ac = gpu.gpu_sort(a)
        esi, egi, eac = oracle_mod.ani_sort(a)
        np.testing.assert_array_equal(ac, eac)
        np.testing.assert_array_equal(si, esi)
        np.testing.assert_array_equal(gi, egi)


def _host_sort(a):
    order = np.argsort(a, kind="stable")
    gather = np.empty(a.size, np.int64)
    gather[order] = np.arange(a.size)
    counts = np.bincount(a, minlength=4)
    starts = np.concatenate([[0], np.cumsum(counts)])[:4]
    return gather - starts[a], gather, counts


def test_large_sorts_on_two_streams_do_not_share_scratch(gpu):
    """Batches above 65,536 atoms use a scratch buffer that the library keeps per (device, stream): two
    sorts in flight on two streams must both come out right."""
    import ctypes
    import torch
    from khan_b200 import _lib
    lib = _lib.lib()
    rng = np.random.default_rng(31)
    arrays = [rng.integers(0, 4, n).astype(np.int32) for n in (400_003, 333_337)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    dev_in = [gpu.to_dev(a) for a in arrays]
    outs = [[torch.empty(a.size, dtype=torch.int32, device=gpu.DEV), torch.empty(a.size, dtype=torch.int32, device=gpu.DEV),
             torch.empty(4, dtype=torch.int32, device=gpu.DEV)] for a in arrays]
    torch.cuda.synchronize()
    for _ in range(3):      # several rounds, so that the two streams really overlap
        for a, d, o, st in zip(arrays, dev_in, outs, streams):
            assert lib.ani_sort(d.data_ptr(), a.size, o[0].data_ptr(), o[1].data_ptr(), o[2].data_ptr(),
                                ctypes.c_void_p(st.cuda_stream)) == 0
    torch.cuda.synchronize()
    for a, o in zip(arrays, outs):
        scatter, gather, counts = _host_sort(a)
        np.testing.assert_array_equal(o[0].cpu().numpy(), scatter)
        np.testing.assert_array_equal(o[1].cpu().numpy(), gather)
        np.testing.assert_array_equal(o[2].cpu().numpy(), counts)


def test_large_sort_refuses_to_allocate_inside_a_stream_capture(gpu):
    """The first large sort on a stream has to allocate its scratch, which a stream capture cannot
    record: the call is refused (nothing launched) and works in the same capture once the scratch exists."""
    import ctypes
    import torch
    from khan_b200 import _lib
    lib = _lib.lib()
    a = np.random.default_rng(32).integers(0, 4, 70_001).astype(np.int32)
    d = gpu.to_dev(a)
    o = [torch.empty(a.size, dtype=torch.int32, device=gpu.DEV), torch.empty(a.size, dtype=torch.int32, device=gpu.DEV),
         torch.empty(4, dtype=torch.int32, device=gpu.DEV)]

    def call(stream):
        return lib.ani_sort(d.data_ptr(), a.size, o[0].data_ptr(), o[1].data_ptr(), o[2].data_ptr(),
                            ctypes.c_void_p(stream.cuda_stream))

    fresh = torch.cuda.Stream()      # a stream the library has never seen: no scratch yet
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(fresh):
        g.capture_begin()
        refused = call(fresh)
        g.capture_end()
    assert refused == -10 and "captur" in lib.ani_status_string(-10).decode()
    assert call(fresh) == 0          # outside a capture: allocates
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.stream(fresh):
        g2.capture_begin()
        recorded = call(fresh)
        g2.capture_end()
    assert recorded == 0
    o[1].zero_()
    g2.replay()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(o[1].cpu().numpy(), _host_sort(a)[1])


def test_sort_rejects_bad_element(gpu):
    from khan_b200 import ani_mod
    a = np.array([0, 1, 7, 2], np.int32)
    gpu.gpu_sort(a)
    assert ani_mod.device_status() == -4
    assert ani_mod.device_status() == 0  # reading clears it


# --------------------------------------------------------------------------- forward
@pytest.mark.parametrize("fixture", ["kat.npz", "c0_head.npz"])
@pytest.mark.parametrize("tag,dt", [("f32", np.float32), ("f64", np.float64)])
def test_forward_golden(gpu, golden, fixture, tag, dt):
    g = golden(fixture)
    b = syn.Batch(g["xs"], g["ys"], g["zs"], g["atomic_numbers"], g["mol_offsets"],
                  g["mol_atom_counts"])
    feats = gpu.gpu_featurize(b, dt)
    for t, e in enumerate(ELEMS):
        assert feats[t].shape == g[f"feat_{e}_{tag}"].shape
        assert normwise(feats[t], g[f"feat_{e}_{tag}"]) < FTOL[dt]


def test_forward_config0_checksums(gpu, golden):
    g = golden("c0_sums.npz")
    b = syn.Batch(g["xs"], g["ys"], g["zs"], g["atomic_numbers"], g["mol_offsets"],
                  g["mol_atom_counts"])
    for tag, dt, tol in (("f32", np.float32, 1e-5), ("f64", np.float64, 1e-12)):
        feats = gpu.gpu_featurize(b, dt)
        s = np.array([f.astype(np.float64).sum() for f in feats])
        s2 = np.array([(f.astype(np.float64) ** 2).sum() for f in feats])
        np.testing.assert_allclose(s, g["sum_" + tag], rtol=tol * 10)
        np.testing.assert_allclose(s2, g["sumsq_" + tag], rtol=tol * 10)


def _concat(*batches):
    """Several batches as one (molecules of the first, then of the second, ...)."""
    offs, base = [], 0
    for b in batches:
        offs.append(b.mol_offsets + base)
        base += b.n_atoms
    return syn.Batch(*(np.concatenate([getattr(b, f) for b in batches]) for f in ("xs", "ys", "zs", "atomic_numbers")),
                     np.concatenate(offs).astype(np.int32),
                     np.concatenate([b.mol_atom_counts for b in batches]).astype(np.int32))


def _dense_blobs(n_mols, n, radius, seed):
    """Molecules of n atoms inside a small sphere: more than 24 neighbours within A_Rc around most atoms."""
    rng = np.random.default_rng(seed)
    mols = []
    for _ in range(n_mols):
        pos = np.zeros((n, 3))
        k = 0
        while k < n:
            c = rng.uniform(-radius, radius, 3)
            if c @ c > radius * radius or (k and np.min(np.sum((pos[:k] - c) ** 2, axis=1)) < 0.36):
                continue
            pos[k] = c
            k += 1
        mols.append((rng.integers(0, 4, n).astype(np.int32), pos))
    return syn._assemble(mols)


CASES = {
    # small molecules with a 40- and a 70-atom molecule among them: the batch takes the kernels for
    # small molecules (mean size), the two large ones their in-kernel route
    "large_among_small": lambda: _concat(syn.gdb_like_batch(60, 3), syn.config4(seed=5, n_mols=2, n_min=40, n_max=70),
                                         syn.gdb_like_batch(30, 4)),
    # 30 atoms within 2.2 A of a point: up to 29 neighbours within A_Rc (the angular lists hold 24)
    "dense_small": lambda: _concat(_dense_blobs(3, 30, 2.2, 6), syn.gdb_like_batch(20, 8, heavy_min=1, heavy_max=2)),
    "exactly_32_atoms": lambda: _concat(syn.config4(seed=6, n_mols=5, n_min=32, n_max=32),
                                        syn.gdb_like_batch(40, 9, heavy_min=1, heavy_max=3)),
    "config0": lambda: syn.config0(),
    "config1": lambda: syn.config1(),
    "config4_part": lambda: syn.config4(n_mols=12),
    "tiny_mols": lambda: syn.gdb_like_batch(40, 7, heavy_min=1, heavy_max=1),
    "mid_33_to_70_atoms": lambda: syn.config4(seed=9, n_mols=6, n_min=33, n_max=70),
    # batches that take the kernels for larger molecules, with neighbourhoods beyond their lists: 40 atoms
    # within 2.3 A of a point (up to 39 neighbours within A_Rc, the angular lists hold 32) and 80 atoms
    # within 2.25 A (79 neighbours within R_Rc, the radial lists hold 64)
    "dense_large": lambda: _concat(_dense_blobs(2, 40, 2.3, 11), syn.config4(seed=7, n_mols=4, n_min=40, n_max=90)),
    "very_dense_large": lambda: _concat(_dense_blobs(1, 80, 2.25, 12),
                                        syn.config4(seed=8, n_mols=3, n_min=40, n_max=60)),
}


@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_forward_vs_oracle(gpu, oracle_mod, ref_impl, case, dt):
    b = CASES[case]()
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    x, y, z = b.coords(dt)
    ref = oracle_mod.featurize(x, y, z, b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac,
                               impl=ref_impl, threads=8)
    feats = gpu.gpu_featurize(b, dt)
    for t in range(4):
        assert feats[t].shape == ref[t].shape
        assert normwise(feats[t], ref[t]) < FTOL[dt], (case, t)


def test_sort_no_scratch_and_scratch_paths_agree(gpu, oracle_mod):
    # 65536 atoms take the single-launch path, 65537 the three-launch path with scratch
    rng = np.random.default_rng(77)
    a = rng.integers(0, 4, 65537).astype(np.int32)
    big = gpu.gpu_sort(a)
    small = gpu.gpu_sort(a[:65536])
    e_big, e_small = oracle_mod.ani_sort(a), oracle_mod.ani_sort(a[:65536])
    for got, exp in ((big, e_big), (small, e_small)):
        for g, e in zip(got, exp):
            np.testing.assert_array_equal(g, e)


def test_forward_is_bit_reproducible(gpu):
    b = syn.config1(n_mols=256)
    one = gpu.gpu_featurize(b, np.float32)
    two = gpu.gpu_featurize(b, np.float32)
    for a, c in zip(one, two):
        np.testing.assert_array_equal(a, c)


def test_forward_overwrites_stale_output(gpu, oracle_mod):
    # no pre-zero requirement: rows are fully written even where the features are zero
    import torch
    from khan_b200 import ani_mod
    b = syn.kat_fixture()
    x, y, z, a, mo, mac = gpu.batch_tensors(b, np.float32)
    si, gi, ac = ani_mod.ani_sort(a)
    acs = ac.cpu().numpy()
    out = torch.full((b.n_atoms, 384), float("nan"), device=x.device)
    ani_mod.featurize_into(x, y, z, a, mo, mac, si, acs, out)
    assert torch.isfinite(out).all()


# --------------------------------------------------------------------------- gradient
@pytest.mark.parametrize("fixture", ["kat.npz", "c0_head.npz"])
@pytest.mark.parametrize("tag,dt", [("f32", np.float32), ("f64", np.float64)])
def test_gradient_golden(gpu, golden, fixture, tag, dt):
    g = golden(fixture)
    b = syn.Batch(g["xs"], g["ys"], g["zs"], g["atomic_numbers"], g["mol_offsets"],
                  g["mol_atom_counts"])
    up = [g["up_" + e] for e in ELEMS]
    out = gpu.gpu_featurize_grad(b, dt, up)
    for k, c in enumerate("xyz"):
        assert np.isfinite(out[k]).all()
        assert normwise(out[k], g[f"grad_{c}_{tag}"]) < FTOL[dt]


@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_gradient_vs_oracle(gpu, oracle_mod, case, dt):
    b = CASES[case]()
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    up = syn.upstream_grads(b, ac, dtype=dt)
    x, y, z = b.coords(dt)
    ref = oracle_mod.featurize_grad(*(v.astype(np.float64) for v in (x, y, z)), b.atomic_numbers,
                                    b.mol_offsets, b.mol_atom_counts, si, ac,
                                    *[u.astype(np.float64) for u in up], impl="port", threads=8)
    out = gpu.gpu_featurize_grad(b, dt, up)
    for k in range(3):
        assert np.isfinite(out[k]).all()
        assert normwise(out[k], ref[k]) < FTOL[dt], (case, k)


def test_float32_gradient_vs_the_float32_reference_where_it_is_finite(gpu, oracle_mod, ref_impl):
    """The reference's own float32 gradient divides by sin(theta) and by 1 + cos(theta_t - theta) without a
    guard (gpu_featurizer/kernel_cpu.cpp:335-353) and is non-finite for part of realistic inputs, so the
    primary check above uses its float64 build.  Here: on the atoms where the float32 reference IS finite,
    the GPU agrees with it too; how many atoms it loses is printed."""
    b = syn.config1(n_mols=256)
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    up = syn.upstream_grads(b, ac, dtype=np.float32)
    x, y, z = b.coords(np.float32)
    ref32 = oracle_mod.featurize_grad(x, y, z, b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac, *up,
                                      impl=ref_impl, threads=8)
    ref64 = oracle_mod.featurize_grad(*(v.astype(np.float64) for v in (x, y, z)), b.atomic_numbers, b.mol_offsets,
                                      b.mol_atom_counts, si, ac, *[u.astype(np.float64) for u in up],
                                      impl="port", threads=8)
    out = gpu.gpu_featurize_grad(b, np.float32, up)
    finite = np.isfinite(ref32[0]) & np.isfinite(ref32[1]) & np.isfinite(ref32[2])
    # one non-finite term poisons the sums of its whole molecule in the reference: compare molecule-wise
    mol_of = np.repeat(np.arange(b.n_mols), b.mol_atom_counts)
    good_mol = np.ones(b.n_mols, bool)
    good_mol[mol_of[~finite]] = False
    keep = good_mol[mol_of]
    print(f"float32 reference gradient: {int((~finite).sum())} of {b.n_atoms} atoms non-finite, "
          f"{int((~good_mol).sum())} of {b.n_mols} molecules affected")
    assert keep.sum() > b.n_atoms // 2
    for k in range(3):
        assert np.isfinite(out[k]).all()
        scale = np.abs(ref64[k]).max()
        # the float32 reference itself is only this close to its float64 build (cancellation in its
        # expanded expressions): the GPU must be at least as close to it as that, and within 1e-5 of float64
        ref_gap = np.abs(ref32[k][keep] - ref64[k][keep]).max() / scale
        assert np.abs(out[k][keep] - ref32[k][keep]).max() / scale < max(1e-5, 2 * ref_gap)
        assert np.abs(out[k] - ref64[k]).max() / scale < 1e-5


def test_config4_at_full_size(gpu, oracle_mod, ref_impl):
    """Benchmark configuration 4 as stated: 256 molecules of 64-256 atoms, float32.  Forward against the
    reference build, gradient against the float64 oracle on the float32-rounded inputs."""
    b = syn.config4()
    assert b.n_mols == 256 and b.mol_atom_counts.min() >= 64 and b.mol_atom_counts.max() <= 256
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    x, y, z = b.coords(np.float32)
    ref = oracle_mod.featurize(x, y, z, b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac,
                               impl=ref_impl, threads=8)
    feats = gpu.gpu_featurize(b, np.float32)
    for t in range(4):
        assert normwise(feats[t], ref[t]) < 1e-5
    up = syn.upstream_grads(b, ac, dtype=np.float32)
    gref = oracle_mod.featurize_grad(*(v.astype(np.float64) for v in (x, y, z)), b.atomic_numbers, b.mol_offsets,
                                     b.mol_atom_counts, si, ac, *[u.astype(np.float64) for u in up],
                                     impl="port", threads=8)
    out = gpu.gpu_featurize_grad(b, np.float32, up)
    for k in range(3):
        assert np.isfinite(out[k]).all()
        assert normwise(out[k], gref[k]) < 1e-5


def test_gradient_is_bit_reproducible(gpu):
    """Batches of small molecules: every output is written once from a fixed summation order (no atomics),
    so two runs agree bit for bit, in both precisions."""
    b = syn.config1(n_mols=512)
    ac = np.bincount(b.atomic_numbers, minlength=4)
    for dt in (np.float32, np.float64):
        up = syn.upstream_grads(b, ac, dtype=dt)
        one = gpu.gpu_featurize_grad(b, dt, up)
        two = gpu.gpu_featurize_grad(b, dt, up)
        for a, c in zip(one, two):
            np.testing.assert_array_equal(a, c)


def test_gradient_takes_unaligned_upstream_buffers(gpu, oracle_mod):
    """Upstream buffers that are not 16-byte aligned cannot be fetched with 16-byte copies: the call takes
    the other kernel and gives the same result."""
    import torch
    from khan_b200 import ani_mod
    b = syn.config1(n_mols=64)
    x, y, z, a, mo, mac = gpu.batch_tensors(b, np.float32)
    si, gi, ac = ani_mod.ani_sort(a)
    acs = ac.cpu().numpy()
    up = syn.upstream_grads(b, acs, dtype=np.float32)
    aligned = ani_mod.featurize_grad(x, y, z, a, mo, mac, si, acs, *[gpu.to_dev(u) for u in up])
    shifted = []
    for u in up:   # a view that starts 4 bytes into an allocation
        buf = torch.empty(u.size + 1, dtype=torch.float32, device=x.device)
        buf[1:] = gpu.to_dev(u)
        shifted.append(buf[1:])
        assert buf[1:].data_ptr() % 16 == 4 or u.size == 0
    other = ani_mod.featurize_grad(x, y, z, a, mo, mac, si, acs, *shifted)
    ani_mod.check_device_status("featurize_grad")
    for p, q in zip(aligned, other):
        assert normwise(q.cpu().numpy(), p.cpu().numpy()) < 1e-5


def test_gradient_sums_to_zero_per_molecule(gpu):
    # translation invariance, a size-independent property checked at the full config-1 size
    b = syn.config1()
    ac = np.bincount(b.atomic_numbers, minlength=4)
    up = syn.upstream_grads(b, ac, dtype=np.float64)
    out = gpu.gpu_featurize_grad(b, np.float64, up)
    for k in range(3):
        per_mol = np.add.reduceat(out[k], b.mol_offsets)
        assert np.abs(per_mol).max() < 1e-9 * np.abs(out[k]).max()


def test_gradient_finite_differences_on_gpu(gpu):
    # gpu_featurizer/test_kernel.py:463-535 with the double settings (delta 1e-6, tol 1e-9 there;
    # central differences here)
    b = syn.kat_fixture()
    ac = np.bincount(b.atomic_numbers, minlength=4)
    rng = np.random.default_rng(2)
    up = [rng.normal(size=int(c) * 384) for c in ac]
    grads = gpu.gpu_featurize_grad(b, np.float64, up)

    def loss(xs):
        bb = syn.Batch(xs, b.ys, b.zs, b.atomic_numbers, b.mol_offsets, b.mol_atom_counts)
        f = gpu.gpu_featurize(bb, np.float64)
        return sum(float((a * c).sum()) for a, c in zip(f, up))

    for i in range(b.n_atoms):
        xp, xm = b.xs.copy(), b.xs.copy()
        xp[i] += 1e-6
        xm[i] -= 1e-6
        assert abs((loss(xp) - loss(xm)) / 2e-6 - grads[0][i]) < 1e-6


# --------------------------------------------------------------------------- edge cases
def test_empty_batch(gpu):
    import torch
    from khan_b200 import ani_mod
    e = torch.zeros(0, device=gpu.DEV)
    ei = torch.zeros(0, dtype=torch.int32, device=gpu.DEV)
    si, gi, ac = ani_mod.ani_sort(ei)
    assert ac.cpu().tolist() == [0, 0, 0, 0]
    feats = ani_mod.featurize(e, e, e, ei, ei, ei, si, ac)
    assert all(f.numel() == 0 for f in feats)
    gx, gy, gz = ani_mod.featurize_grad(e, e, e, ei, ei, ei, si, ac, *feats)
    assert gx.numel() == 0


def test_dense_cluster_takes_the_streaming_path(gpu, oracle_mod):
    # 120 atoms inside a 3 A sphere: more neighbours than the shared-memory lists hold
    rng = np.random.default_rng(5)
    n = 120
    pos = np.zeros((n, 3))
    k = 0
    while k < n:
        c = rng.uniform(-3.0, 3.0, 3)
        if c @ c > 9.0 or (k and np.min(np.sum((pos[:k] - c) ** 2, axis=1)) < 0.49):
            continue
        pos[k] = c
        k += 1
    types = rng.integers(0, 4, n).astype(np.int32)
    b = syn.Batch(pos[:, 0].copy(), pos[:, 1].copy(), pos[:, 2].copy(), types,
                  np.array([0], np.int32), np.array([n], np.int32))
    si, gi, ac = oracle_mod.ani_sort(types)
    for dt in (np.float32, np.float64):
        x, y, z = b.coords(dt)
        ref = oracle_mod.featurize(x, y, z, types, b.mol_offsets, b.mol_atom_counts, si, ac)
        feats = gpu.gpu_featurize(b, dt)
        for t in range(4):
            assert normwise(feats[t], ref[t]) < FTOL[dt]
        up = syn.upstream_grads(b, ac, dtype=dt)
        gref = oracle_mod.featurize_grad(*(v.astype(np.float64) for v in (x, y, z)), types,
                                         b.mol_offsets, b.mol_atom_counts, si, ac,
                                         *[u.astype(np.float64) for u in up])
        out = gpu.gpu_featurize_grad(b, dt, up)
        for k in range(3):
            assert normwise(out[k], gref[k]) < FTOL[dt]


def test_one_large_molecule(gpu, oracle_mod):
    # a single 700-atom molecule: every warp of the molecule walks 22 atoms, 22 scan chunks each
    b = syn.config4(seed=11, n_mols=1, n_min=700, n_max=700)
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    x, y, z = b.coords(np.float64)
    ref = oracle_mod.featurize(x, y, z, b.atomic_numbers, b.mol_offsets, b.mol_atom_counts, si, ac,
                               threads=1)
    feats = gpu.gpu_featurize(b, np.float64)
    for t in range(4):
        assert normwise(feats[t], ref[t]) < 1e-12
    up = syn.upstream_grads(b, ac, dtype=np.float64)
    gref = oracle_mod.featurize_grad(x, y, z, b.atomic_numbers, b.mol_offsets, b.mol_atom_counts,
                                     si, ac, *up)
    out = gpu.gpu_featurize_grad(b, np.float64, up)
    for k in range(3):
        assert normwise(out[k], gref[k]) < 1e-12


def test_unordered_molecule_table(gpu, oracle_mod):
    # molecule ranges listed in a shuffled order, with unused atoms between them
    b = syn.config1(n_mols=40)
    rng = np.random.default_rng(8)
    keep = np.sort(rng.choice(40, size=25, replace=False))
    order = rng.permutation(keep)
    shuffled = syn.Batch(b.xs, b.ys, b.zs, b.atomic_numbers, b.mol_offsets[order].copy(),
                         b.mol_atom_counts[order].copy())
    si, gi, ac = oracle_mod.ani_sort(b.atomic_numbers)
    x, y, z = b.coords(np.float32)
    ref = oracle_mod.featurize(x, y, z, b.atomic_numbers, shuffled.mol_offsets,
                               shuffled.mol_atom_counts, si, ac)
    import torch
    from khan_b200 import ani_mod
    xt, yt, zt, a, mo, mac = gpu.batch_tensors(shuffled, np.float32)
    out = torch.full((b.n_atoms, 384), 123.0, device=xt.device)
    ani_mod.featurize_into(xt, yt, zt, a, mo, mac, gpu.to_dev(si), ac.astype(np.int32), out)
    got = out.cpu().numpy()
    start = np.concatenate([[0], np.cumsum(ac)])
    used = np.zeros(b.n_atoms, bool)
    for off, cnt in zip(shuffled.mol_offsets, shuffled.mol_atom_counts):
        used[off:off + cnt] = True
    for t in range(4):
        rows = got[start[t]:start[t + 1]]
        mask = used[b.atomic_numbers == t]
        assert normwise(rows[mask], ref[t].reshape(-1, 384)[mask]) < 1e-5
        assert (rows[~mask] == 123.0).all()  # rows of atoms outside every molecule are untouched
    up = syn.upstream_grads(b, ac, dtype=np.float32)
    gref = oracle_mod.featurize_grad(*(v.astype(np.float64) for v in (x, y, z)), b.atomic_numbers,
                                     shuffled.mol_offsets, shuffled.mol_atom_counts, si, ac,
                                     *[u.astype(np.float64) for u in up])
    outg = gpu.gpu_featurize_grad(shuffled, np.float32, up, si=si, ac=ac)
    for k in range(3):
        assert normwise(outg[k], gref[k]) < 1e-5
        assert (outg[k][~used] == 0).all()


def test_inconsistent_offsets_are_reported_not_dereferenced(gpu):
    import torch
    from khan_b200 import ani_mod
    b = syn.kat_fixture()
    x, y, z, a, mo, mac = gpu.batch_tensors(b, np.float32)
    si, gi, ac = ani_mod.ani_sort(a)
    bad_mo = torch.tensor([0, 9], dtype=torch.int32, device=x.device)  # 9 + 3 > 11 atoms
    ani_mod.featurize(x, y, z, a, bad_mo, mac, si, ac)
    assert ani_mod.device_status() == -6


def test_rigid_motion_invariance_at_full_size(gpu):
    """Size-independent property at the full config-1 size: features do not change under a rigid
    motion of every molecule, and the coordinate gradient rotates with the coordinates."""
    b = syn.config1()
    rng = np.random.default_rng(17)
    q, _ = np.linalg.qr(rng.normal(size=(3, 3)))
    if np.linalg.det(q) < 0:
        q[:, 0] = -q[:, 0]
    shift = np.array([0.7, -1.3, 2.1])
    import copy
    moved = copy.copy(b)
    xyz = np.stack(b.coords(np.float64), axis=1) @ q.T + shift
    moved.xs, moved.ys, moved.zs = xyz[:, 0].copy(), xyz[:, 1].copy(), xyz[:, 2].copy()
    assert np.abs(np.stack(moved.coords(np.float64), axis=1) - xyz).max() == 0
    f0 = gpu.gpu_featurize(b, np.float64)
    f1 = gpu.gpu_featurize(moved, np.float64)
    for t in range(4):
        assert normwise(f1[t], f0[t]) < 1e-11
    ac = np.bincount(b.atomic_numbers, minlength=4)
    up = syn.upstream_grads(b, ac, dtype=np.float64)
    g0 = np.stack(gpu.gpu_featurize_grad(b, np.float64, up), axis=1)
    g1 = np.stack(gpu.gpu_featurize_grad(moved, np.float64, up), axis=1)
    assert np.abs(g1 - g0 @ q.T).max() < 1e-10 * np.abs(g0).max()
