"""TEST INFRASTRUCTURE ONLY: numpy front end of the CPU oracle.

Three interchangeable back ends compute the ANI-1 AEV path on the host:

``port``      ``libani_oracle.so`` -- the plain-C restatement in ``ani_oracle.c``.
``ref``       ``_ref/libani_ref_o2.so`` -- the reference's own
              ``gpu_featurizer/kernel_cpu.cpp`` compiled unmodified with -O2 and IEEE
              arithmetic (the parity oracle).
``ref_fast``  ``_ref/libani_ref_fast.so`` -- the same source with the reference
              Makefile's ``-O3 -Ofast`` (the timed CPU baseline).

Only ``tests/``, the smoke check and the bench's CPU-baseline legs may import this
package; the product (``khan_b200``) never does.

The wrappers mirror the reference's functor layer: outputs are allocated here from
``atom_counts`` and zero-filled before the kernel runs, as
``gpu_featurizer/functor_op_cpu.cpp:31-38,68-78,107-114`` does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
FEATURE_SIZE = 384

_PORT_PATH = os.path.join(_HERE, "libani_oracle.so")
_REF_PATHS = {
    "ref": os.path.join(_HERE, "_ref", "libani_ref_o2.so"),
    "ref_fast": os.path.join(_HERE, "_ref", "libani_ref_fast.so"),
}
_libs: dict = {}
_lock = threading.Lock()


def build(verbose: bool = False) -> None:
    """Run ``make`` beside this file (port always; ``_ref`` when the reference is there)."""
    out = subprocess.run(["make", "-C", _HERE], capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if verbose:
        print(out.stdout)


def available(impl: str) -> bool:
    path = _PORT_PATH if impl == "port" else _REF_PATHS[impl]
    return os.path.exists(path)


def best_impl() -> str:
    """The reference build when present, else the port."""
    return "ref" if available("ref") else "port"


def _lib(impl: str):
    with _lock:
        if impl in _libs:
            return _libs[impl]
        path = _PORT_PATH if impl == "port" else _REF_PATHS[impl]
        if not os.path.exists(path):
            if impl == "port":
                build()
            else:
                raise FileNotFoundError(f"oracle back end {impl!r} not built: {path}")
        _libs[impl] = ctypes.CDLL(path)
        return _libs[impl]


def _ptr(a: np.ndarray, offset_elems: int = 0):
    return ctypes.c_void_p(a.ctypes.data + offset_elems * a.itemsize)


def _sym(impl: str, op: str, dtype) -> "ctypes._CFuncPtr":
    suf = "f32" if np.dtype(dtype) == np.float32 else "f64"
    prefix = "oracle" if impl == "port" else "ref"
    fn = getattr(_lib(impl), f"{prefix}_{op}_{suf}")
    fn.restype = None
    return fn


def _i32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


def ani_sort(atomic_numbers):
    """AniSort (gpu_featurizer/ani_sort.cpp:71-115): returns scatter, gather, counts[4]."""
    a = _i32(atomic_numbers)
    n = a.shape[0]
    scatter = np.zeros(n, np.int32)
    gather = np.zeros(n, np.int32)
    counts = np.zeros(4, np.int32)
    fn = _lib("port").oracle_ani_sort
    fn.restype = None
    fn(_ptr(a), ctypes.c_int(n), _ptr(scatter), _ptr(gather), _ptr(counts))
    return scatter, gather, counts


def _chunks(n_mols: int, threads: int):
    threads = max(1, min(threads, n_mols)) if n_mols else 1
    edges = np.linspace(0, n_mols, threads + 1).astype(int)
    return [(int(edges[i]), int(edges[i + 1])) for i in range(threads) if edges[i + 1] > edges[i]]


def _run_chunked(call, n_mols: int, threads: int):
    parts = _chunks(n_mols, threads)
    if len(parts) <= 1:
        for s, e in parts:
            call(s, e)
        return
    with ThreadPoolExecutor(len(parts)) as ex:
        list(ex.map(lambda se: call(*se), parts))


def featurize(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs,
              atom_counts, impl: str = "port", threads: int = 1):
    """Featurize forward; returns the four flat per-element buffers (H, C, N, O)."""
    dt = np.asarray(xs).dtype
    xs, ys, zs = (np.ascontiguousarray(v, dtype=dt) for v in (xs, ys, zs))
    a, mo, mac, si = map(_i32, (atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs))
    acs = _i32(atom_counts)
    outs = [np.zeros(int(acs[t]) * FEATURE_SIZE, dt) for t in range(4)]
    fn = _sym(impl, "featurize", dt)

    def call(s, e):
        fn(_ptr(xs), _ptr(ys), _ptr(zs), _ptr(a), _ptr(mo, s), _ptr(mac, s), ctypes.c_int(e - s),
           _ptr(si), *[_ptr(o) for o in outs])

    # NOTE: the radial loop also writes row(j) of a partner atom, always inside the same
    # molecule, so molecule chunks touch disjoint rows.
    _run_chunked(call, mo.shape[0], threads)
    return outs


def featurize_grad(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs,
                   atom_counts, h_grads, c_grads, n_grads, o_grads, impl: str = "port",
                   threads: int = 1):
    """FeaturizeGrad (vector-Jacobian product); returns x_grads, y_grads, z_grads."""
    dt = np.asarray(xs).dtype
    xs, ys, zs = (np.ascontiguousarray(v, dtype=dt) for v in (xs, ys, zs))
    a, mo, mac, si = map(_i32, (atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs))
    gs = [np.ascontiguousarray(g, dtype=dt).reshape(-1) for g in (h_grads, c_grads, n_grads, o_grads)]
    outs = [np.zeros(xs.shape[0], dt) for _ in range(3)]
    fn = _sym(impl, "featurize_grad", dt)

    def call(s, e):
        fn(_ptr(xs), _ptr(ys), _ptr(zs), _ptr(a), _ptr(mo, s), _ptr(mac, s), ctypes.c_int(e - s),
           _ptr(si), *[_ptr(g) for g in gs], *[_ptr(o) for o in outs])

    _run_chunked(call, mo.shape[0], threads)
    return outs


def featurize_grad_inverse(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts,
                           scatter_idxs, atom_counts, x_grads, y_grads, z_grads,
                           impl: str = "port", threads: int = 1, reference_indexing: bool = False):
    """FeaturizeGradInverse; returns four flat per-element buffers.

    ``reference_indexing`` (port only) selects the reference's own indexing of the input
    vector by the central atom's element id (gpu_featurizer/kernel_cpu.cpp:111-169);
    the default is the Jacobian-vector product.
    """
    dt = np.asarray(xs).dtype
    xs, ys, zs = (np.ascontiguousarray(v, dtype=dt) for v in (xs, ys, zs))
    a, mo, mac, si = map(_i32, (atomic_numbers, mol_offsets, mol_atom_counts, scatter_idxs))
    acs = _i32(atom_counts)
    vs = [np.ascontiguousarray(v, dtype=dt) for v in (x_grads, y_grads, z_grads)]
    outs = [np.zeros(int(acs[t]) * FEATURE_SIZE, dt) for t in range(4)]
    fn = _sym(impl, "featurize_grad_inverse", dt)
    extra = [ctypes.c_int(1 if reference_indexing else 0)] if impl == "port" else []

    def call(s, e):
        fn(_ptr(xs), _ptr(ys), _ptr(zs), _ptr(a), _ptr(mo, s), _ptr(mac, s), ctypes.c_int(e - s),
           _ptr(si), *[_ptr(v) for v in vs], *[_ptr(o) for o in outs], *extra)

    _run_chunked(call, mo.shape[0], threads)
    return outs


def ani_charge(xs, ys, zs, qs, mol_offsets, mol_atom_counts):
    """AniCharge (gpu_featurizer/ani_charges.cpp:58-113): damped Coulomb energy per molecule."""
    dt = np.asarray(xs).dtype
    xs, ys, zs, qs = (np.ascontiguousarray(v, dtype=dt) for v in (xs, ys, zs, qs))
    mo, mac = map(_i32, (mol_offsets, mol_atom_counts))
    out = np.zeros(mo.shape[0], dt)
    _sym("port", "charge", dt)(_ptr(xs), _ptr(ys), _ptr(zs), _ptr(qs), _ptr(mo), _ptr(mac),
                               ctypes.c_int(mo.shape[0]), _ptr(out))
    return out


def ani_charge_grad(xs, ys, zs, qs, mol_offsets, mol_atom_counts, grads):
    """AniChargeGrad (gpu_featurizer/ani_charges.cpp:138-214): dL/dq from dL/dE per molecule."""
    dt = np.asarray(xs).dtype
    xs, ys, zs, qs, grads = (np.ascontiguousarray(v, dtype=dt) for v in (xs, ys, zs, qs, grads))
    mo, mac = map(_i32, (mol_offsets, mol_atom_counts))
    out = np.zeros(xs.shape[0], dt)
    _sym("port", "charge_grad", dt)(_ptr(xs), _ptr(ys), _ptr(zs), _ptr(qs), _ptr(mo), _ptr(mac),
                                    ctypes.c_int(mo.shape[0]), ctypes.c_int(xs.shape[0]), _ptr(grads), _ptr(out))
    return out


def count_work(xs, ys, zs, mol_offsets, mol_atom_counts):
    """(radial pairs, angular triplets) of a batch, with the forward's float comparisons."""
    xs, ys, zs = (np.ascontiguousarray(v, dtype=np.float32) for v in (xs, ys, zs))
    mo, mac = _i32(mol_offsets), _i32(mol_atom_counts)
    p = ctypes.c_longlong(0)
    t = ctypes.c_longlong(0)
    fn = _lib("port").oracle_count_work_f32
    fn.restype = None
    fn(_ptr(xs), _ptr(ys), _ptr(zs), _ptr(mo), _ptr(mac), ctypes.c_int(mo.shape[0]),
       ctypes.byref(p), ctypes.byref(t))
    return int(p.value), int(t.value)


def linearize(i: int, j: int, k: int, l: int) -> int:
    fn = _lib("port").oracle_linearize
    fn.restype = ctypes.c_int
    return int(fn(i, j, k, l))
