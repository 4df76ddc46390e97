"""Loader and builder of ``libani_b200.so``, the C-ABI shared library of CUDA kernels.

The library is built in-tree (``khan_b200/libani_b200.so``) by :func:`build` with nvcc for
sm_100a only.  :func:`lib` fails loudly when the library is missing or does not load: there
is no CPU or eager fallback anywhere in this package.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("ANI_B200_LIB") or os.path.join(_HERE, "libani_b200.so")
CSRC = os.path.join(_HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(_HERE), "include")
SOURCES = ["ani_b200.cu"]
HEADERS = ["ani_params.h", "ani_common.cuh", "ani_device_math.cuh", "ani_feeder.h", "ani_peer.cuh", "ani_sort.cuh", "ani_featurize.cuh", "ani_featurize_mol.cuh", "ani_featurize_large.cuh", "ani_featurize_round_passes.inl", "ani_grad.cuh", "ani_grad_mol.cuh", "ani_grad_pair_pass.inl",
           "ani_grad_inverse.cuh", "ani_mlp.cuh", "ani_mlp_pipe.cuh", "ani_mlp_forward.cuh", "ani_mlp_backward.cuh", "ani_mlp_wgrad.cuh", "ani_charge.cuh", "ani_optim.cuh", "ani_energy.cuh", "ani_host_pack.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-pthread", "-shared",
]

_lock = threading.Lock()
_lib = None

c_int_p = ctypes.POINTER(ctypes.c_int)
_vp = ctypes.c_void_p
_i = ctypes.c_int

class MlpArgs(ctypes.Structure):
    """``ani_mlp_args`` of include/ani_b200.h: seventeen arrays of four device pointers."""
    _fields_ = [(name, ctypes.c_void_p * 4) for name in (
        "features", "w1", "b1", "w2", "b2", "w3", "b3", "w4", "b4", "energy", "act1", "act2", "act3",
        "dact1", "dact2", "dact3", "packed")]


class MlpPackArgs(ctypes.Structure):
    """``ani_mlp_pack_args`` of include/ani_b200.h."""
    _fields_ = [(name, ctypes.c_void_p * 4) for name in ("w1", "w2", "w3", "packed")]


class HostPackArgs(ctypes.Structure):
    """``ani_host_pack_args`` of include/ani_b200.h."""
    _fields_ = [("picks", ctypes.c_void_p), ("n_picks", ctypes.c_int), ("n_mols_total", ctypes.c_longlong),
                ("mol_ptr", ctypes.c_void_p), ("src_xyz", ctypes.c_void_p), ("src_stride", ctypes.c_longlong),
                ("src_is_f64", ctypes.c_int), ("src_types", ctypes.c_void_p), ("src_ys", ctypes.c_void_p),
                ("src_grads", ctypes.c_void_p), ("noise", ctypes.c_void_p), ("dst_xyz", ctypes.c_void_p),
                ("dst_grads", ctypes.c_void_p), ("dst_ys", ctypes.c_void_p), ("dst_stride", ctypes.c_longlong),
                ("dst_is_f64", ctypes.c_int), ("dst_types", ctypes.c_void_p), ("dst_mol_ids", ctypes.c_void_p),
                ("dst_mol_offsets", ctypes.c_void_p), ("dst_mol_counts", ctypes.c_void_p),
                ("cap_atoms", ctypes.c_int), ("cap_mols", ctypes.c_int), ("n_atoms_out", ctypes.c_void_p),
                ("acs_out", ctypes.c_void_p), ("src_mol_acs", ctypes.c_void_p)]


class FeederSlot(ctypes.Structure):
    """``ani_feeder_slot`` of include/ani_b200.h."""
    _fields_ = [("pack", HostPackArgs), ("host_arena", ctypes.c_void_p), ("dev_arena", ctypes.c_void_p),
                ("nbytes", ctypes.c_size_t)]


class FeederBatch(ctypes.Structure):
    """``ani_feeder_batch`` of include/ani_b200.h."""
    _fields_ = [("slot", ctypes.c_int), ("batch_index", ctypes.c_longlong), ("n_atoms", ctypes.c_int),
                ("n_mols", ctypes.c_int), ("acs", ctypes.c_int * 4)]


class PassArgs(ctypes.Structure):
    """``ani_pass_args`` of include/ani_b200.h."""
    _P4 = ctypes.c_void_p * 4
    _fields_ = ([("phases", ctypes.c_int), ("n_atoms", ctypes.c_int), ("n_mols", ctypes.c_int),
                 ("acs_host", ctypes.c_void_p), ("activation", ctypes.c_int), ("split_precision", ctypes.c_int)]
                + [(n, ctypes.c_void_p) for n in (
                    "xs", "ys", "zs", "atomic_numbers", "mol_offsets", "mol_atom_counts", "scatter_idxs", "gather_idxs",
                    "atom_counts", "features", "feature_grads", "x_grads", "y_grads", "z_grads", "energy_sorted",
                    "grad_energy_sorted", "act1", "act2", "act3", "dact1", "dact2", "dact3", "dz1", "dz2", "dz3",
                    "labels")]
                + [("grad_scale", ctypes.c_float), ("mol_energy", ctypes.c_void_p), ("l2s", ctypes.c_void_p)]
                + [(n, ctypes.c_void_p * 4) for n in (
                    "w1", "b1", "w2", "b2", "w3", "b3", "w4", "b4", "dw1", "db1", "dw2", "db2", "dw3", "db3", "dw4",
                    "db4", "packed")]
                + [("zero_ptr", ctypes.c_void_p), ("zero_bytes", ctypes.c_size_t)])


PASS_PACK, PASS_FEATURIZE, PASS_FORWARD, PASS_ENERGY, PASS_BACKWARD, PASS_WEIGHT_GRAD, PASS_COORD_GRAD = (
    1, 2, 4, 8, 16, 32, 64)


class MlpBackwardArgs(ctypes.Structure):
    """``ani_mlp_backward_args`` of include/ani_b200.h."""
    _fields_ = [(name, ctypes.c_void_p * 4) for name in (
        "grad_energy", "w1", "w2", "w3", "w4", "dact1", "dact2", "dact3", "dz1", "dz2", "dz3",
        "grad_features", "packed")]


class MlpWeightGradArgs(ctypes.Structure):
    """``ani_mlp_weight_grad_args`` of include/ani_b200.h."""
    _fields_ = [(name, ctypes.c_void_p * 4) for name in (
        "features", "act1", "act2", "dz1", "dz2", "dz3", "dw1", "dw2", "dw3", "db1", "db2", "db3",
        "act3", "grad_energy", "dw4", "db4")]


# name -> (restype, argtypes); one entry per declaration in include/ani_b200.h
SIGNATURES = {
    "ani_feature_size": (_i, []),
    "ani_status_string": (ctypes.c_char_p, [_i]),
    "ani_last_cuda_error": (ctypes.c_char_p, []),
    "ani_device_status": (_i, [_vp]),
    "ani_sort": (_i, [_vp, _i, _vp, _vp, _vp, _vp]),
    "ani_sort_noalloc": (_i, [_vp, _i, _vp, _vp, _vp, _vp]),
    "ani_sort_noalloc_max_atoms": (_i, []),
    "ani_featurize_f32": (_i, [_vp] * 6 + [_i] + [_vp] * 5 + [c_int_p, _vp]),
    "ani_featurize_f64": (_i, [_vp] * 6 + [_i] + [_vp] * 5 + [c_int_p, _vp]),
    "ani_featurize_grad_f32": (_i, [_vp] * 6 + [_i] + [_vp] * 8 + [c_int_p, _vp]),
    "ani_featurize_grad_f64": (_i, [_vp] * 6 + [_i] + [_vp] * 8 + [c_int_p, _vp]),
    "ani_featurize_grad_inverse_f32": (_i, [_vp] * 6 + [_i] + [_vp] * 8 + [c_int_p, _vp]),
    "ani_featurize_grad_inverse_f64": (_i, [_vp] * 6 + [_i] + [_vp] * 8 + [c_int_p, _vp]),
    "ani_mlp_packed_bytes": (ctypes.c_size_t, []),
    "ani_mlp_pack_weights_f32": (_i, [ctypes.POINTER(MlpPackArgs), _vp]),
    "ani_mlp_backward_f32": (_i, [ctypes.POINTER(MlpBackwardArgs), c_int_p, _i, _vp]),
    "ani_mlp_weight_grad_f32": (_i, [ctypes.POINTER(MlpWeightGradArgs), c_int_p, _i, _vp]),
    "ani_molecule_energy_f32": (_i, [_vp] * 4 + [_i, _i, _vp, ctypes.c_float, _vp, _vp, _vp, _vp]),
    "ani_nadam_step_f32": (_i, [_vp] * 5 + [ctypes.c_longlong, _vp, _vp, _vp]),
    "ani_clip_rows_f32": (_i, [_vp, _vp, _vp, _i, ctypes.c_float, _vp]),
    "ani_scale_by_loss_f32": (_i, [_vp, ctypes.c_longlong, _vp, _i, _i, _vp, _vp]),
    "ani_host_pack_batch": (_i, [_vp]),
    "ani_network_pass_f32": (_i, [ctypes.POINTER(PassArgs), _vp]),
    "ani_feeder_create": (_i, [_i, _vp, _i, ctypes.POINTER(_vp)]),
    "ani_feeder_begin": (_i, [_vp, _vp, ctypes.c_longlong, _i]),
    "ani_feeder_next": (_i, [_vp, ctypes.POINTER(FeederBatch)]),
    "ani_feeder_wait": (_i, [_vp, _i, _vp]),
    "ani_feeder_release": (_i, [_vp, _i, _vp]),
    "ani_feeder_end": (_i, [_vp]),
    "ani_feeder_destroy": (_i, [_vp]),
    "ani_peer_create": (_i, [_i, _i, ctypes.c_longlong, ctypes.POINTER(_vp)]),
    "ani_peer_handle": (_i, [_vp, _vp]),
    "ani_peer_connect": (_i, [_vp, _i, _vp]),
    "ani_peer_connect_raw": (_i, [_vp, _i, _vp]),
    "ani_peer_block": (_vp, [_vp]),
    "ani_peer_set_spin_limit": (_i, [_vp, ctypes.c_uint]),
    "ani_peer_set_two_halves": (_i, [_vp, _i]),
    "ani_peer_mean_f32": (_i, [_vp, _vp, ctypes.c_longlong, _vp]),
    "ani_peer_destroy": (_i, [_vp]),
    "ani_charge_f32": (_i, [_vp] * 6 + [_i, _i, _vp, _vp]),
    "ani_charge_f64": (_i, [_vp] * 6 + [_i, _i, _vp, _vp]),
    "ani_charge_grad_f32": (_i, [_vp] * 6 + [_i, _i, _vp, _vp, _vp]),
    "ani_charge_grad_f64": (_i, [_vp] * 6 + [_i, _i, _vp, _vp, _vp]),
    "ani_mlp_forward_f32": (_i, [ctypes.POINTER(MlpArgs), c_int_p, _i, _i, _vp]),
}


def nvcc_path() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: cannot build libani_b200.so")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.join(INCLUDE, "ani_b200.h")]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA sources for sm_100a into ``khan_b200/libani_b200.so``."""
    with _lock:
        if not force and not _stale():
            return LIB_PATH
        cmd = [nvcc_path()] + NVCC_FLAGS + ["-o", LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
        out = subprocess.run(cmd, capture_output=True, text=True, cwd=CSRC)
        if verbose or out.returncode != 0:
            print(" ".join(cmd))
            print(out.stdout, out.stderr)
        if out.returncode != 0:
            raise RuntimeError("nvcc failed building libani_b200.so:\n" + out.stderr)
        return LIB_PATH


def lib() -> ctypes.CDLL:
    """The loaded library with argument types declared.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; "
                "g.build()'` (needs nvcc).  khan_b200 has no CPU fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
        return _lib


def same_device(device, *tensors, where: str = "kernel launch") -> None:
    """Raises unless every given tensor (None entries are skipped) lives on ``device``.  Every pointer
    that goes into a launch must belong to the launching device: the kernels use plain loads and
    stores, peer access between devices is never enabled, and a pointer into another GPU's memory
    would fault on the device."""
    import torch
    dev = torch.device(device)
    want = (dev.type, dev.index if dev.index is not None else (torch.cuda.current_device() if dev.type == "cuda" else None))
    for t in tensors:
        if t is None:
            continue
        have = (t.device.type, t.device.index)
        if have != want:
            raise ValueError(f"{where}: a tensor on {t.device} was passed to a launch on {dev}; "
                             "all buffers and weights of a call must be on the launching GPU")


class AniError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().ani_status_string(status).decode()
        if status == -3:
            msg += ": " + lib().ani_last_cuda_error().decode()
        super().__init__(f"{where}: {msg} (status {status})")


def check(status: int, where: str) -> None:
    if status != 0:
        raise AniError(status, where)
