"""The C-ABI library loads without a GPU and exports every symbol include/ani_b200.h declares."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from khan_b200 import _lib


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ani_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ani_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def handle():
    _lib.build()
    return _lib.lib()


def test_header_and_signature_table_agree():
    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol(handle):
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(raw, name), name


def test_host_only_entry_points(handle):
    assert handle.ani_feature_size() == 384
    assert handle.ani_status_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -6, -7, -8, -9):
        assert handle.ani_status_string(code) != b"unknown status"


def test_argument_checks_need_no_gpu(handle):
    four = (ctypes.c_int * 4)(0, 0, 0, 0)
    # empty batch: valid, does nothing
    assert handle.ani_featurize_f32(None, None, None, None, None, None, 0, None, None, None, None,
                                    None, four, None) == 0
    assert handle.ani_featurize_grad_f64(None, None, None, None, None, None, 0, None, None, None,
                                         None, None, None, None, None, four, None) == 0
    # missing acs / negative sizes are rejected before anything is launched
    assert handle.ani_featurize_f32(None, None, None, None, None, None, 0, None, None, None, None,
                                    None, None, None) == -1
    bad = (ctypes.c_int * 4)(1, -1, 0, 0)
    assert handle.ani_featurize_f32(None, None, None, None, None, None, 1, None, None, None, None,
                                    None, bad, None) == -2
    assert handle.ani_sort(None, -1, None, None, None, None) == -2
    one = (ctypes.c_int * 4)(1, 0, 0, 0)
    assert handle.ani_featurize_f32(None, None, None, None, None, None, 1, None, None, None, None,
                                    None, one, None) == -1


def test_weight_grad_rejects_misaligned_matrices_before_launching(handle):
    """The tensor-core weight-gradient kernel uses 16-byte accesses: a matrix pointer that is
    only 4-byte aligned is refused on the host (nothing is dereferenced, no GPU needed)."""
    args = _lib.MlpWeightGradArgs()
    for name, _ in args._fields_:
        getattr(args, name)[0] = 0x10000
    one = (ctypes.c_int * 4)(5, 0, 0, 0)
    args.dw2[0] = 0x10004
    assert handle.ani_mlp_weight_grad_f32(ctypes.byref(args), one, 1, None) == -9
    args.dw2[0] = None
    assert handle.ani_mlp_weight_grad_f32(ctypes.byref(args), one, 1, None) == -1
    fwd = _lib.MlpArgs()
    for name, _ in fwd._fields_:
        getattr(fwd, name)[0] = 0x20000
    fwd.features[0] = 0x20008
    assert handle.ani_mlp_forward_f32(ctypes.byref(fwd), one, 0, 1, None) == -9
    bwd = _lib.MlpBackwardArgs()
    for name, _ in bwd._fields_:
        getattr(bwd, name)[0] = 0x30000
    bwd.dz2[0] = 0x30004
    assert handle.ani_mlp_backward_f32(ctypes.byref(bwd), one, 1, None) == -9
    assert handle.ani_nadam_step_f32(None, None, None, None, None, 10, None, None, None) == -1
    assert handle.ani_nadam_step_f32(None, None, None, None, None, 0, None, None, None) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.lib()
