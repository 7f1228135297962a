"""CPU: the C-ABI library loads, exports every symbol the header declares, and its host-only entry
points (status strings, fills, comparisons, argument validation) behave.  No kernel is launched."""
import ctypes as C
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "ko_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ko_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(ko, lib):
    names = _declared_symbols()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/ko_b200.h but not exported"
    assert set(names) == set(ko.native.PROTOTYPES), "native.PROTOTYPES and the header disagree"


def test_status_strings_and_version(lib):
    assert lib.ko_status_string(0) == b"KO_OK"
    assert lib.ko_status_string(3) == b"KO_ERR_SHAPE"
    assert lib.ko_status_string(99) == b"KO_ERR_UNKNOWN"
    assert lib.ko_version() >= 100


def test_argument_validation_needs_no_gpu(lib):
    # rejected before any CUDA call is made
    assert lib.ko_softmax_f32(None, None, -1, 4, None) == 1
    assert b"negative" in lib.ko_last_error_string()
    assert lib.ko_softmax_f32(None, None, 4, 4, None) == 1
    assert lib.ko_layernorm_f32(None, None, 4, 4, 1e-5, None, None, 2, None) == 1
    assert b"ddof" in lib.ko_last_error_string()
    assert lib.ko_sgemm_f32(-1, 1, 1, None, None, None, None, None) == 1
    assert lib.ko_sgemm_f32(4, 4, 4, None, None, None, None, None) == 1
    # empty problems are legal no-ops
    assert lib.ko_softmax_f32(None, None, 0, 128, None) == 0
    assert lib.ko_layernorm_bf16(None, None, 0, 128, 1e-5, None, None, 0, None) == 0
    assert lib.ko_sgemm_f32(0, 8, 8, None, None, None, None, None) == 0
    assert lib.ko_fill_uniform(None, 7, 4, 0, 0, 0, 0.0, 1.0) == 1
    assert lib.ko_tensor_create(16, 0, None) == 1


def test_check_functions(lib):
    want = np.array([1.0, -2.0, 0.0, 4.0], dtype=np.float32)
    got = np.array([1.0, -2.5, 0.5, 4.0], dtype=np.float32)
    out = C.c_double()
    assert lib.ko_check_max_abs_f32(got.ctypes.data, want.ctypes.data, 4, C.byref(out)) == 0 and out.value == 0.5
    assert lib.ko_check_max_rel_f32(got.ctypes.data, want.ctypes.data, 4, 1.0, C.byref(out)) == 0 and out.value == 0.5
    assert lib.ko_check_rel_frobenius_f32(got.ctypes.data, want.ctypes.data, 4, C.byref(out)) == 0
    assert abs(out.value - np.sqrt(0.5 / 21.0)) < 1e-12
    rows = np.array([[0.25, 0.75], [0.5, 0.25]], dtype=np.float32)
    assert lib.ko_check_max_rowsum_err_f32(rows.ctypes.data, 2, 2, C.byref(out)) == 0 and abs(out.value - 0.25) < 1e-7
    bad = np.array([np.nan], dtype=np.float32)
    assert lib.ko_check_max_abs_f32(bad.ctypes.data, want.ctypes.data, 1, C.byref(out)) == 0 and out.value == np.inf
    assert lib.ko_check_max_abs_f32(None, None, 4, C.byref(out)) == 1


def test_product_does_not_reach_into_the_oracle():
    """No source of the product package or the header mentions the oracle directory."""
    pkg = os.path.join(ROOT, "kernel_optimization_b200")
    for base, _dirs, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".h", ".cu", ".cc", ".cuh")):
                text = open(os.path.join(base, f), errors="replace").read()
                assert "oracle" not in text.lower(), f"{os.path.join(base, f)} refers to the oracle"


def test_every_tuning_symbol_is_exported_and_bound(ko, lib):
    """include/ko_b200_tuning.h: the launch-geometry overrides are part of the library and of the ctypes binding."""
    text = open(os.path.join(ROOT, "include", "ko_b200_tuning.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = sorted(set(re.findall(r"\b(ko_[a-z0-9_]+)\s*\(", text)))
    assert len(names) >= 6
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/ko_b200_tuning.h but not exported"
    assert set(names) == set(ko.native.TUNING_PROTOTYPES)
