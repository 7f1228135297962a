"""ctypes binding of ``libko_b200.so`` -- one prototype per declaration in ``include/ko_b200.h``."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_PKG, "lib", "libko_b200.so")


class KoError(RuntimeError):
    """A C entry point returned a non-zero ko_status_t."""

    def __init__(self, status: int, name: str, message: str):
        super().__init__(f"{name} -> {status} ({message})")
        self.status = status


def library_path() -> str:
    return _LIB_PATH


_i64, _i32, _u32, _f32, _f64, _int = C.c_int64, C.c_int32, C.c_uint32, C.c_float, C.c_double, C.c_int
_vp, _sz = C.c_void_p, C.c_size_t
_f64p = C.POINTER(C.c_double)

# name -> (restype, argtypes); keep in step with include/ko_b200.h
PROTOTYPES = {
    "ko_status_string": (C.c_char_p, [_int]),
    "ko_last_error_string": (C.c_char_p, []),
    "ko_version": (_int, []),
    "ko_poll_device_status": (_int, []),
    "ko_selftest_bounded_wait": (_int, [C.c_uint, _vp]),
    "ko_tensor_create": (_int, [_sz, _int, C.POINTER(_vp)]),
    "ko_tensor_destroy": (_int, [_vp]),
    "ko_tensor_host_ptr": (_vp, [_vp]),
    "ko_tensor_device_ptr": (_vp, [_vp]),
    "ko_tensor_size_in_bytes": (_sz, [_vp]),
    "ko_tensor_device": (_int, [_vp]),
    "ko_tensor_host_to_device": (_int, [_vp]),
    "ko_tensor_host_to_device_async": (_int, [_vp, _vp]),
    "ko_tensor_device_to_host": (_int, [_vp]),
    "ko_tensor_device_to_host_async": (_int, [_vp, _vp]),
    "ko_fill_uniform": (_int, [_vp, _int, _i64, _u32, _u32, _i64, _f32, _f32]),
    "ko_fill_normal": (_int, [_vp, _int, _i64, _u32, _u32, _i64, _f32, _f32]),
    "ko_fill_causal_mask_f32": (_int, [_vp, _i64, _i32, _i64, _i32, _f32]),
    "ko_check_max_abs_f32": (_int, [_vp, _vp, _i64, _f64p]),
    "ko_check_max_rel_f32": (_int, [_vp, _vp, _i64, _f64, _f64p]),
    "ko_check_rel_frobenius_f32": (_int, [_vp, _vp, _i64, _f64p]),
    "ko_check_max_rowsum_err_f32": (_int, [_vp, _i64, _i32, _f64p]),
    "ko_softmax_f32": (_int, [_vp, _vp, _i64, _i32, _vp]),
    "ko_softmax_f16": (_int, [_vp, _vp, _i64, _i32, _vp]),
    "ko_softmax_bf16": (_int, [_vp, _vp, _i64, _i32, _vp]),
    "ko_layernorm_f32": (_int, [_vp, _vp, _i64, _i32, _f32, _vp, _vp, _int, _vp]),
    "ko_layernorm_bf16": (_int, [_vp, _vp, _i64, _i32, _f32, _vp, _vp, _int, _vp]),
    "ko_layernorm_f16": (_int, [_vp, _vp, _i64, _i32, _f32, _vp, _vp, _int, _vp]),
    "ko_softmax_f32_host": (_int, [_vp, _vp, _i64, _i32, _int, _vp]),
    "ko_layernorm_f32_host": (_int, [_vp, _vp, _i64, _i32, _f32, _vp, _vp, _int, _int, _vp]),
    "ko_sgemm_f32": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ko_sgemm_f32_no_alloc": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _int, _vp]),
    "ko_gemm_f16_f32": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ko_gemm_bf16_f32": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ko_gemm_f16_f16": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ko_gemm_bf16_bf16": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ko_gemm_tc": (_int, [_int, _int, _int, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ko_context_create": (_int, [_int, C.POINTER(_vp)]),
    "ko_context_destroy": (_int, [_vp]),
    "ko_context_stats": (_int, [_vp, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz)]),
    "ko_sgemm_f32_ctx": (_int, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ko_gemm_tc_ctx": (_int, [_vp, _int, _int, _int, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ko_probe_functor": (_int, [_int, _int, _int, _vp, _vp, _vp, _vp, _i64, _vp]),
    "ko_probe_reduce": (_int, [_int, _int, _vp, _vp, _i64, _int, _vp]),
    "ko_probe_limits": (_int, [_vp, _vp, _vp, _vp, _vp]),
    "ko_probe_welford": (_int, [_int, _vp, _i64, _i32, _vp, _int, _vp]),
    "ko_probe_gemm_tensor_core_template": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ko_probe_mma_ldmatrix": (_int, [_vp, _vp, _vp, _vp, _i32, _vp]),
    "ko_probe_composed_rowop": (_int, [_int, _vp, _vp, _i64, _i32, _f32, _vp, _vp, _int, _vp]),
}

class RowKnobs(C.Structure):
    """ko_row_knobs_t of include/ko_b200_tuning.h: launch-geometry overrides of the row operators (0 = default)."""

    _fields_ = [("tier", _int), ("rows_per_warp", _int), ("block", _int), ("grid_cap", _i64), ("stage_rows", _int),
                ("stages", _int), ("ctas_per_sm", _int), ("cluster", _int)]


_knobs_p = C.POINTER(RowKnobs)

# launch-geometry overrides (include/ko_b200_tuning.h)
TUNING_PROTOTYPES = {
    "ko_softmax_f32_tuned": (_int, [_vp, _vp, _i64, _i32, _knobs_p, _vp]),
    "ko_layernorm_f32_tuned": (_int, [_vp, _vp, _i64, _i32, _f32, _vp, _vp, _int, _knobs_p, _vp]),
    "ko_layernorm_bf16_tuned": (_int, [_vp, _vp, _i64, _i32, _f32, _vp, _vp, _int, _knobs_p, _vp]),
    "ko_layernorm_f16_tuned": (_int, [_vp, _vp, _i64, _i32, _f32, _vp, _vp, _int, _knobs_p, _vp]),
    "ko_sgemm_f32_tuned": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _int, _int, _vp]),
    "ko_gemm_tc_tuned": (_int, [_int, _int, _int, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _int, _int, _vp]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the native library (once).  Fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "or `cmake -S . -B build -G Ninja && cmake --build build`; there is no fallback path"
            )
        handle = C.CDLL(_LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError here means the header and the library disagree
            fn.restype, fn.argtypes = res, args
        for name, (res, args) in TUNING_PROTOTYPES.items():
            fn = getattr(handle, name, None)
            if fn is not None:
                fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int, name: str) -> None:
    if status != 0:
        msg = lib().ko_last_error_string().decode(errors="replace")
        code = lib().ko_status_string(status).decode()
        raise KoError(status, name, f"{code}: {msg}")
