"""ctypes/numpy front end of the CPU oracle (``libko_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by the tests, by the smoke check and by the benchmark's
CPU-baseline leg.  Nothing in the product package imports this module; the CUDA library has
no CPU fallback.

Each function wraps the C routine of the same name (``ko_oracle.c``), which restates
arithmetic of the reference project donglinz/kernel_optimization (file:line citations are in
the C source and header).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libko_oracle.so")


def build(force: bool = False) -> str:
    """Compile ``libko_oracle.so`` with the Makefile beside this file (no-op when up to date)."""
    if force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_LIB_PATH)
        for f in ("ko_oracle.c", "ko_oracle.h")
    ):
        subprocess.run(["make", "-C", _HERE, "libko_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def _load() -> C.CDLL:
    build()
    lib = C.CDLL(_LIB_PATH)
    f32p, f64p, u16p, u32p = (C.POINTER(t) for t in (C.c_float, C.c_double, C.c_uint16, C.c_uint32))
    i64, i32, u32, f32, f64, ci = C.c_int64, C.c_int32, C.c_uint32, C.c_float, C.c_double, C.c_int
    sig = {
        "ko_oracle_philox4x32_10": (None, [u32p, u32p, u32p]),
        "ko_oracle_fill_uniform_f32": (None, [f32p, i64, u32, u32, i64, f32, f32]),
        "ko_oracle_fill_normal_f32": (None, [f32p, i64, u32, u32, i64, f32, f32]),
        "ko_oracle_causal_mask_f32": (None, [f32p, i64, i32, i64, i32, f32]),
        "ko_oracle_round_f32_to_bf16": (None, [f32p, u16p, i64]),
        "ko_oracle_round_f32_to_f16": (None, [f32p, u16p, i64]),
        "ko_oracle_widen_bf16": (None, [u16p, f32p, i64]),
        "ko_oracle_widen_f16": (None, [u16p, f32p, i64]),
        "ko_oracle_softmax_f64": (None, [f32p, f64p, i64, i32]),
        "ko_oracle_softmax_f32": (None, [f32p, f32p, i64, i32, ci, ci]),
        "ko_oracle_layernorm_f64": (None, [f32p, f64p, i64, i32, f64, f32p, f32p, ci]),
        "ko_oracle_layernorm_f32": (None, [f32p, f32p, i64, i32, f32, f32p, f32p, ci, ci, ci]),
        "ko_oracle_welford_stats_f32": (None, [f32p, f32p, i64, i32]),
        "ko_oracle_welford_stats_f64": (None, [f32p, f64p, i64, i32]),
        "ko_oracle_sgemm_f32": (None, [i64, i64, i64, f32p, f32p, f32p, f32p, ci]),
        "ko_oracle_sgemm_f64": (None, [i64, i64, i64, f32p, f32p, f32p, f64p, ci]),
        "ko_oracle_gemm_tn_f32": (None, [i64, i64, i64, f32p, f32p, f32p, f32p, ci]),
        "ko_oracle_gemm_tn_f64": (None, [i64, i64, i64, f32p, f32p, f32p, f64p, ci]),
        "ko_oracle_max_abs_err": (f64, [f32p, f64p, i64]),
        "ko_oracle_max_rel_err": (f64, [f32p, f64p, i64, f64]),
        "ko_oracle_rel_frobenius": (f64, [f32p, f64p, i64]),
        "ko_oracle_max_rowsum_err": (f64, [f32p, i64, i32]),
        "ko_oracle_max_threads": (ci, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


_lib = _load()


def _p(a: np.ndarray | None, ctype):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(C.POINTER(ctype))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    return int(_lib.ko_oracle_max_threads())


# ---------------------------------------------------------------- generator
def philox4x32_10(ctr, key) -> np.ndarray:
    c = np.asarray(ctr, dtype=np.uint32).copy()
    k = np.asarray(key, dtype=np.uint32).copy()
    out = np.empty(4, dtype=np.uint32)
    _lib.ko_oracle_philox4x32_10(_p(c, C.c_uint32), _p(k, C.c_uint32), _p(out, C.c_uint32))
    return out


def fill_uniform(shape, seed: int, tensor_id: int, lo=-1.0, hi=1.0, elem_offset: int = 0) -> np.ndarray:
    out = np.empty(shape, dtype=np.float32)
    _lib.ko_oracle_fill_uniform_f32(_p(out, C.c_float), out.size, seed, tensor_id, elem_offset, lo, hi)
    return out


def fill_normal(shape, seed: int, tensor_id: int, mean=0.0, std=1.0, elem_offset: int = 0) -> np.ndarray:
    out = np.empty(shape, dtype=np.float32)
    _lib.ko_oracle_fill_normal_f32(_p(out, C.c_float), out.size, seed, tensor_id, elem_offset, mean, std)
    return out


def causal_mask_(x: np.ndarray, row_offset: int = 0, block: int = 512, value: float = -1e4) -> np.ndarray:
    rows, cols = x.shape
    _lib.ko_oracle_causal_mask_f32(_p(x, C.c_float), rows, cols, row_offset, block, value)
    return x


# ---------------------------------------------------------------- 16-bit floats (raw uint16 storage)
def to_bf16_bits(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    _lib.ko_oracle_round_f32_to_bf16(_p(x, C.c_float), _p(out, C.c_uint16), x.size)
    return out


def to_f16_bits(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    _lib.ko_oracle_round_f32_to_f16(_p(x, C.c_float), _p(out, C.c_uint16), x.size)
    return out


def from_bf16_bits(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    _lib.ko_oracle_widen_bf16(_p(h, C.c_uint16), _p(out, C.c_float), h.size)
    return out


def from_f16_bits(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    _lib.ko_oracle_widen_f16(_p(h, C.c_uint16), _p(out, C.c_float), h.size)
    return out


# ---------------------------------------------------------------- operators
def softmax_f64(x) -> np.ndarray:
    x = _f32(x)
    rows, cols = x.shape
    out = np.empty(x.shape, dtype=np.float64)
    _lib.ko_oracle_softmax_f64(_p(x, C.c_float), _p(out, C.c_double), rows, cols)
    return out


def softmax_f32(x, literal: bool = False, threads: int = 0) -> np.ndarray:
    x = _f32(x)
    rows, cols = x.shape
    out = np.empty(x.shape, dtype=np.float32)
    _lib.ko_oracle_softmax_f32(_p(x, C.c_float), _p(out, C.c_float), rows, cols, int(literal), threads)
    return out


def layernorm_f64(x, eps: float, gamma=None, beta=None, ddof: int = 0) -> np.ndarray:
    x = _f32(x)
    rows, cols = x.shape
    g = None if gamma is None else _f32(gamma)
    b = None if beta is None else _f32(beta)
    out = np.empty(x.shape, dtype=np.float64)
    _lib.ko_oracle_layernorm_f64(_p(x, C.c_float), _p(out, C.c_double), rows, cols, eps,
                                 _p(g, C.c_float), _p(b, C.c_float), ddof)
    return out


def layernorm_f32(x, eps: float, gamma=None, beta=None, ddof: int = 0, literal: bool = False,
                  threads: int = 0) -> np.ndarray:
    x = _f32(x)
    rows, cols = x.shape
    g = None if gamma is None else _f32(gamma)
    b = None if beta is None else _f32(beta)
    out = np.empty(x.shape, dtype=np.float32)
    _lib.ko_oracle_layernorm_f32(_p(x, C.c_float), _p(out, C.c_float), rows, cols, eps,
                                 _p(g, C.c_float), _p(b, C.c_float), ddof, int(literal), threads)
    return out


def welford_stats_f32(x) -> np.ndarray:
    """[rows, 3] = (count, mean, M2) in FP32, the reference warp kernel's update/merge order."""
    x = _f32(x)
    out = np.empty((x.shape[0], 3), dtype=np.float32)
    _lib.ko_oracle_welford_stats_f32(_p(x, C.c_float), _p(out, C.c_float), x.shape[0], x.shape[1])
    return out


def welford_stats_f64(x) -> np.ndarray:
    """[rows, 3] = (count, mean, M2) in float64, two passes."""
    x = _f32(x)
    out = np.empty((x.shape[0], 3), dtype=np.float64)
    _lib.ko_oracle_welford_stats_f64(_p(x, C.c_float), _p(out, C.c_double), x.shape[0], x.shape[1])
    return out


def _gemm(fn, out_dtype, out_ctype, M, N, K, a, b, c, threads):
    out = np.empty((M, N), dtype=out_dtype)
    fn(M, N, K, _p(a, C.c_float), _p(b, C.c_float), _p(c, C.c_float), _p(out, out_ctype), threads)
    return out


def sgemm_f32(a, b, c=None, threads: int = 0) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    c = None if c is None else _f32(c)
    (M, K), (K2, N) = a.shape, b.shape
    assert K == K2
    return _gemm(_lib.ko_oracle_sgemm_f32, np.float32, C.c_float, M, N, K, a, b, c, threads)


def sgemm_f64(a, b, c=None, threads: int = 0) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    c = None if c is None else _f32(c)
    (M, K), (K2, N) = a.shape, b.shape
    assert K == K2
    return _gemm(_lib.ko_oracle_sgemm_f64, np.float64, C.c_double, M, N, K, a, b, c, threads)


def gemm_tn_f32(a, bt, c=None, threads: int = 0) -> np.ndarray:
    """a: [M,K] row-major; bt: [N,K] (the column-major [K,N] operand as stored), both FP32 values."""
    a, bt = _f32(a), _f32(bt)
    c = None if c is None else _f32(c)
    (M, K), (N, K2) = a.shape, bt.shape
    assert K == K2
    return _gemm(_lib.ko_oracle_gemm_tn_f32, np.float32, C.c_float, M, N, K, a, bt, c, threads)


def gemm_tn_f64(a, bt, c=None, threads: int = 0) -> np.ndarray:
    a, bt = _f32(a), _f32(bt)
    c = None if c is None else _f32(c)
    (M, K), (N, K2) = a.shape, bt.shape
    assert K == K2
    return _gemm(_lib.ko_oracle_gemm_tn_f64, np.float64, C.c_double, M, N, K, a, bt, c, threads)


# ---------------------------------------------------------------- metrics
def _pair(got, want):
    got = _f32(got)
    want = np.ascontiguousarray(want, dtype=np.float64)
    assert got.shape == want.shape
    return got, want


def max_abs_err(got, want) -> float:
    got, want = _pair(got, want)
    return float(_lib.ko_oracle_max_abs_err(_p(got, C.c_float), _p(want, C.c_double), got.size))


def max_rel_err(got, want, floor: float = 1.0) -> float:
    got, want = _pair(got, want)
    return float(_lib.ko_oracle_max_rel_err(_p(got, C.c_float), _p(want, C.c_double), got.size, floor))


def rel_frobenius(got, want) -> float:
    got, want = _pair(got, want)
    return float(_lib.ko_oracle_rel_frobenius(_p(got, C.c_float), _p(want, C.c_double), got.size))


def max_rowsum_err(got) -> float:
    got = _f32(got)
    rows, cols = got.shape
    return float(_lib.ko_oracle_max_rowsum_err(_p(got, C.c_float), rows, cols))
