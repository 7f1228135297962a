"""B200 (sm_100a) row softmax / Welford LayerNorm / SGEMM / tcgen05 GEMM operator set.

The product is the native library ``lib/libko_b200.so`` (hand-written CUDA behind the C ABI of
``include/ko_b200.h``).  This package is the thin Python plumbing around it: a ctypes loader, a
``Tensor`` mirror of the reference's host/device buffer class and wrappers that pass torch device
pointers and the current CUDA stream to the C entry points.  There is no CPU or PyTorch fallback:
if the library is missing, importing :mod:`kernel_optimization_b200.native` raises.
"""
from .native import KoError, lib, library_path  # noqa: F401
from .ops import (  # noqa: F401
    Tensor,
    fill_causal_mask_,
    fill_normal,
    fill_uniform,
    gemm_tc,
    layernorm,
    layernorm_host,
    sgemm,
    softmax,
    softmax_host,
)

__version__ = "0.1.0"
