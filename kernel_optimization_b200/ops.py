"""Python-side mirror of the operator interface: torch (or raw pointers) in, C ABI underneath.

torch is used only for device memory and the current CUDA stream; every operator call goes to
``libko_b200.so``.  ``Tensor`` mirrors the reference's ``class Tensor`` (common/tensor.h:11-40):
a page-locked host buffer plus a device buffer with copies in both directions.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import native

DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
_NP_OF = {DTYPE_F32: np.float32, DTYPE_F16: np.uint16, DTYPE_BF16: np.uint16}
_SIZE_OF = {DTYPE_F32: 4, DTYPE_F16: 2, DTYPE_BF16: 2}


def _current_stream_ptr() -> int:
    import torch

    return int(torch.cuda.current_stream().cuda_stream)


def _ptr(t) -> int | None:
    """Device address of a torch tensor (must be contiguous), an int address, or None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if not t.is_cuda:
        raise ValueError("operator inputs must live on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError("operator inputs must be contiguous")
    return int(t.data_ptr())


class Tensor:
    """Host (pinned) + device buffer of ``size_in_bytes`` bytes owned by the native library."""

    def __init__(self, size_in_bytes: int, device: int = -1):
        self._h = C.c_void_p()
        native.check(native.lib().ko_tensor_create(size_in_bytes, device, C.byref(self._h)), "ko_tensor_create")

    @classmethod
    def from_shape(cls, shape, byte_per_element: int, device: int = -1) -> "Tensor":
        return cls(int(np.prod(shape, dtype=np.int64)) * byte_per_element, device)

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown: the module globals are already gone, the process frees the buffers
            pass

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            native.lib().ko_tensor_destroy(self._h)
            self._h = C.c_void_p()

    @property
    def size_in_bytes(self) -> int:
        return int(native.lib().ko_tensor_size_in_bytes(self._h))

    @property
    def device(self) -> int:
        return int(native.lib().ko_tensor_device(self._h))

    @property
    def device_ptr(self) -> int:
        return int(native.lib().ko_tensor_device_ptr(self._h) or 0)

    def host_ref(self, dtype=np.float32) -> np.ndarray:
        """numpy view of the host buffer (no copy)."""
        n = self.size_in_bytes // np.dtype(dtype).itemsize
        addr = native.lib().ko_tensor_host_ptr(self._h)
        buf = (C.c_char * self.size_in_bytes).from_address(addr)
        return np.frombuffer(buf, dtype=dtype, count=n)

    def host_to_device(self) -> None:
        native.check(native.lib().ko_tensor_host_to_device(self._h), "ko_tensor_host_to_device")

    def host_to_device_async(self, stream: int | None = None) -> None:
        s = _current_stream_ptr() if stream is None else stream
        native.check(native.lib().ko_tensor_host_to_device_async(self._h, s), "ko_tensor_host_to_device_async")

    def device_to_host(self) -> None:
        native.check(native.lib().ko_tensor_device_to_host(self._h), "ko_tensor_device_to_host")

    def device_to_host_async(self, stream: int | None = None) -> None:
        s = _current_stream_ptr() if stream is None else stream
        native.check(native.lib().ko_tensor_device_to_host_async(self._h, s), "ko_tensor_device_to_host_async")


# ------------------------------------------------------------------ seeded host fills
def fill_uniform(shape, seed: int, tensor_id: int, lo=-1.0, hi=1.0, dtype: int = DTYPE_F32, elem_offset: int = 0,
                 out: np.ndarray | None = None) -> np.ndarray:
    a = np.empty(shape, dtype=_NP_OF[dtype]) if out is None else out
    native.check(native.lib().ko_fill_uniform(a.ctypes.data, dtype, a.size, seed, tensor_id, elem_offset, lo, hi),
                 "ko_fill_uniform")
    return a


def fill_normal(shape, seed: int, tensor_id: int, mean=0.0, std=1.0, dtype: int = DTYPE_F32, elem_offset: int = 0,
                out: np.ndarray | None = None) -> np.ndarray:
    a = np.empty(shape, dtype=_NP_OF[dtype]) if out is None else out
    native.check(native.lib().ko_fill_normal(a.ctypes.data, dtype, a.size, seed, tensor_id, elem_offset, mean, std),
                 "ko_fill_normal")
    return a


def fill_causal_mask_(a: np.ndarray, row_offset: int = 0, block: int = 512, value: float = -1e4) -> np.ndarray:
    rows, cols = a.shape
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    native.check(native.lib().ko_fill_causal_mask_f32(a.ctypes.data, rows, cols, row_offset, block, value),
                 "ko_fill_causal_mask_f32")
    return a


# ------------------------------------------------------------------ operators (torch tensors on the GPU)
def softmax(x, out=None, stream: int | None = None):
    """Row softmax over the last dimension of a 2-D FP32, FP16 or BF16 CUDA tensor (FP32 arithmetic)."""
    import torch

    assert x.dim() == 2 and x.dtype in (torch.float32, torch.float16, torch.bfloat16)
    out = torch.empty_like(x) if out is None else out
    assert out.dtype == x.dtype
    s = _current_stream_ptr() if stream is None else stream
    rows, cols = x.shape
    lib = native.lib()
    fn = {torch.float32: lib.ko_softmax_f32, torch.float16: lib.ko_softmax_f16, torch.bfloat16: lib.ko_softmax_bf16}[x.dtype]
    native.check(fn(_ptr(x), _ptr(out), rows, cols, s), "ko_softmax")
    return out


def layernorm(x, eps: float, gamma=None, beta=None, ddof: int = 0, out=None, stream: int | None = None):
    """LayerNorm forward over the last dimension of a 2-D FP32, FP16 or BF16 CUDA tensor (FP32 statistics)."""
    import torch

    assert x.dim() == 2 and x.dtype in (torch.float32, torch.float16, torch.bfloat16)
    for p in (gamma, beta):
        assert p is None or (p.dtype == x.dtype and p.numel() == x.shape[1])
    out = torch.empty_like(x) if out is None else out
    s = _current_stream_ptr() if stream is None else stream
    rows, cols = x.shape
    lib = native.lib()
    fn = {torch.float32: lib.ko_layernorm_f32, torch.float16: lib.ko_layernorm_f16, torch.bfloat16: lib.ko_layernorm_bf16}[x.dtype]
    native.check(fn(_ptr(x), _ptr(out), rows, cols, eps, _ptr(gamma), _ptr(beta), ddof, s), "ko_layernorm")
    return out


def softmax_host(t_in: Tensor, t_out: Tensor, rows: int, cols: int, chunks: int = 0, stream: int | None = None) -> None:
    """FP32 row softmax of the HOST contents of ``t_in`` into the host buffer of ``t_out``: copy in, kernel and
    copy out are pipelined over ``chunks`` row ranges (0 = 8).  Stream-ordered like a kernel launch."""
    s = _current_stream_ptr() if stream is None else stream
    native.check(native.lib().ko_softmax_f32_host(t_in._h, t_out._h, rows, cols, chunks, s), "ko_softmax_f32_host")


def layernorm_host(t_in: Tensor, t_out: Tensor, rows: int, cols: int, eps: float, gamma=None, beta=None, ddof: int = 0,
                   chunks: int = 0, stream: int | None = None) -> None:
    """FP32 LayerNorm of the HOST contents of ``t_in`` into the host buffer of ``t_out`` (gamma / beta: CUDA tensors)."""
    s = _current_stream_ptr() if stream is None else stream
    native.check(native.lib().ko_layernorm_f32_host(t_in._h, t_out._h, rows, cols, eps, _ptr(gamma), _ptr(beta), ddof, chunks, s),
                 "ko_layernorm_f32_host")


def sgemm(a, b, c=None, out=None, stream: int | None = None):
    """D = A @ B (+ C); row-major FP32 CUDA tensors."""
    import torch

    assert a.dtype == b.dtype == torch.float32 and a.dim() == b.dim() == 2 and a.shape[1] == b.shape[0]
    M, K = a.shape
    N = b.shape[1]
    out = torch.empty((M, N), dtype=torch.float32, device=a.device) if out is None else out
    s = _current_stream_ptr() if stream is None else stream
    native.check(native.lib().ko_sgemm_f32(M, N, K, _ptr(a), _ptr(b), _ptr(c), _ptr(out), s), "ko_sgemm_f32")
    return out


def gemm_tc(a, b, c=None, out=None, stream: int | None = None, out_dtype=None, b_row_major: bool = False):
    """D[M,N] = A[M,K] @ B[K,N] (+ C) with FP16/BF16 inputs and FP32 accumulation.

    ``b`` is the column-major [K,N] operand as stored, i.e. a contiguous [N,K] tensor, or with
    ``b_row_major`` a contiguous [K,N] tensor.  ``out_dtype`` is float32 (default) or the input dtype;
    ``c`` has the output dtype.
    """
    import torch

    assert a.dtype == b.dtype and a.dtype in (torch.float16, torch.bfloat16)
    M, K = a.shape
    if b_row_major:
        K2, N = b.shape
    else:
        N, K2 = b.shape
    assert K == K2
    out_dtype = (out.dtype if out is not None else torch.float32) if out_dtype is None else out_dtype
    assert out_dtype in (torch.float32, a.dtype), "D is FP32 or the input type"
    assert c is None or c.dtype == out_dtype
    out = torch.empty((M, N), dtype=out_dtype, device=a.device) if out is None else out
    assert out.dtype == out_dtype
    s = _current_stream_ptr() if stream is None else stream
    in_fmt = 0 if a.dtype == torch.float16 else 1
    out_fmt = 0 if out_dtype == torch.float32 else (1 if out_dtype == torch.float16 else 2)
    native.check(native.lib().ko_gemm_tc(in_fmt, out_fmt, 1 if b_row_major else 0, M, N, K, _ptr(a), _ptr(b), _ptr(c), _ptr(out), s),
                 "ko_gemm_tc")
    return out
