"""Generate golden vectors by running the REFERENCE project's own kernels on a B200.

Needs ``oracle/_ref/libko_ref_kernels.so`` (``make -C oracle ref`` in a checkout that has the
reference sources; the reference kernels are compiled unmodified for sm_100a) and a GPU.  Inputs
come from the oracle's seeded generator, so the fixtures store only shapes, seeds and the
reference's outputs.  Usage (from the repo root, on a GPU machine):

    python tests/golden/make_reference_vectors.py [output.npz]

The committed ``tests/golden/reference_kernels_b200.npz`` was produced by this script; the CPU
tests compare the oracle's ``literal`` modes with it, the GPU tests compare the product with it.
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ko_oracle as oracle  # noqa: E402

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libko_ref_kernels.so")

# (name, rows, cols, seed, std, causal)
SOFTMAX_CASES = [("softmax_32x128", 32, 128, 0, 2.0, False), ("softmax_16x512_causal", 16, 512, 4, 2.0, True)]
# (name, rows, cols, seed, eps)
LAYERNORM_CASES = [("layernorm_8x768", 8, 768, 1, 1e-4)]
# (name, M, N, K, seed, with_c)
SGEMM_CASES = [("sgemm_64x64x64", 64, 64, 64, 2, False), ("sgemm_128x64x256_c", 128, 64, 256, 2, True)]


def softmax_input(rows, cols, seed, std, causal):
    x = oracle.fill_normal((rows, cols), seed, 0, 0.0, std)
    if causal:
        oracle.causal_mask_(x, 0, 512, -1e4)
    return x


def layernorm_inputs(rows, cols, seed):
    x = oracle.fill_normal((rows, cols), seed, 0, 0.0, 1.0)
    gamma = oracle.fill_uniform((cols,), seed, 1, 0.5, 1.5)
    beta = oracle.fill_normal((cols,), seed, 2, 0.0, 0.1)
    return x, gamma, beta


def sgemm_inputs(M, N, K, seed, with_c):
    a = oracle.fill_uniform((M, K), seed, 0, -1.0, 1.0)
    b = oracle.fill_uniform((K, N), seed, 1, -1.0, 1.0)
    c = oracle.fill_uniform((M, N), seed, 2, -1.0, 1.0) if with_c else None
    return a, b, c


def main(out_path: str) -> None:
    ref = C.CDLL(REF_LIB)
    vp, ll, ci, f32 = C.c_void_p, C.c_longlong, C.c_int, C.c_float
    ref.ko_ref_softmax_f32.argtypes = [vp, vp, ll, ci, vp]
    ref.ko_ref_layernorm_f32.argtypes = [vp, vp, ll, ci, f32, vp, vp, ci, vp]
    ref.ko_ref_sgemm_f32.argtypes = [ll, ll, ll, vp, ll, vp, ll, vp, vp, vp]
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    out = {}

    for name, rows, cols, seed, std, causal in SOFTMAX_CASES:
        x = torch.from_numpy(softmax_input(rows, cols, seed, std, causal)).to(dev)
        y = torch.empty_like(x)
        rc = ref.ko_ref_softmax_f32(x.data_ptr(), y.data_ptr(), rows, cols, stream)
        torch.cuda.synchronize()
        assert rc == 0, (name, rc)
        out[name] = y.cpu().numpy()

    for name, rows, cols, seed, eps in LAYERNORM_CASES:
        xh, gh, bh = layernorm_inputs(rows, cols, seed)
        x, g, b = (torch.from_numpy(t).to(dev) for t in (xh, gh, bh))
        for variant, tag in ((0, "warp"), (1, "warp_affine"), (2, "block64")):
            y = torch.empty_like(x)
            rc = ref.ko_ref_layernorm_f32(x.data_ptr(), y.data_ptr(), rows, cols, eps, g.data_ptr(), b.data_ptr(),
                                          variant, stream)
            torch.cuda.synchronize()
            assert rc == 0, (name, tag, rc)
            out[f"{name}_{tag}"] = y.cpu().numpy()

    for name, M, N, K, seed, with_c in SGEMM_CASES:
        ah, bh, ch = sgemm_inputs(M, N, K, seed, with_c)
        # slack behind A and B: the reference reads one K-tile past the end (simt_gemm.h:287-292)
        a = torch.zeros(M * K + 64, dtype=torch.float32, device=dev)
        b = torch.zeros(K * N + 8 * N + 64, dtype=torch.float32, device=dev)
        a[: M * K] = torch.from_numpy(ah).reshape(-1).to(dev)
        b[: K * N] = torch.from_numpy(bh).reshape(-1).to(dev)
        c = None if ch is None else torch.from_numpy(ch).to(dev)
        d = torch.empty((M, N), dtype=torch.float32, device=dev)
        rc = ref.ko_ref_sgemm_f32(M, N, K, a.data_ptr(), a.numel(), b.data_ptr(), b.numel(),
                                  None if c is None else c.data_ptr(), d.data_ptr(), stream)
        torch.cuda.synchronize()
        assert rc == 0, (name, rc)
        out[name] = d.cpu().numpy()

    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_kernels_b200.npz"))
