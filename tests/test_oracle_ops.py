"""CPU: the oracle's operators -- FP32 ports against the float64 versions, the `literal` modes
against what the reference's own kernels produced on a B200 (tests/golden), and the documented
defects of the reference (Subtract adds, WelfordMerge divides at every level)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))


def _softmax_input(oracle, rows, cols, seed, std, causal):
    x = oracle.fill_normal((rows, cols), seed, 0, 0.0, std)
    if causal:
        oracle.causal_mask_(x, 0, 512, -1e4)
    return x


def test_softmax_port_and_literal_against_reference_kernel(oracle, golden):
    for name, rows, cols, seed, causal in (("softmax_32x128", 32, 128, 0, False), ("softmax_16x512_causal", 16, 512, 4, True)):
        x = _softmax_input(oracle, rows, cols, seed, 2.0, causal)
        ref = golden[name]
        # the reference is built with -use_fast_math: agreement to a few 1e-7, not bit for bit
        assert np.abs(oracle.softmax_f32(x, literal=True) - ref).max() <= 5e-7
        assert np.abs(oracle.softmax_f32(x) - ref).max() <= 5e-7
        assert oracle.max_abs_err(ref, oracle.softmax_f64(x)) <= 1e-6      # the benchmark's tolerance
        assert oracle.max_abs_err(oracle.softmax_f32(x), oracle.softmax_f64(x)) <= 1e-6
        assert oracle.max_rowsum_err(oracle.softmax_f32(x)) <= 1e-5


def test_softmax_literal_overflows_where_fixed_does_not(oracle):
    x = np.full((2, 128), 50.0, dtype=np.float32)  # 2*rowmax = 100 > 88.7
    with np.errstate(all="ignore"):
        assert not np.isfinite(oracle.softmax_f32(x, literal=True)).all()
    assert np.allclose(oracle.softmax_f32(x), 1.0 / 128)


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 5), (7, 100), (64, 128), (5, 131), (2, 4096), (3, 40000)])
def test_softmax_port_vs_float64(oracle, rows, cols):
    x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
    assert oracle.max_abs_err(oracle.softmax_f32(x), oracle.softmax_f64(x)) <= 1e-6
    assert oracle.max_rowsum_err(oracle.softmax_f32(x)) <= 1e-5
    assert np.array_equal(oracle.softmax_f32(x, threads=1), oracle.softmax_f32(x, threads=4))


def _ln_inputs(oracle, rows, cols, seed=1):
    return (oracle.fill_normal((rows, cols), seed, 0, 0.0, 1.0), oracle.fill_uniform((cols,), seed, 1, 0.5, 1.5),
            oracle.fill_normal((cols,), seed, 2, 0.0, 0.1))


def test_layernorm_literal_reproduces_reference_kernel(oracle, golden):
    x, g, b = _ln_inputs(oracle, 8, 768)
    for name, lit in (("layernorm_8x768_warp", oracle.layernorm_f32(x, 1e-4, literal=True)),
                      ("layernorm_8x768_warp_affine", oracle.layernorm_f32(x, 1e-4, g, b, literal=True))):
        ref = golden[name]
        assert np.abs(lit - ref).max() <= 2e-6 * np.abs(ref).max()
    # ... and what the reference computes is not LayerNorm: the per-level divide shrinks the variance
    # by orders of magnitude and the mean is added instead of subtracted
    ref = golden["layernorm_8x768_warp"]
    assert ref.std() > 10.0
    assert np.abs(ref - oracle.layernorm_f64(x, 1e-4)).max() > 10.0
    # the block variant launched with 64 threads additionally folds stale lanes (common.h:59-63)
    assert np.abs(golden["layernorm_8x768_block64"] - oracle.layernorm_f64(x, 1e-4)).max() > 10.0


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 5), (7, 100), (64, 768), (5, 131), (2, 4096), (3, 40000)])
@pytest.mark.parametrize("ddof", [0, 1])
def test_layernorm_port_vs_float64(oracle, rows, cols, ddof):
    x, g, b = _ln_inputs(oracle, rows, cols)
    want = oracle.layernorm_f64(x, 1e-12, g, b, ddof)
    if cols == 1 and ddof == 0:
        assert np.allclose(want, b)  # zero variance: output is beta
    assert oracle.max_rel_err(oracle.layernorm_f32(x, 1e-12, g, b, ddof), want) <= 1e-5
    np_mean = x.astype(np.float64).mean(1, keepdims=True)
    np_var = x.astype(np.float64).var(1, ddof=ddof if cols > ddof else 0, keepdims=True)
    if cols > ddof:
        np_ln = (x - np_mean) / np.sqrt(np_var + 1e-12) * g + b
        assert np.abs(np_ln - want).max() <= 1e-9 * max(1.0, np.abs(want).max())


def test_layernorm_constant_rows(oracle):
    x = np.full((4, 768), 3.25, dtype=np.float32)
    assert np.array_equal(oracle.layernorm_f32(x, 1e-12), np.zeros_like(x))
    assert np.array_equal(oracle.layernorm_f64(x, 1e-12), np.zeros_like(x, dtype=np.float64))


@pytest.mark.parametrize("rows,cols", [(3, 4), (17, 128), (9, 768), (5, 1000), (2, 4099)])
def test_welford_statistics_port_vs_float64(oracle, rows, cols):
    """(count, mean, M2) of the reference-order FP32 restatement (update per vector slot, slot fold, shuffle tree,
    merge without the per-level division) against the two-pass float64 statistics and numpy."""
    x = oracle.fill_normal((rows, cols), 1, 5, 0.75, 2.0)
    want = oracle.welford_stats_f64(x)
    x64 = x.astype(np.float64)
    assert np.array_equal(want[:, 0], np.full(rows, float(cols)))
    assert np.allclose(want[:, 1], x64.mean(axis=1), rtol=0, atol=1e-13)
    assert np.allclose(want[:, 2], ((x64 - x64.mean(axis=1, keepdims=True)) ** 2).sum(axis=1), rtol=1e-12)
    port = oracle.welford_stats_f32(x)
    assert np.array_equal(port[:, 0], want[:, 0].astype(np.float32))
    assert np.abs(port[:, 1] - want[:, 1]).max() <= 1e-6
    assert (np.abs(port[:, 2] - want[:, 2]) / want[:, 2]).max() <= 1e-5
    # the same triple is what the port's LayerNorm divides once: var = M2 / cols
    y = oracle.layernorm_f32(x, 0.0)
    rstd = 1.0 / np.sqrt(port[:, 2].astype(np.float64) / cols)
    assert np.abs(y - (x64 - port[:, 1:2]) * rstd[:, None]).max() <= 2e-6


def test_sgemm_port_is_bit_identical_to_reference_kernel(oracle, golden):
    a, b = oracle.fill_uniform((64, 64), 2, 0), oracle.fill_uniform((64, 64), 2, 1)
    assert np.array_equal(oracle.sgemm_f32(a, b), golden["sgemm_64x64x64"])
    a, b, c = oracle.fill_uniform((128, 256), 2, 0), oracle.fill_uniform((256, 64), 2, 1), oracle.fill_uniform((128, 64), 2, 2)
    assert np.array_equal(oracle.sgemm_f32(a, b, c), golden["sgemm_128x64x256_c"])
    # the reference's own acceptance test: |D - cuBLAS| <= 1e-3 (gemm/main.cu:157-174); float64 stands in for cuBLAS
    assert np.abs(golden["sgemm_128x64x256_c"] - oracle.sgemm_f64(a, b, c)).max() <= 1e-3


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 7, 3), (64, 64, 8), (100, 36, 52), (129, 65, 17), (256, 256, 256)])
def test_gemm_oracles_against_numpy(oracle, M, N, K):
    a, b, c = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1), oracle.fill_uniform((M, N), 2, 2)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(oracle.sgemm_f64(a, b) - want).max() <= 1e-12 * K
    assert np.abs(oracle.sgemm_f64(a, b, c) - (want + c)).max() <= 1e-12 * K
    assert oracle.rel_frobenius(oracle.sgemm_f32(a, b), want) <= 1e-6
    assert np.array_equal(oracle.sgemm_f32(a, b, threads=1), oracle.sgemm_f32(a, b, threads=3))
    bt = np.ascontiguousarray(b.T)
    assert np.abs(oracle.gemm_tn_f64(a, bt) - want).max() <= 1e-12 * K
    assert oracle.rel_frobenius(oracle.gemm_tn_f32(a, bt, c), want + c) <= 1e-6


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_mixed_precision_gemm_oracle(oracle, kind):
    M, N, K = 96, 80, 200
    a, b = oracle.fill_uniform((M, K), 3, 0), oracle.fill_uniform((N, K), 3, 1)
    to_bits, from_bits = (oracle.to_f16_bits, oracle.from_f16_bits) if kind == "f16" else (oracle.to_bf16_bits, oracle.from_bf16_bits)
    ar, br = from_bits(to_bits(a)), from_bits(to_bits(b))
    want = oracle.gemm_tn_f64(ar, br)
    assert np.abs(want - ar.astype(np.float64) @ br.astype(np.float64).T).max() <= 1e-12 * K
    assert oracle.rel_frobenius(oracle.gemm_tn_f32(ar, br), want) <= 1e-6
    # rounding the inputs is what costs accuracy, not the accumulation
    assert oracle.rel_frobenius((a.astype(np.float64) @ b.astype(np.float64).T).astype(np.float32), want) > 1e-4


def test_metrics(oracle):
    want = np.array([[1.0, -2.0], [0.0, 4.0]])
    got = np.array([[1.0, -2.5], [0.5, 4.0]], dtype=np.float32)
    assert oracle.max_abs_err(got, want) == 0.5
    assert oracle.max_rel_err(got, want, floor=1.0) == 0.5       # |0.5-0|/max(0,1)
    assert abs(oracle.rel_frobenius(got, want) - np.sqrt(0.5 / 21.0)) < 1e-12
    assert abs(oracle.max_rowsum_err(np.array([[0.25, 0.75], [0.5, 0.25]], dtype=np.float32)) - 0.25) < 1e-7
    assert oracle.max_abs_err(np.array([np.nan], dtype=np.float32), np.array([0.0])) == np.inf
