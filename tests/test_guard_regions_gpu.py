"""GPU: guard regions around every device operand.  Each operand sits in the middle of a larger allocation whose
4 KB before and after it are filled with 0xFF bytes (a NaN in every element type used here):

  * a store that lands outside an output leaves non-0xFF bytes in a guard, which is asserted untouched afterwards
    (an overrun of the kind the reference's SGEMM has on the read side, nn_operators/gemm/simt_gemm.h:287-292, would
    show here if it were on the write side);
  * a load that strays outside an input brings a NaN in, which would surface in the output, and outputs are
    pre-filled with NaN so that an element the kernel never wrote stays visible -- both are covered by comparing the
    whole output with the oracle.

Nothing here faults: the guards belong to the same allocation.  Operand sizes are deliberately not multiples of 16
bytes where the entry point allows it, so that the trailing guard starts right behind the last element.  The shapes
are the tail shapes of the per-operator parity tests; every tier and epilogue is forced through the tuning calls."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GUARD = 4096


class Guarded:
    """nbytes of device memory (256-byte aligned start) with GUARD bytes of 0xFF on both sides."""

    def __init__(self, cuda, nbytes):
        self.cuda, self.nbytes = cuda, nbytes
        self.buf = cuda.full((GUARD + nbytes + GUARD,), 0xFF, dtype=cuda.uint8, device="cuda")
        self.bytes = self.buf[GUARD:GUARD + nbytes]

    @classmethod
    def of(cls, cuda, array):
        """an input operand holding `array` (numpy, any dtype)"""
        g = cls(cuda, array.nbytes)
        if array.nbytes:
            g.bytes.copy_(cuda.from_numpy(np.ascontiguousarray(array).view(np.uint8).reshape(-1)))
        return g

    def ptr(self):
        return self.buf.data_ptr() + GUARD

    def numpy(self, dtype, shape):
        return self.bytes.cpu().numpy().view(dtype).reshape(shape)

    def intact(self):
        head, tail = self.buf[:GUARD], self.buf[GUARD + self.nbytes:]
        return bool((head == 0xFF).all()) and bool((tail == 0xFF).all())


def _stream(cuda):
    return cuda.cuda.current_stream().cuda_stream


def _finish(cuda, lib, rc, *operands):
    assert rc == 0, lib.ko_last_error_string()
    cuda.cuda.synchronize()
    assert lib.ko_poll_device_status() == 0, lib.ko_last_error_string()
    for i, g in enumerate(operands):
        assert g.intact(), f"operand {i}: bytes outside the buffer were overwritten"


# ------------------------------------------------------------------------------------------------
# row operators
# ------------------------------------------------------------------------------------------------
ROW_SHAPES_F32 = [(1, 1), (3, 1), (5, 4), (7, 100), (5, 131), (1000, 128), (33, 640), (37, 1024), (9, 2052), (11, 4096),
                  (3, 20000), (2, 32768), (3, 40000), (2, 131072)]
F32_TIERS = {  # tier -> (rows, cols) it accepts among the shapes above
    0: lambda r, c: True,
    1: lambda r, c: c % 4 == 0 and c <= 2048,
    2: lambda r, c: c % 4 == 0 and c <= 32768,
    3: lambda r, c: True,
    4: lambda r, c: c % 4 == 0 and c <= 2048 and c >= 64,
    6: lambda r, c: c % 4 == 0 and c >= 4096,
    7: lambda r, c: c % 4 == 0 and c <= 32768,
    8: lambda r, c: c % 4 == 0,
}


@pytest.mark.parametrize("tier", sorted(F32_TIERS))
@pytest.mark.parametrize("rows,cols", ROW_SHAPES_F32)
def test_softmax_f32_stays_inside_its_buffers(cuda, lib, oracle, rows, cols, tier):
    from kernel_optimization_b200.native import RowKnobs

    if not F32_TIERS[tier](rows, cols):
        pytest.skip("shape outside this tier")
    x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
    gin, gout = Guarded.of(cuda, x), Guarded(cuda, x.nbytes)
    rc = lib.ko_softmax_f32_tuned(gin.ptr(), gout.ptr(), rows, cols, RowKnobs(tier=tier) if tier else None, _stream(cuda))
    _finish(cuda, lib, rc, gin, gout)
    y = gout.numpy(np.float32, (rows, cols))
    assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= 1e-6


@pytest.mark.parametrize("tier", [0, 1, 2, 3, 4, 5, 6, 8, 82, 9])
@pytest.mark.parametrize("rows,cols", ROW_SHAPES_F32)
def test_layernorm_f32_stays_inside_its_buffers(cuda, lib, oracle, rows, cols, tier):
    from kernel_optimization_b200.native import RowKnobs

    ok = {0: True, 1: cols % 4 == 0 and cols <= 2048, 2: cols % 4 == 0 and cols <= 32768, 3: True,
          4: cols % 4 == 0 and 64 <= cols <= 2048, 5: cols % 4 == 0 and cols <= 16384, 6: cols % 4 == 0 and cols >= 4096,
          8: cols % 4 == 0, 82: cols % 4 == 0, 9: cols % 4 == 0 and cols <= 512}[tier]
    if not ok:
        pytest.skip("shape outside this tier")
    x = oracle.fill_normal((rows, cols), 1, 0, 0.0, 1.0)
    g, b = oracle.fill_uniform((cols,), 1, 1, 0.5, 1.5), oracle.fill_normal((cols,), 1, 2, 0.0, 0.1)
    gin, gout, gg, gb = Guarded.of(cuda, x), Guarded(cuda, x.nbytes), Guarded.of(cuda, g), Guarded.of(cuda, b)
    knobs = RowKnobs(tier=8, rows_per_warp=2) if tier == 82 else (RowKnobs(tier=tier) if tier else None)  # 82: rows in pairs
    rc = lib.ko_layernorm_f32_tuned(gin.ptr(), gout.ptr(), rows, cols, 1e-5, gg.ptr(), gb.ptr(), 0, knobs, _stream(cuda))
    _finish(cuda, lib, rc, gin, gout, gg, gb)
    y = gout.numpy(np.float32, (rows, cols))
    assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-5, g, b)) <= 1e-5


ROW_SHAPES_16 = [(1, 8), (7, 100), (9, 136), (33, 256), (100, 768), (17, 2048), (9, 2056), (5, 4096), (3, 20000), (2, 40008), (150, 65544)]


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("op", ["softmax", "layernorm"])
@pytest.mark.parametrize("rows,cols", ROW_SHAPES_16)
def test_16bit_row_operators_stay_inside_their_buffers(cuda, lib, oracle, rows, cols, op, kind):
    to_bits, from_bits = (oracle.to_f16_bits, oracle.from_f16_bits) if kind == "f16" else (oracle.to_bf16_bits, oracle.from_bf16_bits)
    ulp = 2.0 ** -10 if kind == "f16" else 2.0 ** -7
    xb = to_bits(oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0))
    gin, gout = Guarded.of(cuda, xb), Guarded(cuda, xb.nbytes)
    if op == "softmax":
        fn = lib.ko_softmax_f16 if kind == "f16" else lib.ko_softmax_bf16
        rc = fn(gin.ptr(), gout.ptr(), rows, cols, _stream(cuda))
        _finish(cuda, lib, rc, gin, gout)
        want = oracle.softmax_f64(from_bits(xb))
        got = from_bits(gout.numpy(np.uint16, (rows, cols))).astype(np.float64)
        assert np.abs(got - want).max() <= ulp * 0.51 + 1e-6
    else:
        gbits, bbits = to_bits(oracle.fill_uniform((cols,), 1, 1, 0.5, 1.5)), to_bits(oracle.fill_normal((cols,), 1, 2, 0.0, 0.1))
        gg, gb = Guarded.of(cuda, gbits), Guarded.of(cuda, bbits)
        fn = lib.ko_layernorm_f16 if kind == "f16" else lib.ko_layernorm_bf16
        rc = fn(gin.ptr(), gout.ptr(), rows, cols, 1e-5, gg.ptr(), gb.ptr(), 0, _stream(cuda))
        _finish(cuda, lib, rc, gin, gout, gg, gb)
        want = oracle.layernorm_f64(from_bits(xb), 1e-5, from_bits(gbits), from_bits(bbits))
        got = from_bits(gout.numpy(np.uint16, (rows, cols)))
        assert oracle.max_rel_err(got, want) <= ulp * 0.51 + 1e-5


# ------------------------------------------------------------------------------------------------
# SGEMM: every kernel variant, unit ranges and whole tiles, with and without C
# ------------------------------------------------------------------------------------------------
SGEMM_SHAPES = [(1, 1, 1), (64, 64, 8), (100, 36, 52), (129, 65, 17), (256, 256, 256), (300, 200, 1000), (17, 513, 33),
                (1024, 1024, 64), (65, 4000, 129), (2304, 2432, 130)]


@pytest.mark.parametrize("variant,split_k", [(0, 0), (1, 1), (2, 1), (3, 1), (4, 1), (4, 3), (6, 0), (7, 0), (8, 0), (8, 2)])
@pytest.mark.parametrize("M,N,K", SGEMM_SHAPES)
def test_sgemm_stays_inside_its_buffers(cuda, lib, oracle, M, N, K, variant, split_k):
    a, b = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1)
    c = oracle.fill_uniform((M, N), 2, 2) if (M + N + K) % 2 else None
    ga, gb, gd = Guarded.of(cuda, a), Guarded.of(cuda, b), Guarded(cuda, M * N * 4)
    gc = Guarded.of(cuda, c) if c is not None else None
    rc = lib.ko_sgemm_f32_tuned(M, N, K, ga.ptr(), gb.ptr(), gc.ptr() if gc else None, gd.ptr(), variant, split_k, _stream(cuda))
    _finish(cuda, lib, rc, ga, gb, gd, *([gc] if gc else []))
    assert oracle.rel_frobenius(gd.numpy(np.float32, (M, N)), oracle.sgemm_f64(a, b, c)) <= 1e-6


def test_sgemm_no_alloc_stays_inside_its_buffers(cuda, lib, oracle):
    for (M, N, K), split_k in (((300, 200, 1000), 2), ((129, 65, 170), 4), ((512, 384, 1024), 0)):
        a, b = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1)
        ga, gb, gd = Guarded.of(cuda, a), Guarded.of(cuda, b), Guarded(cuda, M * N * 4)
        rc = lib.ko_sgemm_f32_no_alloc(M, N, K, ga.ptr(), gb.ptr(), None, gd.ptr(), split_k, _stream(cuda))
        _finish(cuda, lib, rc, ga, gb, gd)
        assert oracle.rel_frobenius(gd.numpy(np.float32, (M, N)), oracle.sgemm_f64(a, b)) <= 1e-6


# ------------------------------------------------------------------------------------------------
# tcgen05 GEMM: every tile width, the two-SM kernel (bn = 2048) and K slices, both epilogues (TMA store / direct), both
# B layouts, FP32 and 16-bit D
# ------------------------------------------------------------------------------------------------
TC_SHAPES = [(1, 4, 8), (100, 36, 56), (129, 260, 136), (128, 64, 64), (256, 512, 256), (1000, 520, 200), (300, 8, 64), (200, 37, 64)]


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("bn", [0, 64, 128, 256, 512, 2048, 256 | (3 << 16)])   # the last: three K slices per tile
@pytest.mark.parametrize("mode", ["tma_store", "direct", "plus_c", "out16", "row_major_b"])
@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_tensor_core_gemm_stays_inside_its_buffers(cuda, lib, oracle, M, N, K, mode, bn, kind):
    to_bits, from_bits = (oracle.to_f16_bits, oracle.from_f16_bits) if kind == "f16" else (oracle.to_bf16_bits, oracle.from_bf16_bits)
    fmt = 0 if kind == "f16" else 1
    out16 = mode == "out16"
    row_b = mode == "row_major_b"
    if mode == "tma_store" and N % 4:
        pytest.skip("a TMA store needs a 16-byte row pitch")
    if out16 and N % 8 and bn:  # keep the matrix of cases small: odd pitches of 16-bit D only with the default tile
        pytest.skip("covered with bn = 0")
    if row_b and N % 8:
        pytest.skip("row-major B needs a 16-byte row pitch")
    ab = to_bits(oracle.fill_uniform((M, K), 3, 0))
    bt = to_bits(oracle.fill_uniform((N, K), 3, 1))               # [N, K]: column-major B
    b_dev = np.ascontiguousarray(bt.T) if row_b else bt            # [K, N] when row-major
    c = oracle.fill_uniform((M, N), 3, 2) if mode == "plus_c" else None
    out_fmt = 0 if not out16 else (1 if kind == "f16" else 2)
    ga, gb = Guarded.of(cuda, ab), Guarded.of(cuda, b_dev)
    gd = Guarded(cuda, M * N * (2 if out16 else 4))
    gc = Guarded.of(cuda, c) if c is not None else None
    store_mode = {"tma_store": 1, "direct": 2}.get(mode, 0)
    rc = lib.ko_gemm_tc_tuned(fmt, out_fmt, 1 if row_b else 0, M, N, K, ga.ptr(), gb.ptr(), gc.ptr() if gc else None, gd.ptr(), bn,
                              store_mode, _stream(cuda))
    _finish(cuda, lib, rc, ga, gb, gd, *([gc] if gc else []))
    want = oracle.gemm_tn_f64(from_bits(ab), from_bits(bt), c)
    if out16:
        got = from_bits(gd.numpy(np.uint16, (M, N)))
        assert oracle.rel_frobenius(got, want) <= (2.0 ** -10 if kind == "f16" else 2.0 ** -7)
    else:
        assert oracle.rel_frobenius(gd.numpy(np.float32, (M, N)), want) <= 1e-5
