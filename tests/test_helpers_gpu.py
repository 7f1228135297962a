"""GPU: the source-level helper templates (functors, AlignedArray forms, to_scalar, limits, WarpReduce,
BlockReduce, the Welford update / merge / warp / block combiners) run in device code through the
``ko_probe_*`` entry points and are compared with host arithmetic and the oracle's Welford statistics.

Tolerances: IEEE add / subtract / multiply / divide / max / fused multiply-add are correctly rounded on both
sides, so those compare bit for bit; ``expf`` / ``rsqrtf`` are within 2 ulp of the float64 value; reductions
of N values in another order within N * 2^-24 of the float64 sum; Welford statistics against the float64
two-pass value: count exact, mean within 1e-6 absolute (rows are O(1)), M2 within 1e-5 relative (the LayerNorm
tolerance).  16-bit functors: one rounding of the exact result (two for divide, four half-ulps for exp / rsqrt)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

F32, F16, BF16 = 0, 1, 2
REDUCE_MAX, REDUCE_SUM, EXP, RSQRT, ADD, SUBTRACT, MULTIPLY, DIVIDE, MULTIPLY_ADD = range(9)
SCALAR, VEC_VEC, VEC_SCALAR = 0, 1, 2


def _stream(cuda):
    return cuda.cuda.current_stream().cuda_stream


def _ok(lib, rc):
    assert rc == 0, lib.ko_last_error_string()


def _ulps(got, want64):
    """distance in units of the FP32 spacing at |want|"""
    want32 = want64.astype(np.float32)
    spacing = np.spacing(np.abs(want32)).astype(np.float64)
    return np.abs(got.astype(np.float64) - want64) / spacing


def _fma_f32(a, b, c):
    """a * b + c rounded once to FP32: the product of two FP32 values is exact in float64; the float64 sum is then
    rounded twice (to float64, to FP32), which can differ from the single rounding in the last bit only."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64))


HOST_F32 = {
    REDUCE_MAX: lambda a, b, c: np.maximum(a, b),
    REDUCE_SUM: lambda a, b, c: a + b,
    ADD: lambda a, b, c: a + b,
    SUBTRACT: lambda a, b, c: a - b,
    MULTIPLY: lambda a, b, c: a * b,
    DIVIDE: lambda a, b, c: a / b,
}


@pytest.mark.parametrize("functor", [REDUCE_MAX, REDUCE_SUM, ADD, SUBTRACT, MULTIPLY, DIVIDE])
@pytest.mark.parametrize("form", [SCALAR, VEC_VEC, VEC_SCALAR])
def test_binary_functors_f32_bit_exact(cuda, lib, oracle, functor, form):
    n = 4 * 1000
    a = oracle.fill_normal((n,), 11, 0, 0.0, 3.0)
    b = oracle.fill_uniform((n,), 11, 1, 0.5, 2.5) * np.where(np.arange(n) % 3 == 0, -1, 1).astype(np.float32)
    ad, bd = cuda.from_numpy(a).cuda(), cuda.from_numpy(b).cuda()
    out = cuda.full((n,), float("nan"), device="cuda")
    _ok(lib, lib.ko_probe_functor(functor, form, F32, ad.data_ptr(), bd.data_ptr(), None, out.data_ptr(), n, _stream(cuda)))
    cuda.cuda.synchronize()
    rhs = np.repeat(b[: n // 4], 4) if form == VEC_SCALAR else b  # vector i is paired with the scalar b[i]
    want = HOST_F32[functor](a, rhs, None)
    assert np.array_equal(out.cpu().numpy(), want)


def test_subtract_subtracts_and_multiply_add_rounds_to_nearest(cuda, lib):
    """The two deliberate corrections: the reference's Subtract returns a + b and its MultiplyAdd<float> rounds
    toward minus infinity."""
    a = np.array([5.0, 1.0, 1.0, -7.5], dtype=np.float32)
    b = np.array([3.0, 2.0**-24, 1.0, 2.5], dtype=np.float32)
    c = np.array([0.0, 1.0, 2.0**-30, 0.0], dtype=np.float32)
    ad, bd, cd = (cuda.from_numpy(v).cuda() for v in (a, b, c))
    out = cuda.empty(4, device="cuda")
    _ok(lib, lib.ko_probe_functor(SUBTRACT, SCALAR, F32, ad.data_ptr(), bd.data_ptr(), None, out.data_ptr(), 4, _stream(cuda)))
    assert out.cpu().numpy().tolist() == [2.0, 1.0 - 2.0**-24, 0.0, -10.0]  # (the reference's a + b would give 8, 1 + 2^-24 -> 1, 2, -5)
    _ok(lib, lib.ko_probe_functor(MULTIPLY_ADD, VEC_VEC, F32, ad.data_ptr(), bd.data_ptr(), cd.data_ptr(), out.data_ptr(), 4,
                                  _stream(cuda)))
    got = out.cpu().numpy()
    # 1 * 2^-24 + 1 = 1 + half an ulp: to nearest-even gives 1 (toward -inf would too); 1*1 + 2^-30 -> 1;
    # the discriminating case is a negative tiny addend
    assert got.tolist() == [15.0, 1.0, 1.0, -18.75]
    a2 = np.array([1.0, 1.0, 1.0, 1.0], dtype=np.float32)
    c2 = np.array([-(2.0**-30)] * 4, dtype=np.float32)
    a2d, c2d = cuda.from_numpy(a2).cuda(), cuda.from_numpy(c2).cuda()
    _ok(lib, lib.ko_probe_functor(MULTIPLY_ADD, SCALAR, F32, a2d.data_ptr(), a2d.data_ptr(), c2d.data_ptr(), out.data_ptr(), 4,
                                  _stream(cuda)))
    assert out.cpu().numpy().tolist() == [1.0] * 4  # round-toward-minus-infinity would give 1 - 2^-24


@pytest.mark.parametrize("form", [SCALAR, VEC_VEC])
def test_unary_and_ternary_functors_f32(cuda, lib, oracle, form):
    n = 4 * 1000
    x = oracle.fill_normal((n,), 12, 0, 0.0, 4.0)
    pos = oracle.fill_uniform((n,), 12, 1, 1e-6, 50.0)
    c = oracle.fill_normal((n,), 12, 2, 0.0, 1.0)
    xd, pd, cd = (cuda.from_numpy(v).cuda() for v in (x, pos, c))
    out = cuda.full((n,), float("nan"), device="cuda")
    _ok(lib, lib.ko_probe_functor(EXP, form, F32, xd.data_ptr(), None, None, out.data_ptr(), n, _stream(cuda)))
    assert _ulps(out.cpu().numpy(), np.exp(x.astype(np.float64))).max() <= 2.0
    _ok(lib, lib.ko_probe_functor(RSQRT, form, F32, pd.data_ptr(), None, None, out.data_ptr(), n, _stream(cuda)))
    assert _ulps(out.cpu().numpy(), 1.0 / np.sqrt(pos.astype(np.float64))).max() <= 2.0
    _ok(lib, lib.ko_probe_functor(MULTIPLY_ADD, form, F32, xd.data_ptr(), pd.data_ptr(), cd.data_ptr(), out.data_ptr(), n,
                                  _stream(cuda)))
    assert _ulps(out.cpu().numpy(), _fma_f32(x, pos, c)).max() <= 0.5 + 1e-6


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("form", [SCALAR, VEC_VEC, VEC_SCALAR])
def test_functors_16bit(cuda, lib, oracle, dtype, form):
    """AlignedArray<half, 8> / <__nv_bfloat16, 8>: arithmetic in the 16-bit type, one rounding per operation."""
    tdt = cuda.float16 if dtype == F16 else cuda.bfloat16
    eps16 = 2.0**-11 if dtype == F16 else 2.0**-8
    n = 8 * 500
    a = cuda.from_numpy(oracle.fill_normal((n,), 13, 0, 0.0, 2.0)).cuda().to(tdt)
    b = cuda.from_numpy(oracle.fill_uniform((n,), 13, 1, 0.5, 2.0)).cuda().to(tdt)
    c = cuda.from_numpy(oracle.fill_normal((n,), 13, 2, 0.0, 1.0)).cuda().to(tdt)
    out = cuda.empty(n, device="cuda", dtype=tdt)
    a64, b64, c64 = (v.double().cpu().numpy() for v in (a, b, c))
    rhs = np.repeat(b64[: n // 8], 8) if form == VEC_SCALAR else b64

    def run(functor):
        _ok(lib, lib.ko_probe_functor(functor, form, dtype, a.data_ptr(), b.data_ptr(), c.data_ptr(), out.data_ptr(), n,
                                      _stream(cuda)))
        return out.double().cpu().numpy()

    def close(got, want, ulps):
        assert np.all(np.abs(got - want) <= ulps * eps16 * np.maximum(np.abs(want), 2.0**-14))

    close(run(ADD), a64 + rhs, 1.0)
    close(run(SUBTRACT), a64 - rhs, 1.0)
    close(run(MULTIPLY), a64 * rhs, 1.0)
    close(run(DIVIDE), a64 / rhs, 2.0)
    assert np.array_equal(run(REDUCE_MAX), np.maximum(a64, rhs))
    close(run(REDUCE_SUM), a64 + rhs, 1.0)
    if form != VEC_SCALAR:
        close(run(EXP), np.exp(a64), 4.0)
        # Rsqrt reads its first operand: pass the positive tensor there
        _ok(lib, lib.ko_probe_functor(RSQRT, form, dtype, b.data_ptr(), None, None, out.data_ptr(), n, _stream(cuda)))
        close(out.double().cpu().numpy(), 1.0 / np.sqrt(b64), 4.0)
        close(run(MULTIPLY_ADD), a64 * b64 + c64, 1.0)  # fused: one rounding of the exact a * b + c


def test_probe_rejects_bad_requests(cuda, lib):
    buf = cuda.zeros(64, device="cuda")
    s = _stream(cuda)
    assert lib.ko_probe_functor(99, 0, F32, buf.data_ptr(), buf.data_ptr(), None, buf.data_ptr(), 4, s) == 1
    assert lib.ko_probe_functor(EXP, VEC_SCALAR, F32, buf.data_ptr(), buf.data_ptr(), None, buf.data_ptr(), 4, s) == 1
    assert lib.ko_probe_functor(ADD, VEC_VEC, F32, buf.data_ptr(), buf.data_ptr(), None, buf.data_ptr(), 6, s) == 3
    assert lib.ko_probe_functor(ADD, VEC_VEC, F32, buf.data_ptr() + 4, buf.data_ptr(), None, buf.data_ptr(), 4, s) == 2
    assert lib.ko_probe_reduce(1, 1, buf.data_ptr(), buf.data_ptr(), 1, 48, s) == 3
    assert lib.ko_probe_welford(2, buf.data_ptr(), 1, 6, buf.data_ptr(), 32, s) == 3
    assert lib.ko_probe_composed_rowop(0, buf.data_ptr(), buf.data_ptr(), 1, 8, 0.0, buf.data_ptr(), None, 32, s) == 1


def test_limits_on_device(cuda, lib):
    f = cuda.zeros(1, device="cuda")
    i = cuda.zeros(1, device="cuda", dtype=cuda.int32)
    h = cuda.zeros(2, device="cuda", dtype=cuda.int16)
    _ok(lib, lib.ko_probe_limits(f.data_ptr(), i.data_ptr(), h.data_ptr(), h.data_ptr() + 2, _stream(cuda)))
    assert f.item() == float(np.finfo(np.float32).max)
    assert i.item() == 2**31 - 1
    bits = h.cpu().numpy().view(np.uint16)
    assert np.array([bits[0]], dtype=np.uint16).view(np.float16)[0] == 65504.0
    assert bits[1] == 0x7F7F  # largest finite bfloat16


# ------------------------------------------------------------------------------------------------
# reductions
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("op", [0, 1])
def test_warp_reduce_and_to_scalar(cuda, lib, oracle, op):
    groups = 257
    x = oracle.fill_normal((groups, 32), 14, 0, 0.0, 5.0)
    xd = cuda.from_numpy(x).cuda()
    out = cuda.full((groups,), float("nan"), device="cuda")
    _ok(lib, lib.ko_probe_reduce(0, op, xd.data_ptr(), out.data_ptr(), groups, 32, _stream(cuda)))
    got = out.cpu().numpy()
    if op == 0:
        assert np.array_equal(got, x.max(axis=1))
    else:
        assert np.abs(got - x.astype(np.float64).sum(axis=1)).max() <= 32 * 2.0**-24 * np.abs(x).sum(axis=1).max()
    # to_scalar over AlignedArray<float, 4>: left-to-right fold
    out4 = cuda.full((groups * 8,), float("nan"), device="cuda")
    _ok(lib, lib.ko_probe_reduce(2, op, xd.data_ptr(), out4.data_ptr(), groups * 8, 4, _stream(cuda)))
    v = x.reshape(-1, 4)
    want = v.max(axis=1) if op == 0 else ((v[:, 0] + v[:, 1]) + v[:, 2]) + v[:, 3]
    assert np.array_equal(out4.cpu().numpy(), want)


def test_warp_reduce_int32_from_the_limits_identity(cuda, lib, oracle):
    groups = 64
    x = np.rint(oracle.fill_normal((groups, 32), 15, 0, 0.0, 1000.0)).astype(np.float32)
    x[3, :] = -2.0e9  # below every other key, above -INT32_MAX
    out = cuda.zeros(groups, device="cuda")
    _ok(lib, lib.ko_probe_reduce(3, 0, cuda.from_numpy(x).cuda().data_ptr(), out.data_ptr(), groups, 32, _stream(cuda)))
    assert np.array_equal(out.cpu().numpy(), x.max(axis=1))


@pytest.mark.parametrize("width", [32, 64, 128, 480, 992, 1024])
def test_block_reduce_any_block_size(cuda, lib, oracle, width):
    """64 ones reduced by a 64-thread block must give 64: the reference's BlockReduce folds the stale lanes of
    warp 0 in unless the block has 1024 threads."""
    groups = 19
    ones = cuda.ones(groups * width, device="cuda")
    out = cuda.full((2 * groups,), float("nan"), device="cuda")
    _ok(lib, lib.ko_probe_reduce(1, 1, ones.data_ptr(), out.data_ptr(), groups, width, _stream(cuda)))
    assert np.array_equal(out.cpu().numpy(), np.full(2 * groups, float(width), dtype=np.float32))
    x = oracle.fill_normal((groups, width), 16, width, 0.0, 3.0)
    xd = cuda.from_numpy(x).cuda()
    _ok(lib, lib.ko_probe_reduce(1, 0, xd.data_ptr(), out.data_ptr(), groups, width, _stream(cuda)))
    got = out.cpu().numpy()
    assert np.array_equal(got[:groups], x.max(axis=1)) and np.array_equal(got[groups:], x.max(axis=1))
    _ok(lib, lib.ko_probe_reduce(1, 1, xd.data_ptr(), out.data_ptr(), groups, width, _stream(cuda)))
    got = out.cpu().numpy()
    want = x.astype(np.float64).sum(axis=1)
    assert np.array_equal(got[:groups], got[groups:])  # back-to-back calls on one cache agree
    assert np.abs(got[:groups] - want).max() <= width * 2.0**-24 * np.abs(x).sum(axis=1).max()


# ------------------------------------------------------------------------------------------------
# Welford
# ------------------------------------------------------------------------------------------------
def _check_triples(got, x, oracle):
    want = oracle.welford_stats_f64(x)
    assert np.array_equal(got[:, 0], want[:, 0].astype(np.float32)), "count"
    assert np.abs(got[:, 1] - want[:, 1]).max() <= 1e-6, "mean"
    assert (np.abs(got[:, 2] - want[:, 2]) / np.maximum(want[:, 2], 1e-30)).max() <= 1e-5, "M2"


WELFORD_KINDS = [0, 1, 2, 3, 4]


@pytest.mark.parametrize("kind", WELFORD_KINDS)
@pytest.mark.parametrize("cols", [4, 128, 768, 1000])
def test_welford_thread_and_warp_forms(cuda, lib, oracle, kind, cols):
    rows = 37
    x = oracle.fill_normal((rows, cols), 1, 0, 0.5, 1.0)
    out = cuda.full((rows, 3), float("nan"), device="cuda")
    _ok(lib, lib.ko_probe_welford(kind, cuda.from_numpy(x).cuda().data_ptr(), rows, cols, out.data_ptr(), 32, _stream(cuda)))
    _check_triples(out.cpu().numpy(), x, oracle)


@pytest.mark.parametrize("kind", [5, 6])
@pytest.mark.parametrize("block", [32, 64, 192, 992, 1024])
def test_welford_block_forms_any_block_size(cuda, lib, oracle, kind, block):
    rows, cols = 11, 768
    x = oracle.fill_normal((rows, cols), 1, 3, -2.0, 3.0)
    out = cuda.full((rows, 3), float("nan"), device="cuda")
    _ok(lib, lib.ko_probe_welford(kind, cuda.from_numpy(x).cuda().data_ptr(), rows, cols, out.data_ptr(), block, _stream(cuda)))
    _check_triples(out.cpu().numpy(), x, oracle)


def test_welford_constant_rows_and_short_rows(cuda, lib, oracle):
    """var = 0 rows, and rows shorter than the number of lanes (most lanes hold empty triples)."""
    x = np.full((5, 8), 3.25, dtype=np.float32)
    for kind, block in [(0, 32), (1, 32), (2, 32), (3, 32), (4, 32), (5, 256), (6, 1024)]:
        out = cuda.full((5, 3), float("nan"), device="cuda")
        _ok(lib, lib.ko_probe_welford(kind, cuda.from_numpy(x).cuda().data_ptr(), 5, 8, out.data_ptr(), block, _stream(cuda)))
        got = out.cpu().numpy()
        assert np.array_equal(got, np.tile(np.array([8.0, 3.25, 0.0], dtype=np.float32), (5, 1))), (kind, got)


# ------------------------------------------------------------------------------------------------
# whole operators composed of the helpers
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("block", [32, 64, 96, 256, 1024])
@pytest.mark.parametrize("cols", [4, 128, 1000, 4096])
def test_composed_softmax_matches_the_oracle(cuda, lib, oracle, block, cols):
    rows = 23
    x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
    x[1, :] += 60.0  # exp(x + max) would overflow here: the corrected Subtract keeps it finite
    out = cuda.full((rows, cols), float("nan"), device="cuda")
    _ok(lib, lib.ko_probe_composed_rowop(0, cuda.from_numpy(x).cuda().data_ptr(), out.data_ptr(), rows, cols, 0.0, None, None,
                                         block, _stream(cuda)))
    y = out.cpu().numpy()
    assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= 1e-6
    assert oracle.max_rowsum_err(y) <= 1e-5


@pytest.mark.parametrize("block", [32, 64, 192, 1024])
@pytest.mark.parametrize("affine", [False, True])
def test_composed_layernorm_matches_the_oracle(cuda, lib, oracle, block, affine):
    rows, cols = 29, 768
    x = oracle.fill_normal((rows, cols), 1, 0, 0.0, 1.0)
    g = oracle.fill_uniform((cols,), 1, 1, 0.5, 1.5) if affine else None
    b = oracle.fill_normal((cols,), 1, 2, 0.0, 0.1) if affine else None
    gd = cuda.from_numpy(g).cuda() if affine else None
    bd = cuda.from_numpy(b).cuda() if affine else None
    out = cuda.full((rows, cols), float("nan"), device="cuda")
    _ok(lib, lib.ko_probe_composed_rowop(1, cuda.from_numpy(x).cuda().data_ptr(), out.data_ptr(), rows, cols, 1e-12,
                                         gd.data_ptr() if affine else None, bd.data_ptr() if affine else None, block,
                                         _stream(cuda)))
    assert oracle.max_rel_err(out.cpu().numpy(), oracle.layernorm_f64(x, 1e-12, g, b)) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (256, 384, 64), (100, 36, 52), (129, 65, 17), (300, 200, 1000), (128, 128, 64),
                                   (1000, 520, 200), (2048, 1024, 4096), (131, 4104, 72), (20000, 128, 256)])
@pytest.mark.parametrize("with_c", [False, True])
def test_reference_tensor_core_template_through_its_launch_syntax(cuda, lib, oracle, M, N, K, with_c):
    """gemm<GemmKernelTensorCore<half, ...>><<<grid, thread_per_block, smem>>>: half operands, row-major B, FP32 accumulation,
    D rounded once to half; against the float64 product of the rounded inputs.  K and N multiples of 8 run on tcgen05 (operand
    tiles copied into the swizzled layouts by cp.async, descriptors built in the kernel), other shapes on the FP32 pipe; tails in
    M, N and K, one to 64 K-blocks, more tiles than blocks."""
    ab = oracle.to_f16_bits(oracle.fill_uniform((M, K), 3, 0))
    bb = oracle.to_f16_bits(oracle.fill_uniform((K, N), 3, 1))
    cb = oracle.to_f16_bits(oracle.fill_uniform((M, N), 3, 2)) if with_c else None
    dev = lambda bits: cuda.from_numpy(bits.view(np.int16)).cuda()  # noqa: E731
    ad, bd = dev(ab), dev(bb)
    cd = dev(cb) if with_c else None
    dd = cuda.full((M, N), 0x7E00, dtype=cuda.int16, device="cuda")  # NaN
    _ok(lib, lib.ko_probe_gemm_tensor_core_template(M, N, K, ad.data_ptr(), bd.data_ptr(), cd.data_ptr() if with_c else None, dd.data_ptr(),
                                                    _stream(cuda)))
    cuda.cuda.synchronize()
    got = oracle.from_f16_bits(dd.cpu().numpy().view(np.uint16)).astype(np.float64)
    want = oracle.from_f16_bits(ab).astype(np.float64) @ oracle.from_f16_bits(bb).astype(np.float64)
    if with_c:
        want = want + oracle.from_f16_bits(cb).astype(np.float64)
    assert np.isfinite(got).all()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3


@pytest.mark.parametrize("K", [8, 16, 64])
def test_reference_mma_and_ldmatrix_names(cuda, lib, oracle, K):
    """MMA<16,8,8> (mma.sync, FP16 accumulation) fed by LDMatrix<2,false> / LDMatrix<1,true> as in the reference's warp loop.
    Small integers: every product and partial sum is exact in FP16, so D must equal A @ B + C exactly."""
    rng = np.random.default_rng(K)
    a = rng.integers(-4, 5, size=(16, K)).astype(np.float32)
    b = rng.integers(-4, 5, size=(K, 8)).astype(np.float32)
    c = rng.integers(-8, 9, size=(16, 8)).astype(np.float32)
    dev = lambda m: cuda.from_numpy(oracle.to_f16_bits(m).view(np.int16)).cuda()  # noqa: E731
    ad, bd, cd = dev(a), dev(b), dev(c)
    dd = cuda.full((16, 8), 0x7E00, dtype=cuda.int16, device="cuda")  # NaN
    _ok(lib, lib.ko_probe_mma_ldmatrix(ad.data_ptr(), bd.data_ptr(), cd.data_ptr(), dd.data_ptr(), K, _stream(cuda)))
    cuda.cuda.synchronize()
    got = oracle.from_f16_bits(dd.cpu().numpy().view(np.uint16))
    assert np.array_equal(got, a @ b + c)
    assert lib.ko_probe_mma_ldmatrix(ad.data_ptr(), bd.data_ptr(), cd.data_ptr(), dd.data_ptr(), 12, _stream(cuda)) != 0
