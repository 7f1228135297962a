"""GPU parity of ko_gemm_f16_f32 / ko_gemm_bf16_f32 (tcgen05, through the C ABI) against the float64
oracle on the rounded inputs.  Tolerance (benchmark specification): relative Frobenius error <= 1e-3; with exact
products and FP32 accumulation the kernel actually lands near 1e-6, which is asserted too so that
a dropped K-step or a mis-addressed tile cannot hide under the loose bound."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_FRO = 1e-3


def tight(K):
    """FP32 accumulation over K terms: about sqrt(K) * 2^-24, with head-room."""
    return 2e-6 * max(1.0, (K / 256.0) ** 0.5)


def _bits(oracle, kind):
    return (oracle.to_f16_bits, oracle.from_f16_bits) if kind == "f16" else (oracle.to_bf16_bits, oracle.from_bf16_bits)


def _dev16(cuda, bits, kind):
    return cuda.from_numpy(bits.view(np.int16)).cuda().view(cuda.float16 if kind == "f16" else cuda.bfloat16)


def _run(cuda, lib, kind, ab, bb, c=None, bn=0, store_mode=0, out16=False, b_row_major=False):
    """ab: [M,K] bits; bb: [N,K] bits (column-major B) or, with b_row_major, [K,N] bits; c: float32 [M,N] or, with
    out16, bits of the input type.  Returns float32 D, or D's bits with out16."""
    M, K = ab.shape
    N = bb.shape[1] if b_row_major else bb.shape[0]
    ad, bd = _dev16(cuda, ab, kind), _dev16(cuda, bb, kind)
    if out16:
        cd = None if c is None else _dev16(cuda, c, kind)
        dd = _dev16(cuda, np.full((M, N), 0x7e00 if kind == "f16" else 0x7fc0, dtype=np.uint16), kind)   # NaN
    else:
        cd = None if c is None else cuda.from_numpy(c).cuda()
        dd = cuda.full((M, N), float("nan"), dtype=cuda.float32, device="cuda")
    out_fmt = 0 if not out16 else (1 if kind == "f16" else 2)
    rc = lib.ko_gemm_tc_tuned(0 if kind == "f16" else 1, out_fmt, 1 if b_row_major else 0, M, N, K, ad.data_ptr(), bd.data_ptr(),
                              None if cd is None else cd.data_ptr(), dd.data_ptr(), bn, store_mode, cuda.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.ko_last_error_string()
    cuda.cuda.synchronize()
    assert lib.ko_poll_device_status() == 0, lib.ko_last_error_string()
    if out16:
        return dd.view(cuda.int16).cpu().numpy().view(np.uint16)
    return dd.cpu().numpy()


def _case(cuda, lib, oracle, kind, M, N, K, with_c=False, bn=0, seed=3, store_mode=0):
    to_bits, from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), seed, 0)), to_bits(oracle.fill_uniform((N, K), seed, 1))
    c = oracle.fill_uniform((M, N), seed, 2) if with_c else None
    d = _run(cuda, lib, kind, ab, bb, c, bn, store_mode)
    want = oracle.gemm_tn_f64(from_bits(ab), from_bits(bb), c)
    err = oracle.rel_frobenius(d, want)
    assert err <= TOL_FRO and err <= tight(K), (kind, M, N, K, bn, err)
    return d


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("bn", [64, 128, 256, 512])   # 512: the 256 x 256 tile (two 128-row halves per CTA)
def test_single_tile_and_k_steps(cuda, lib, oracle, kind, bn):
    for K in (64, 128, 8, 72, 1024):
        _case(cuda, lib, oracle, kind, 128, min(bn, 256), K, bn=bn)
        if bn == 512:
            _case(cuda, lib, oracle, kind, 256, 256, K, bn=bn)


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (1, 4, 8), (100, 36, 56), (129, 260, 136), (1000, 520, 200),
                                   (2048, 1024, 512), (131, 4100, 64), (5000, 12, 320)])
def test_tails_and_multiple_tiles(cuda, lib, oracle, kind, M, N, K):
    for bn in (0, 128):
        _case(cuda, lib, oracle, kind, M, N, K, bn=bn)
    _case(cuda, lib, oracle, kind, M, N, K, with_c=True)


@pytest.mark.parametrize("bn", [64, 128, 256, 512])
def test_both_epilogues_give_the_same_bits(cuda, lib, oracle, bn):
    for M, N, K in ((128, 256, 64), (1000, 520, 200), (129, 260, 136), (4096, 1024, 128)):
        d_tma = _case(cuda, lib, oracle, "bf16", M, N, K, bn=bn, store_mode=1)
        d_direct = _case(cuda, lib, oracle, "bf16", M, N, K, bn=bn, store_mode=2)
        assert np.array_equal(d_tma, d_direct)


def test_n_not_multiple_of_four_takes_scalar_stores(cuda, lib, oracle):
    _case(cuda, lib, oracle, "bf16", 200, 37, 64)
    _case(cuda, lib, oracle, "f16", 200, 37, 64, with_c=True)


def test_more_tiles_than_sms_and_both_accumulators(cuda, lib, oracle):
    # 64 x 32 = 2048 tiles of 128 x 128: every CTA walks many tiles, alternating TMEM buffers
    _case(cuda, lib, oracle, "bf16", 8192, 4096, 64, bn=128)
    d1 = _case(cuda, lib, oracle, "f16", 4096, 4096, 256, bn=256)
    d2 = _case(cuda, lib, oracle, "f16", 4096, 4096, 256, bn=128)
    assert oracle.rel_frobenius(d2, d1.astype(np.float64)) <= tight(256)


def test_exact_small_integers(cuda, lib, oracle):
    """Inputs that are small integers make every product and partial sum exact: the result must
    equal the integer matrix product bit for bit, whatever the accumulation order."""
    rng = np.random.default_rng(3)
    M, N, K = 384, 320, 192
    a, b = rng.integers(-4, 5, (M, K)).astype(np.float32), rng.integers(-4, 5, (N, K)).astype(np.float32)
    want = (a.astype(np.int64) @ b.astype(np.int64).T).astype(np.float32)
    for kind in ("f16", "bf16"):
        to_bits, _ = _bits(oracle, kind)
        assert np.array_equal(_run(cuda, lib, kind, to_bits(a), to_bits(b)), want)


def test_baseline_shapes(cuda, lib, oracle, ko):
    """C4: 4096^3 and the BERT FFN shape 16384 x 3072 x 768, U(-1,1) seed 3.  The float64 oracle
    checks 64 full rows (first/last tile rows included) and 4096 random entries; cuBLAS-free."""
    rng = np.random.default_rng(3)
    for kind, code in (("f16", 1), ("bf16", 2)):
        _, from_bits = _bits(oracle, kind)
        for M, N, K in ((4096, 4096, 4096), (16384, 3072, 768)):
            ab, bb = ko.fill_uniform((M, K), 3, 0, dtype=code), ko.fill_uniform((N, K), 3, 1, dtype=code)
            d = _run(cuda, lib, kind, ab, bb)
            rows = np.unique(np.r_[0:16, M - 16:M, rng.integers(0, M, 32)])
            want = oracle.gemm_tn_f64(from_bits(ab[rows]), from_bits(bb))
            assert oracle.rel_frobenius(d[rows], want) <= tight(K)
            ri, ci = rng.integers(0, M, 4096), rng.integers(0, N, 4096)
            spot = np.einsum("ik,ik->i", from_bits(ab[ri]).astype(np.float64), from_bits(bb[ci]).astype(np.float64))
            assert np.abs(d[ri, ci] - spot).max() <= 1e-3 * np.abs(spot).max()
            assert np.isfinite(d).all()


def test_argument_checks(cuda, lib):
    s = cuda.cuda.current_stream().cuda_stream
    a = cuda.zeros((128, 64), dtype=cuda.bfloat16, device="cuda")
    d = cuda.zeros((128, 128), dtype=cuda.float32, device="cuda")
    assert lib.ko_gemm_bf16_f32(128, 128, 60, a.data_ptr(), a.data_ptr(), None, d.data_ptr(), s) == 3   # K % 8
    assert lib.ko_gemm_bf16_f32(128, 128, 64, a.data_ptr() + 2, a.data_ptr(), None, d.data_ptr(), s) == 2  # alignment
    assert lib.ko_gemm_bf16_f32(128, 128, 64, None, a.data_ptr(), None, d.data_ptr(), s) == 1
    assert lib.ko_gemm_bf16_f32(0, 128, 64, None, None, None, None, s) == 0


# ---------------------------------------------------------------------------------------------------
# row-major B (the reference driver's layout) and 16-bit D (the reference's ElementC = half)
# ---------------------------------------------------------------------------------------------------
# A 16-bit D carries its own rounding: half an ulp per element, 2^-11 relative for FP16 and 2^-9 for BF16, so the
# 1e-3 bound (stated for FP32 output) holds for FP16 and becomes 2^-9 for BF16.  The sharp check is the other one:
# the 16-bit result must equal the FP32 result rounded once, bit for bit.
TOL_OUT16 = {"f16": TOL_FRO, "bf16": 2.0 ** -9}
@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("bn", [0, 64, 128, 256, 512])
@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (128, 256, 16), (256, 512, 256), (100, 40, 56), (129, 264, 136),
                                   (1000, 520, 200), (2048, 1024, 512), (131, 4104, 64), (5000, 16, 320)])
def test_row_major_b_matches_column_major_bits(cuda, lib, oracle, kind, bn, M, N, K):
    """Same products, same accumulation order: the two B layouts must agree bit for bit."""
    to_bits, from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), 3, 0)), to_bits(oracle.fill_uniform((N, K), 3, 1))
    d_col = _run(cuda, lib, kind, ab, bb, bn=bn)
    d_row = _run(cuda, lib, kind, ab, np.ascontiguousarray(bb.T), bn=bn, b_row_major=True)
    assert np.array_equal(d_col, d_row)
    err = oracle.rel_frobenius(d_row, oracle.gemm_tn_f64(from_bits(ab), from_bits(bb)))
    assert err <= TOL_FRO and err <= tight(K)


def test_row_major_b_needs_a_16_byte_pitch(cuda, lib):
    a = cuda.zeros((128, 64), dtype=cuda.bfloat16, device="cuda")
    b = cuda.zeros((64, 36), dtype=cuda.bfloat16, device="cuda")
    d = cuda.zeros((128, 36), dtype=cuda.float32, device="cuda")
    rc = lib.ko_gemm_tc(1, 0, 1, 128, 36, 64, a.data_ptr(), b.data_ptr(), None, d.data_ptr(), cuda.cuda.current_stream().cuda_stream)
    assert rc == 3 and "multiple of 8" in lib.ko_last_error_string().decode()


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("store_mode", [1, 2])
@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (256, 512, 256), (100, 40, 56), (129, 264, 136), (1000, 520, 200),
                                   (2048, 1024, 512), (5000, 16, 320)])
def test_16_bit_output_is_the_fp32_result_rounded_once(cuda, lib, oracle, kind, store_mode, M, N, K):
    to_bits, from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), 3, 0)), to_bits(oracle.fill_uniform((N, K), 3, 1))
    d32 = _run(cuda, lib, kind, ab, bb)
    for bn in (0, 64):
        d16 = _run(cuda, lib, kind, ab, bb, bn=bn, store_mode=store_mode, out16=True)
        assert np.array_equal(d16, to_bits(d32 if bn == 0 else _run(cuda, lib, kind, ab, bb, bn=bn)))
    want = oracle.gemm_tn_f64(from_bits(ab), from_bits(bb))
    assert oracle.rel_frobenius(from_bits(d16).astype(np.float64), want) <= TOL_OUT16[kind]


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (200, 37, 64), (129, 264, 136), (1000, 520, 200)])
def test_16_bit_output_with_c_and_odd_pitch(cuda, lib, oracle, kind, M, N, K):
    """D = round(acc + C) with C in D's type; N = 37 takes the scalar stores."""
    to_bits, from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), 3, 0)), to_bits(oracle.fill_uniform((N, K), 3, 1))
    cb = to_bits(oracle.fill_uniform((M, N), 3, 2))
    d16 = _run(cuda, lib, kind, ab, bb, c=cb, out16=True)
    d32 = _run(cuda, lib, kind, ab, bb, c=from_bits(cb))       # FP32 path: acc + C in FP32
    assert np.array_equal(d16, to_bits(d32))
    want = oracle.gemm_tn_f64(from_bits(ab), from_bits(bb), from_bits(cb))
    assert oracle.rel_frobenius(from_bits(d16).astype(np.float64), want) <= TOL_OUT16[kind]


def test_named_16_bit_entry_points_and_row_major_16_bit(cuda, lib, oracle):
    s = cuda.cuda.current_stream().cuda_stream
    for kind, fn, out_fmt in (("f16", lib.ko_gemm_f16_f16, 1), ("bf16", lib.ko_gemm_bf16_bf16, 2)):
        to_bits, from_bits = _bits(oracle, kind)
        M, N, K = 384, 320, 192
        ab, bb = to_bits(oracle.fill_uniform((M, K), 5, 0)), to_bits(oracle.fill_uniform((N, K), 5, 1))
        ad, bd, btd = _dev16(cuda, ab, kind), _dev16(cuda, bb, kind), _dev16(cuda, np.ascontiguousarray(bb.T), kind)
        d1 = _dev16(cuda, np.zeros((M, N), np.uint16), kind)
        d2 = _dev16(cuda, np.zeros((M, N), np.uint16), kind)
        assert fn(M, N, K, ad.data_ptr(), bd.data_ptr(), None, d1.data_ptr(), s) == 0
        assert lib.ko_gemm_tc(0 if kind == "f16" else 1, out_fmt, 1, M, N, K, ad.data_ptr(), btd.data_ptr(), None, d2.data_ptr(), s) == 0
        cuda.cuda.synchronize()
        assert lib.ko_poll_device_status() == 0
        assert cuda.equal(d1.view(cuda.int16), d2.view(cuda.int16))
        got = from_bits(d1.view(cuda.int16).cpu().numpy().view(np.uint16)).astype(np.float64)
        assert oracle.rel_frobenius(got, oracle.gemm_tn_f64(from_bits(ab), from_bits(bb))) <= TOL_OUT16[kind]


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 256), (1000, 520, 200), (129, 264, 136), (2048, 1024, 512), (300, 8, 64),
                                   (5000, 300, 320), (38000, 256, 64)])
def test_256_row_tile_gives_the_bits_of_the_128_row_tile(cuda, lib, oracle, kind, M, N, K):
    """bn = 512: a CTA computes 256 x 256 (two 128-row halves share each B tile, single-buffered accumulators); every
    output still sees the same MMAs in the same order.  (38000 rows: more tiles than SMs, both accumulator phases.)"""
    to_bits, from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), 3, 0)), to_bits(oracle.fill_uniform((N, K), 3, 1))
    c = oracle.fill_uniform((M, N), 3, 2)
    base = _run(cuda, lib, kind, ab, bb, bn=256)
    assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=512), base)
    assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=512, store_mode=2), base)
    assert np.array_equal(_run(cuda, lib, kind, ab, bb, c, bn=512), _run(cuda, lib, kind, ab, bb, c, bn=256))
    assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=512, out16=True), _run(cuda, lib, kind, ab, bb, bn=256, out16=True))
    if M <= 5000:
        err = oracle.rel_frobenius(base, oracle.gemm_tn_f64(from_bits(ab), from_bits(bb)))
        assert err <= TOL_FRO and err <= tight(K)


def test_general_entry_point_validates_its_arguments(cuda, lib):
    s = cuda.cuda.current_stream().cuda_stream
    a = cuda.zeros((128, 64), dtype=cuda.bfloat16, device="cuda")
    b = cuda.zeros((64, 64), dtype=cuda.bfloat16, device="cuda")
    d = cuda.zeros((128, 64), dtype=cuda.float32, device="cuda")
    ok = (1, 0, 0, 128, 64, 64, a.data_ptr(), b.data_ptr(), None, d.data_ptr(), s)
    assert lib.ko_gemm_tc(*ok) == 0
    assert lib.ko_gemm_tc(2, *ok[1:]) == 1                                   # unknown input format
    assert lib.ko_gemm_tc(1, 3, *ok[2:]) == 1                                # unknown output format
    assert lib.ko_gemm_tc(1, 0, 2, *ok[3:]) == 1                             # unknown B layout
    assert lib.ko_gemm_tc(1, 0, 0, 128, 64, 60, *ok[6:]) == 3                # K not a multiple of 8
    assert lib.ko_gemm_tc(1, 0, 0, 0, 64, 64, *ok[6:]) == 0                  # empty output
    assert lib.ko_gemm_tc(1, 0, 0, 128, 64, 64, a.data_ptr(), b.data_ptr(), None, a.data_ptr(), s) == 1   # D aliases A
    assert lib.ko_gemm_tc(1, 0, 0, 128, 64, 64, a.data_ptr() + 2, b.data_ptr(), None, d.data_ptr(), s) == 2  # unaligned A
    cuda.cuda.synchronize()
    assert lib.ko_poll_device_status() == 0


# ---------------------------------------------------------------------------------------------------
# uneven column tiles (bn = 1024 / 1280), and cuBLAS as a second oracle
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(4096, 4096, 128), (2048, 8192, 64), (5000, 1000, 72), (38000, 520, 64), (19000, 1032, 64)])
def test_uneven_column_tiles_give_the_bits_of_equal_tiles(cuda, lib, oracle, kind, M, N, K):
    """N cut into a few more, narrower column tiles (widths multiples of 32, wide tiles dealt first) so that the last
    round of CTAs is full: every output is still one chain of the same MMAs, so the bits are those of the 256-column
    tiling.  Shapes with more tiles than CTAs; some have a clipped last tile; both tile heights, both epilogues, with C."""
    to_bits, from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), 3, 0)), to_bits(oracle.fill_uniform((N, K), 3, 1))
    base = _run(cuda, lib, kind, ab, bb, bn=256)
    s = cuda.cuda.current_stream().cuda_stream
    ran = 0
    for bn in (1024, 1280):
        ad, bd = _dev16(cuda, ab, kind), _dev16(cuda, bb, kind)
        probe = cuda.empty((M, N), dtype=cuda.float32, device="cuda")
        rc = lib.ko_gemm_tc_tuned(0 if kind == "f16" else 1, 0, 0, M, N, K, ad.data_ptr(), bd.data_ptr(), None, probe.data_ptr(), bn, 0, s)
        cuda.cuda.synchronize()
        if rc == 3:
            continue  # this tile height gains nothing from uneven tiles at this shape: refused, nothing launched
        assert rc == 0, lib.ko_last_error_string()
        ran += 1
        assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=bn), base)
        assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=bn, store_mode=2), base)
        if M <= 5000:
            c = oracle.fill_uniform((M, N), 3, 2)
            assert np.array_equal(_run(cuda, lib, kind, ab, bb, c, bn=bn), _run(cuda, lib, kind, ab, bb, c, bn=256))
            assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=bn, out16=True), _run(cuda, lib, kind, ab, bb, bn=256, out16=True))
    assert ran >= 1, "no tile height used uneven column tiles at this shape"
    assert np.array_equal(_run(cuda, lib, kind, ab, bb), base)  # whatever the default picks
    if M * N <= 5000 * 4096:
        err = oracle.rel_frobenius(base, oracle.gemm_tn_f64(from_bits(ab), from_bits(bb)))
        assert err <= TOL_FRO and err <= tight(K)


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(4096, 4096, 4096), (16384, 3072, 768)])
def test_benchmark_shapes_against_cublas(cuda, lib, kind, M, N, K):
    """The whole output of both benchmark shapes against cuBLAS (torch.mm with FP32 output) on the same device operands:
    the second oracle for this kernel, whose reference counterpart is disabled.  Both accumulate exact products in
    FP32, in different orders: relative Frobenius difference within tight(K)."""
    tdt = cuda.float16 if kind == "f16" else cuda.bfloat16
    gen = cuda.Generator(device="cuda")
    gen.manual_seed(3)
    a = (cuda.rand((M, K), device="cuda", generator=gen) * 2 - 1).to(tdt)
    b = (cuda.rand((N, K), device="cuda", generator=gen) * 2 - 1).to(tdt)
    d = cuda.full((M, N), float("nan"), dtype=cuda.float32, device="cuda")
    fn = lib.ko_gemm_f16_f32 if kind == "f16" else lib.ko_gemm_bf16_f32
    assert fn(M, N, K, a.data_ptr(), b.data_ptr(), None, d.data_ptr(), cuda.cuda.current_stream().cuda_stream) == 0, lib.ko_last_error_string()
    cuda.cuda.synchronize()
    assert lib.ko_poll_device_status() == 0
    want = cuda.mm(a, b.t(), out_dtype=cuda.float32)
    rel = ((d.double() - want.double()).norm() / want.double().norm()).item()
    assert rel <= tight(K), rel
    assert bool(cuda.isfinite(d).all())


# ---------------------------------------------------------------------------------------------------
# the two-SM kernel (tcgen05 cta_group::2): bn = 2048 (equal column tiles) / 2304 (uneven)
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (128, 64, 64), (1, 4, 8), (100, 36, 56), (129, 264, 136), (1000, 520, 200),
                                   (2048, 1024, 512), (5000, 300, 320), (38000, 256, 64), (20000, 1032, 72)])
def test_two_sm_kernel_gives_the_bits_of_the_one_sm_kernel(cuda, lib, oracle, kind, M, N, K):
    """A pair of CTAs computes a 256 x 256 tile with tcgen05.mma.cta_group::2, each CTA loading its own rows of A and its
    own half of the B tile: every output is the same chain of MMAs in the same K order, so the bits equal the single-CTA
    kernel's.  Tails in M, N and K; fewer tiles than pairs and many more (both accumulator buffers, ring wrap-around);
    TMA-store and direct epilogues; + C; 16-bit D."""
    to_bits, from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), 3, 0)), to_bits(oracle.fill_uniform((N, K), 3, 1))
    base = _run(cuda, lib, kind, ab, bb, bn=256)
    assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=2048), base)
    assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=2048, store_mode=2), base)
    if M <= 5000:
        c = oracle.fill_uniform((M, N), 3, 2)
        assert np.array_equal(_run(cuda, lib, kind, ab, bb, c, bn=2048), _run(cuda, lib, kind, ab, bb, c, bn=256))
        assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=2048, out16=True), _run(cuda, lib, kind, ab, bb, bn=256, out16=True))
        err = oracle.rel_frobenius(base, oracle.gemm_tn_f64(from_bits(ab), from_bits(bb)))
        assert err <= TOL_FRO and err <= tight(K)


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (128, 64, 64), (100, 40, 56), (129, 264, 136), (1000, 520, 200), (2048, 1024, 512),
                                   (5000, 304, 320), (20000, 1032, 72)])
def test_two_sm_kernel_with_row_major_b(cuda, lib, oracle, kind, M, N, K):
    """Row-major B [K,N] on the two-SM kernel: each CTA loads its 128 columns as two MN-major boxes.  Same bits as the
    column-major two-SM call on the transposed matrix and as the single-CTA row-major call; FP32 and 16-bit D."""
    to_bits, from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), 3, 0)), to_bits(oracle.fill_uniform((N, K), 3, 1))
    b_rm = np.ascontiguousarray(bb.T)
    base = _run(cuda, lib, kind, ab, bb, bn=2048)
    assert np.array_equal(_run(cuda, lib, kind, ab, b_rm, bn=2048, b_row_major=True), base)
    assert np.array_equal(_run(cuda, lib, kind, ab, b_rm, bn=256, b_row_major=True), base)
    assert np.array_equal(_run(cuda, lib, kind, ab, b_rm, bn=2048, b_row_major=True, store_mode=2), base)
    assert np.array_equal(_run(cuda, lib, kind, ab, b_rm, bn=2048, b_row_major=True, out16=True), _run(cuda, lib, kind, ab, bb, bn=256, out16=True))
    err = oracle.rel_frobenius(base, oracle.gemm_tn_f64(from_bits(ab), from_bits(bb)))
    assert err <= TOL_FRO and err <= tight(K)


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(4096, 4096, 128), (19000, 1032, 64), (38000, 520, 64)])
def test_two_sm_kernel_with_uneven_column_tiles(cuda, lib, oracle, kind, M, N, K):
    to_bits, _from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), 3, 0)), to_bits(oracle.fill_uniform((N, K), 3, 1))
    base = _run(cuda, lib, kind, ab, bb, bn=256)
    assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=2304), base)
    assert np.array_equal(_run(cuda, lib, kind, ab, bb, bn=2304, store_mode=2), base)


# ---- K slices: few tiles, long K (FP32 partial tiles through the context's scratch, second kernel adds them in K order)

def _slices(bn, n):
    return bn | (n << 16)


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("bn", [64, 128, 256, 512])
@pytest.mark.parametrize("slices", [2, 3, 7])
@pytest.mark.parametrize("M,N,K", [(128, 256, 1024), (300, 520, 2048), (257, 72, 776), (130, 130, 136), (1, 4, 8)])
def test_k_slices_against_the_oracle(cuda, lib, oracle, kind, bn, slices, M, N, K):
    # more slices than K-blocks is clamped; tails in M, N and K; TMA-store epilogue where D allows it
    _case(cuda, lib, oracle, kind, M, N, K, bn=_slices(bn, slices))


@pytest.mark.parametrize("slices", [2, 5])
@pytest.mark.parametrize("M,N,K", [(300, 520, 2048), (200, 37, 640)])
def test_k_slices_with_c_direct_stores_and_odd_pitch(cuda, lib, oracle, slices, M, N, K):
    _case(cuda, lib, oracle, "bf16", M, N, K, with_c=True, bn=_slices(256, slices), store_mode=2)
    _case(cuda, lib, oracle, "f16", M, N, K, with_c=True, bn=_slices(128, slices))


def test_k_slices_are_deterministic_and_close_to_the_unsliced_bits(cuda, lib, oracle):
    M, N, K = 384, 768, 4096
    to_bits, from_bits = _bits(oracle, "bf16")
    ab, bb = to_bits(oracle.fill_uniform((M, K), 5, 0)), to_bits(oracle.fill_uniform((N, K), 5, 1))
    whole = _run(cuda, lib, "bf16", ab, bb, bn=_slices(256, 1))
    first = _run(cuda, lib, "bf16", ab, bb, bn=_slices(256, 4))
    again = _run(cuda, lib, "bf16", ab, bb, bn=_slices(256, 4))
    assert np.array_equal(first, again)
    # the slices are FP32 sums of exact products added in K order: only the summation order differs
    assert oracle.rel_frobenius(first, whole) <= tight(K)
    # the same slices in another tile shape see the same K ranges per output: identical bits
    assert np.array_equal(first, _run(cuda, lib, "bf16", ab, bb, bn=_slices(128, 4)))


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_k_slices_with_16_bit_output_and_row_major_b(cuda, lib, oracle, kind):
    M, N, K = 200, 264, 1024
    to_bits, from_bits = _bits(oracle, kind)
    ab, bb = to_bits(oracle.fill_uniform((M, K), 6, 0)), to_bits(oracle.fill_uniform((N, K), 6, 1))
    cb = to_bits(oracle.fill_uniform((M, N), 6, 2))
    want32 = _run(cuda, lib, kind, ab, bb, from_bits(cb).astype(np.float32), bn=_slices(256, 3))
    got = _run(cuda, lib, kind, ab, bb, cb, bn=_slices(256, 3), out16=True)
    assert np.array_equal(got, to_bits(want32))   # the FP32 sum (+ C) rounded once
    rm = _run(cuda, lib, kind, ab, np.ascontiguousarray(bb.T), bn=_slices(256, 3), b_row_major=True)
    assert np.array_equal(rm, _run(cuda, lib, kind, ab, bb, bn=_slices(256, 3)))


@pytest.mark.parametrize("M,N,K", [(512, 768, 4096), (128, 128, 8192), (1024, 1024, 8192), (64, 64, 4096)])
def test_default_choice_for_few_tiles_and_long_k(cuda, lib, oracle, M, N, K):
    # shapes the launcher cuts into K slices by default
    _case(cuda, lib, oracle, "bf16", M, N, K)
    _case(cuda, lib, oracle, "f16", M, N, K, with_c=True)


def test_k_slices_argument_checks(cuda, lib):
    a = cuda.zeros((256, 256), dtype=cuda.bfloat16, device="cuda")
    d = cuda.zeros((256, 256), dtype=cuda.float32, device="cuda")
    s = cuda.cuda.current_stream().cuda_stream
    # not in the two-SM kernel, and at most 64 slices
    assert lib.ko_gemm_tc_tuned(1, 0, 0, 256, 256, 256, a.data_ptr(), a.data_ptr(), None, d.data_ptr(), _slices(2048, 2), 0, s) != 0
    assert lib.ko_gemm_tc_tuned(1, 0, 0, 256, 256, 256, a.data_ptr(), a.data_ptr(), None, d.data_ptr(), _slices(256, 65), 0, s) != 0
    cuda.cuda.synchronize()
