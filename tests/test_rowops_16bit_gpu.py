"""GPU parity of the 16-bit row operators (ko_softmax_f16 / ko_softmax_bf16 / ko_layernorm_f16, through the
C ABI) against the float64 oracle evaluated on the widened inputs.

The arithmetic is FP32 and the result is rounded once, so the sharp statement is about bits: the output
must equal the oracle's result rounded to the output type, except for rounding-boundary flips (one ulp, on a
small fraction of the elements).  The error bounds follow from that: half an ulp of the output type on top
of the FP32 tolerances (FP16: 2^-11 relative, BF16: 2^-9)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HALF_ULP = {"f16": 2.0 ** -11, "bf16": 2.0 ** -9}


def _conv(oracle, kind):
    return (oracle.to_f16_bits, oracle.from_f16_bits) if kind == "f16" else (oracle.to_bf16_bits, oracle.from_bf16_bits)


def _dev(cuda, bits, kind):
    return cuda.from_numpy(bits.view(np.int16)).cuda().view(cuda.float16 if kind == "f16" else cuda.bfloat16)


def _bits(cuda, t):
    return t.view(cuda.int16).cpu().numpy().view(np.uint16)


def _softmax(cuda, lib, kind, xb, inplace=False):
    xd = _dev(cuda, xb, kind)
    yd = xd if inplace else cuda.empty_like(xd)
    rows, cols = xb.shape
    fn = lib.ko_softmax_f16 if kind == "f16" else lib.ko_softmax_bf16
    rc = fn(xd.data_ptr(), yd.data_ptr(), rows, cols, cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert rc == 0, lib.ko_last_error_string()
    return _bits(cuda, yd)


# every tier and lane-group size: 8..2048 columns (warp tier), ..16384 (block tier: 256 threads with up to 4 or 8
# vectors each, 512 with 4), longer rows in two passes (reread tier: a row that ends inside a step, several steps per
# row, more rows than blocks), odd counts (stream tier)
SOFTMAX_SHAPES = [(1, 8), (5, 64), (7, 128), (9, 136), (33, 256), (100, 512), (64, 1024), (17, 2048), (9, 2056), (5, 4096),
                  (3, 8192), (5, 10248), (4, 12288), (3, 16384), (4, 16392), (2, 32768), (2, 40000), (3, 262152), (200, 65536),
                  (3000, 20480), (3, 1), (5, 7), (4, 100), (3, 1001),
                  # block tier with exactly the threads a row needs: three vectors per thread up to 3072 columns, six beyond,
                  # up to 24576 columns; rows that fill the threads and rows one vector longer
                  (5, 3072), (5, 3080), (6, 7168), (4, 11264), (3, 13320), (3, 24576), (3, 24584)]


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("rows,cols", SOFTMAX_SHAPES)
def test_softmax_16bit_against_rounded_oracle(cuda, lib, oracle, kind, rows, cols):
    to_bits, from_bits = _conv(oracle, kind)
    xb = to_bits(oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0))
    want = oracle.softmax_f64(from_bits(xb))
    got_bits = _softmax(cuda, lib, kind, xb)
    want_bits = to_bits(want.astype(np.float32))
    got = from_bits(got_bits)
    # flips only where the FP32 value (error <= 1e-6) straddles a rounding boundary
    assert np.mean(got_bits != want_bits) <= 5e-3
    assert np.abs(got.astype(np.float64) - want).max() <= HALF_ULP[kind] * 1.01 + 1e-6       # outputs are <= 1
    # the rounded probabilities still sum to 1 within the accumulated rounding of `cols` terms
    assert np.abs(got.sum(1, dtype=np.float64) - 1.0).max() <= 2 * HALF_ULP[kind]
    assert np.array_equal(_softmax(cuda, lib, kind, xb, inplace=True), got_bits)


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_softmax_16bit_extreme_rows(cuda, lib, oracle, kind):
    """Statistics are FP32: the largest finite FP16 inputs (for BF16: 1e8, the operators' stated range is
    |x| < 1e9, as for FP32 rows), a one-hot row and a constant row are exact."""
    to_bits, from_bits = _conv(oracle, kind)
    big = 65504.0 if kind == "f16" else 1.0e8
    x = np.zeros((4, 256), dtype=np.float32)
    x[0, :] = big
    x[1, :] = -big
    x[2, :] = -big
    x[2, 17] = big
    x[3, :] = 1.5
    got = from_bits(_softmax(cuda, lib, kind, to_bits(x)))
    assert np.isfinite(got).all()
    uniform = from_bits(to_bits(np.full(256, 1.0 / 256, dtype=np.float32)))
    assert np.array_equal(got[0], uniform) and np.array_equal(got[1], uniform) and np.array_equal(got[3], uniform)
    assert got[2, 17] == 1.0 and got[2].sum() == 1.0


def test_softmax_16bit_causal_block(cuda, lib, oracle, ko):
    """The masked-attention pattern of the scaled sweep (entries above the diagonal of every 512-row block are
    -1e4) in BF16: masked probabilities are exactly zero."""
    rows, cols = 1024, 512
    x = ko.fill_normal((rows, cols), 4, 0, 0.0, 2.0)
    ko.fill_causal_mask_(x, 0, 512, -1e4)
    xb = oracle.to_bf16_bits(x)
    got = oracle.from_bf16_bits(_softmax(cuda, lib, "bf16", xb))
    r, c = np.indices((rows, cols))
    assert (got[c > (r % 512)] == 0).all()
    want = oracle.softmax_f64(oracle.from_bf16_bits(xb))
    assert np.abs(got - want).max() <= HALF_ULP["bf16"] * 1.01 + 1e-6


def _layernorm_f16(cuda, lib, xb, eps, gb=None, bb=None, ddof=0, **knobs):
    from kernel_optimization_b200.native import RowKnobs

    xd = _dev(cuda, xb, "f16")
    gd = None if gb is None else _dev(cuda, gb, "f16")
    bd = None if bb is None else _dev(cuda, bb, "f16")
    yd = cuda.empty_like(xd)
    rows, cols = xb.shape
    rc = lib.ko_layernorm_f16_tuned(xd.data_ptr(), yd.data_ptr(), rows, cols, eps, None if gd is None else gd.data_ptr(),
                                    None if bd is None else bd.data_ptr(), ddof, RowKnobs(**knobs) if knobs else None,
                                    cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert rc == 0, lib.ko_last_error_string()
    assert lib.ko_poll_device_status() == 0, lib.ko_last_error_string()
    return _bits(cuda, yd)


LN_SHAPES = [(3, 8), (7, 104), (100, 128), (33, 256), (1000, 768), (37, 1024), (64, 2048), (9, 2056), (11, 4096), (5, 12288),
             (2, 32768), (3, 40000), (5, 131), (3, 1)]


@pytest.mark.parametrize("rows,cols", LN_SHAPES)
@pytest.mark.parametrize("affine", [True, False])
def test_layernorm_f16_against_rounded_oracle(cuda, lib, oracle, rows, cols, affine):
    x = oracle.fill_normal((rows, cols), 1, 0, 0.0, 1.0)
    g, b = oracle.fill_uniform((cols,), 1, 1, 0.5, 1.5), oracle.fill_normal((cols,), 1, 2, 0.0, 0.1)
    xb = oracle.to_f16_bits(x)
    gb, bb = (oracle.to_f16_bits(g), oracle.to_f16_bits(b)) if affine else (None, None)
    eps = 1e-5   # a single-column row has zero variance: eps decides the scale, keep it representable
    want = oracle.layernorm_f64(oracle.from_f16_bits(xb), eps, None if gb is None else oracle.from_f16_bits(gb),
                                None if bb is None else oracle.from_f16_bits(bb))
    got_bits = _layernorm_f16(cuda, lib, xb, eps, gb, bb)
    want_bits = oracle.to_f16_bits(want.astype(np.float32))
    got = oracle.from_f16_bits(got_bits)
    assert np.mean(got_bits != want_bits) <= 2e-3, "only rounding-boundary flips may differ"
    assert oracle.max_rel_err(got, want) <= HALF_ULP["f16"] * 1.01 + 1e-5


@pytest.mark.parametrize("knobs", [dict(tier=1), dict(tier=2, block=256), dict(tier=2, block=1024), dict(tier=3), dict(tier=4),
                                   dict(tier=5), dict(tier=5, block=512, grid_cap=3)],
                         ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items()))
def test_layernorm_f16_tiers_agree(cuda, lib, oracle, knobs):
    for rows, cols in ((21, 4096), (50, 1024), (33, 776)):
        x = oracle.fill_normal((rows, cols), 1, 0, 0.0, 1.0)
        xb = oracle.to_f16_bits(x)
        gb, bb = oracle.to_f16_bits(oracle.fill_uniform((cols,), 1, 1, 0.5, 1.5)), oracle.to_f16_bits(oracle.fill_normal((cols,), 1, 2, 0.0, 0.1))
        base = _layernorm_f16(cuda, lib, xb, 1e-5, gb, bb, tier=1)
        assert np.mean(_layernorm_f16(cuda, lib, xb, 1e-5, gb, bb, **knobs) != base) <= 2e-3


def test_python_wrappers_accept_16bit_tensors(cuda, oracle, ko):
    x = cuda.randn((64, 512), device="cuda")
    for dt in (cuda.float16, cuda.bfloat16):
        xh = x.to(dt)
        p = ko.softmax(xh)
        assert p.dtype == dt and cuda.allclose(p.float(), cuda.softmax(xh.float(), dim=1), atol=4e-3)
        y = ko.layernorm(xh, 1e-5)
        ref = cuda.nn.functional.layer_norm(xh.float(), (512,), eps=1e-5)
        assert y.dtype == dt and cuda.allclose(y.float(), ref, atol=3e-2)


def test_16bit_entry_points_validate_their_arguments(cuda, lib):
    s = cuda.cuda.current_stream().cuda_stream
    x = cuda.zeros((4, 64), dtype=cuda.float16, device="cuda")
    for fn in (lib.ko_softmax_f16, lib.ko_softmax_bf16):
        assert fn(x.data_ptr(), x.data_ptr(), 0, 64, s) == 0            # empty: nothing to do
        assert fn(x.data_ptr(), x.data_ptr(), 4, 0, s) == 0
        assert fn(None, x.data_ptr(), 4, 64, s) == 1                    # NULL pointer
        assert fn(x.data_ptr(), x.data_ptr(), -1, 64, s) == 1           # negative shape
    assert lib.ko_layernorm_f16(x.data_ptr(), x.data_ptr(), 0, 64, 1e-5, None, None, 0, s) == 0
    assert lib.ko_layernorm_f16(None, x.data_ptr(), 4, 64, 1e-5, None, None, 0, s) == 1
    assert lib.ko_layernorm_f16(x.data_ptr(), x.data_ptr(), 4, 64, 1e-5, None, None, 2, s) == 1   # ddof outside {0, 1}
    cuda.cuda.synchronize()
