"""GPU parity of ko_softmax_f32 (through the C ABI) against the float64 oracle, the committed
outputs of the reference's own kernel, and size-independent properties at the full shapes.

Tolerances (BASELINE): max-abs <= 1e-6, every row sum within 1e-5 of 1."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_ABS, TOL_ROWSUM = 1e-6, 1e-5


def _run(cuda, lib, x, rpw=0, block=0, cap=0, inplace=False):
    xd = cuda.from_numpy(x).cuda()
    yd = xd if inplace else cuda.empty_like(xd)
    s = cuda.cuda.current_stream().cuda_stream
    rows, cols = x.shape
    if rpw or block or cap:
        rc = lib.ko_softmax_f32_tuned(xd.data_ptr(), yd.data_ptr(), rows, cols, rpw, block, cap, s)
    else:
        rc = lib.ko_softmax_f32(xd.data_ptr(), yd.data_ptr(), rows, cols, s)
    cuda.cuda.synchronize()
    assert rc == 0, lib.ko_last_error_string()
    return yd.cpu().numpy()


SHAPES = [(1, 1), (3, 1), (5, 4), (7, 100), (5, 131), (1000, 128), (37, 512), (33, 640), (64, 2048), (9, 2052),
          (11, 4096), (6, 12288), (2, 32768), (2, 32772), (3, 40000), (2, 131072)]


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_against_float64_oracle(cuda, lib, oracle, rows, cols):
    x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
    y = _run(cuda, lib, x)
    assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS
    assert oracle.max_rowsum_err(y) <= TOL_ROWSUM


def test_against_reference_kernel_outputs(cuda, lib, oracle, golden):
    x = oracle.fill_normal((32, 128), 0, 0, 0.0, 2.0)
    assert np.abs(_run(cuda, lib, x) - golden["softmax_32x128"]).max() <= TOL_ABS
    x = oracle.fill_normal((16, 512), 4, 0, 0.0, 2.0)
    oracle.causal_mask_(x, 0, 512, -1e4)
    assert np.abs(_run(cuda, lib, x) - golden["softmax_16x512_causal"]).max() <= TOL_ABS


@pytest.mark.parametrize("rpw,block,cap", [(1, 128, 0), (2, 256, 0), (4, 64, 0), (8, 256, 0), (4, 256, 3), (0, 0, 1)])
def test_every_launch_geometry_gives_the_same_rows(cuda, lib, oracle, rpw, block, cap):
    for cols in (128, 256, 512, 768, 1024, 1536, 2048):
        x = oracle.fill_normal((131, cols), 0, 0, 0.0, 2.0)
        y = _run(cuda, lib, x, rpw, block, cap)
        assert np.array_equal(y, _run(cuda, lib, x)), (cols, "row results must not depend on the launch geometry")
        assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS


def test_causal_blocks_and_extreme_logits(cuda, lib, oracle):
    x = oracle.fill_normal((1024, 512), 4, 0, 0.0, 2.0)
    oracle.causal_mask_(x, 0, 512, -1e4)
    y = _run(cuda, lib, x)
    assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS
    r, c = np.arange(1024)[:, None] % 512, np.arange(512)[None, :]
    assert np.all(y[c > r] == 0.0)              # masked entries vanish exactly
    assert y[0, 0] == 1.0 and y[512, 0] == 1.0  # rows with a single live entry
    # logits the reference's exp(x + max) cannot survive (2*max > 88.7)
    big = np.full((4, 128), 60.0, dtype=np.float32)
    big[:, 3] = 61.0
    yb = _run(cuda, lib, big)
    assert np.isfinite(yb).all() and oracle.max_abs_err(yb, oracle.softmax_f64(big)) <= TOL_ABS
    const = np.full((3, 640), -7.5, dtype=np.float32)
    assert np.allclose(_run(cuda, lib, const), 1.0 / 640, rtol=1e-6, atol=0)


def test_in_place_and_repeatable(cuda, lib, oracle):
    x = oracle.fill_normal((777, 128), 0, 0, 0.0, 2.0)
    y = _run(cuda, lib, x)
    assert np.array_equal(_run(cuda, lib, x, inplace=True), y)
    assert np.array_equal(_run(cuda, lib, x), y)


def test_unaligned_pointer_takes_the_scalar_path(cuda, lib, oracle):
    x = oracle.fill_normal((50, 128), 0, 0, 0.0, 2.0)
    buf = cuda.zeros(50 * 128 + 1, dtype=cuda.float32, device="cuda")
    buf[1:] = cuda.from_numpy(x).reshape(-1).cuda()
    out = cuda.empty(50 * 128 + 1, dtype=cuda.float32, device="cuda")
    rc = lib.ko_softmax_f32(buf.data_ptr() + 4, out.data_ptr() + 4, 50, 128, cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert rc == 0
    assert oracle.max_abs_err(out[1:].reshape(50, 128).cpu().numpy(), oracle.softmax_f64(x)) <= TOL_ABS


def test_full_bert_shape_properties(cuda, lib, oracle, ko):
    """C1: [196608, 128], logits N(0, 2^2) seed 0.  Sampled rows against the oracle, every row by
    properties: sums to 1, order-preserving, invariant to a per-row shift."""
    rows, cols = 196608, 128
    x = ko.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
    y = _run(cuda, lib, x)
    assert oracle.max_rowsum_err(y) <= TOL_ROWSUM
    pick = np.r_[0:512, rows - 512:rows, np.random.default_rng(0).integers(0, rows, 4096)]
    assert oracle.max_abs_err(y[pick], oracle.softmax_f64(x[pick])) <= TOL_ABS
    assert np.array_equal(np.argmax(y, 1), np.argmax(x, 1))
    shift = np.repeat(np.arange(rows, dtype=np.float32)[:, None] % 7 - 3, cols, 1)
    assert np.abs(_run(cuda, lib, x + shift) - y).max() <= 2e-6


def test_scaled_causal_shard(cuda, lib, oracle, ko):
    """One 1/8 shard of C5: [196608, 512] with the causal -1e4 pattern, seed 4; every row by
    properties, the first and last 512-row block plus random rows against the oracle."""
    rows, cols = 196608, 512
    x = ko.fill_normal((rows, cols), 4, 0, 0.0, 2.0)
    ko.fill_causal_mask_(x, 0, 512, -1e4)
    y = _run(cuda, lib, x)
    assert oracle.max_rowsum_err(y) <= TOL_ROWSUM
    pick = np.r_[0:512, rows - 512:rows, np.random.default_rng(4).integers(0, rows, 4096)]
    assert oracle.max_abs_err(y[pick], oracle.softmax_f64(x[pick])) <= TOL_ABS
    r, c = np.arange(rows)[:, None] % 512, np.arange(cols)[None, :]
    assert not y[c > r].any()
