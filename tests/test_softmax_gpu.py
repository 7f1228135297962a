"""GPU parity of ko_softmax_f32 (through the C ABI) against the float64 oracle, the committed
outputs of the reference's own kernel, and size-independent properties at the full shapes.

Tolerances (benchmark specification): max-abs <= 1e-6, every row sum within 1e-5 of 1."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_ABS, TOL_ROWSUM = 1e-6, 1e-5


def _run(cuda, lib, x, inplace=False, **knobs):
    from kernel_optimization_b200.native import RowKnobs

    xd = cuda.from_numpy(x).cuda()
    yd = xd if inplace else cuda.empty_like(xd)
    s = cuda.cuda.current_stream().cuda_stream
    rows, cols = x.shape
    if knobs:
        rc = lib.ko_softmax_f32_tuned(xd.data_ptr(), yd.data_ptr(), rows, cols, RowKnobs(**knobs), s)
    else:
        rc = lib.ko_softmax_f32(xd.data_ptr(), yd.data_ptr(), rows, cols, s)
    cuda.cuda.synchronize()
    if rc == 3 and knobs.get("tier") == 4 and knobs.get("stage_rows"):
        return None  # an explicit ring geometry that does not fit in shared memory is refused, not shrunk
    assert rc == 0, lib.ko_last_error_string()
    assert lib.ko_poll_device_status() == 0, lib.ko_last_error_string()
    return yd.cpu().numpy()


SHAPES = [(1, 1), (3, 1), (5, 4), (7, 100), (5, 131), (1000, 128), (37, 512), (33, 640), (64, 2048), (9, 2052),
          (11, 4096), (6, 12288), (2, 32768), (2, 32772), (3, 40000), (2, 131072),
          # block tier with exactly the threads a row needs (a multiple of 32, four vectors each)
          (5, 4100), (7, 8196), (3, 9216), (4, 10240), (2, 16380), (9, 2304), (6, 3328), (5, 2816)]


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


GEOMETRIES = [dict(tier=1, rows_per_warp=1, block=128), dict(tier=1, rows_per_warp=2, block=256),
              dict(tier=1, rows_per_warp=4, block=64), dict(tier=1, rows_per_warp=8), dict(tier=1, rows_per_warp=4, grid_cap=3),
              dict(tier=1, grid_cap=1), dict(tier=4), dict(tier=4, rows_per_warp=1, stages=2), dict(tier=4, rows_per_warp=2, stages=3, ctas_per_sm=2),
              dict(tier=4, rows_per_warp=4, stage_rows=32, stages=5), dict(tier=4, stage_rows=8, stages=2)]


@pytest.mark.parametrize("knobs", GEOMETRIES, ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items()))
def test_warp_and_staged_tiers_give_the_same_rows_for_every_geometry(cuda, lib, oracle, knobs):
    for rows, cols in ((131, 128), (131, 256), (257, 512), (131, 768), (70, 1024), (131, 1536), (67, 2048), (300, 132)):
        x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
        y = _run(cuda, lib, x, **knobs)
        if y is None:
            assert rows * cols * 4 > 100000, "only large explicit rings may be refused"
            continue
        assert np.array_equal(y, _run(cuda, lib, x, tier=1)), (cols, "row results must not depend on tier or geometry")
        assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS


@pytest.mark.parametrize("tier", [2, 3])
def test_block_and_stream_tiers(cuda, lib, oracle, tier):
    for rows, cols in ((9, 128), (5, 4096), (3, 32768), (4, 1000)):
        x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
        y = _run(cuda, lib, x, tier=tier)
        assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS and oracle.max_rowsum_err(y) <= TOL_ROWSUM


@pytest.mark.parametrize("cluster", [0, 2, 4, 8])
def test_cluster_tier_exchanges_partials_through_dsmem(cuda, lib, oracle, cluster):
    for rows, cols in ((5, 4096), (3, 40000), (37, 8192), (2, 131072), (300, 2048), (2, 262144), (3, 1028)):
        x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
        y = _run(cuda, lib, x, tier=6, cluster=cluster)
        assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS and oracle.max_rowsum_err(y) <= TOL_ROWSUM
        assert np.array_equal(y, _run(cuda, lib, x, tier=6, cluster=cluster, grid_cap=16))  # fewer clusters, more rows each


@pytest.mark.parametrize("rows,cols", [(5, 4096), (37, 8192), (3, 20000), (7, 32768), (300, 16388), (2, 4)])
def test_prefetching_block_tier_matches_the_block_tier(cuda, lib, oracle, rows, cols):
    """tier 7: the block's next row lands in shared memory (bulk copy) while the current one is reduced from registers;
    same arithmetic as the block tier, so the same bits, for any number of rows per block (phase bit flips)."""
    x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
    y = _run(cuda, lib, x, tier=7)
    assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS and oracle.max_rowsum_err(y) <= TOL_ROWSUM
    assert np.array_equal(y, _run(cuda, lib, x, tier=2))
    assert np.array_equal(y, _run(cuda, lib, x, tier=7, grid_cap=2))   # two blocks take all rows: many refills each
    assert lib.ko_poll_device_status() == 0


@pytest.mark.parametrize("block", [0, 256, 512, 1024])
def test_reread_tier_two_passes_per_row(cuda, lib, oracle, block):
    """tier 8: one row per block in two passes (online max / sum, then the row again from the L2).  Rows shorter than
    one step of the block, rows that end inside a step, more rows than blocks, and fully masked stretches (-inf) that
    span whole chunks of a thread."""
    for rows, cols in ((5, 4), (3, 4100), (7, 40000), (300, 36864), (2, 262144), (3, 524288 + 8), (150, 65536)):
        x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
        if cols >= 40000:
            x[0, : cols // 2] = -np.inf      # the first half of a row contributes nothing
            x[-1, 17:cols - 5] = -np.inf     # almost everything masked
        y = _run(cuda, lib, x, tier=8, block=block)
        assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS and oracle.max_rowsum_err(y) <= TOL_ROWSUM
        assert np.array_equal(y, _run(cuda, lib, x, tier=8, block=block, grid_cap=3))  # three blocks take all rows
        assert np.array_equal(y, _run(cuda, lib, x, inplace=True, tier=8, block=block))  # out == in: a thread rewrites only what it read
        # every load through the per-thread shared-memory ring of (row, pass, chunk) items, or none: same arithmetic
        ring = _run(cuda, lib, x, tier=8, block=block, stages=3)
        assert np.array_equal(ring, _run(cuda, lib, x, tier=8, block=block, stages=1))
        assert np.array_equal(ring, _run(cuda, lib, x, tier=8, block=block, stages=3, grid_cap=3))
        assert np.array_equal(ring, _run(cuda, lib, x, inplace=True, tier=8, block=block, stages=3))
        assert oracle.max_abs_err(ring, oracle.softmax_f64(x)) <= TOL_ABS
    assert lib.ko_poll_device_status() == 0


def test_long_rows_default_to_the_reread_tier_or_the_cluster_tier(cuda, lib, oracle):
    """Beyond 32768 columns: fewer rows than SMs -> one row per cluster; otherwise two passes per row.  Same results
    as the forced tiers, and rows of any length are served (the cluster tier stops at 262144 columns)."""
    for rows, cols, tier in ((3, 65536, 6), (200, 40000, 8), (2, 300000, 8)):
        x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
        y = _run(cuda, lib, x)
        assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS
        assert np.array_equal(y, _run(cuda, lib, x, tier=tier))


def test_cluster_tier_with_and_without_prefetch(cuda, lib, oracle):
    """Slices beyond 4096 vectors per block are prefetched into shared memory (stages=1 turns that off): same bits."""
    for rows, cols in ((5, 65536), (40, 40000), (3, 262144), (300, 36864)):
        x = oracle.fill_normal((rows, cols), 0, 0, 0.0, 2.0)
        y = _run(cuda, lib, x, tier=6)
        assert oracle.max_abs_err(y, oracle.softmax_f64(x)) <= TOL_ABS
        assert np.array_equal(y, _run(cuda, lib, x, tier=6, stages=1))   # no prefetch, cluster barriers
        assert np.array_equal(y, _run(cuda, lib, x, tier=6, stages=2))   # prefetch, cluster barriers instead of mailboxes
        assert np.array_equal(y, _run(cuda, lib, x, tier=6, grid_cap=4))

    assert lib.ko_poll_device_status() == 0


def test_staged_tier_many_stages_per_block(cuda, lib, oracle):
    """Enough rows that every persistent block wraps its ring several times (phase bits flip)."""
    x = oracle.fill_normal((148 * 8 * 40 + 13, 128), 0, 0, 0.0, 2.0)
    y = _run(cuda, lib, x, tier=4, stage_rows=8, stages=2, rows_per_warp=1)
    assert np.array_equal(y, _run(cuda, lib, x, tier=1))
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
