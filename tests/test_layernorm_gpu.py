"""GPU parity of ko_layernorm_f32 / ko_layernorm_bf16 (through the C ABI) against the float64
oracle and size-independent properties at the full shapes.

Tolerance (benchmark specification): max-rel <= 1e-5 with max-rel = max |y - ref| / max(|ref|, 1).  BF16 output is
compared with the BF16-rounded oracle: at most a rounding-boundary flip (one BF16 ulp) is allowed
and only on a small fraction of the elements."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_REL = 1e-5


def _inputs(oracle, rows, cols, seed=1):
    return (oracle.fill_normal((rows, cols), seed, 0, 0.0, 1.0), oracle.fill_uniform((cols,), seed, 1, 0.5, 1.5),
            oracle.fill_normal((cols,), seed, 2, 0.0, 0.1))


def _run_f32(cuda, lib, x, eps, g=None, b=None, ddof=0, inplace=False, **knobs):
    from kernel_optimization_b200.native import RowKnobs

    xd = cuda.from_numpy(x).cuda()
    gd = None if g is None else cuda.from_numpy(g).cuda()
    bd = None if b is None else cuda.from_numpy(b).cuda()
    yd = xd if inplace else cuda.empty_like(xd)
    rows, cols = x.shape
    rc = lib.ko_layernorm_f32_tuned(xd.data_ptr(), yd.data_ptr(), rows, cols, eps, None if gd is None else gd.data_ptr(),
                                    None if bd is None else bd.data_ptr(), ddof, RowKnobs(**knobs) if knobs else None,
                                    cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert rc == 0, lib.ko_last_error_string()
    assert lib.ko_poll_device_status() == 0, lib.ko_last_error_string()
    return yd.cpu().numpy()


def _dev_bf16(cuda, bits):
    return cuda.from_numpy(bits.view(np.int16)).cuda().view(cuda.bfloat16)


def _run_bf16(cuda, lib, xb, eps, gb=None, bb=None, ddof=0, **knobs):
    from kernel_optimization_b200.native import RowKnobs

    xd = _dev_bf16(cuda, xb)
    gd = None if gb is None else _dev_bf16(cuda, gb)
    bd = None if bb is None else _dev_bf16(cuda, bb)
    yd = cuda.empty_like(xd)
    rows, cols = xb.shape
    rc = lib.ko_layernorm_bf16_tuned(xd.data_ptr(), yd.data_ptr(), rows, cols, eps, None if gd is None else gd.data_ptr(),
                                     None if bd is None else bd.data_ptr(), ddof, RowKnobs(**knobs) if knobs else None,
                                     cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert rc == 0, lib.ko_last_error_string()
    assert lib.ko_poll_device_status() == 0, lib.ko_last_error_string()
    return yd.view(cuda.int16).cpu().numpy().view(np.uint16)


SHAPES = [(1, 1), (3, 1), (5, 4), (7, 100), (5, 131), (100, 128), (33, 256), (1000, 768), (37, 1024), (64, 2048),
          (9, 2052), (11, 4096), (5, 12288), (2, 32768), (3, 40000), (2, 131072)]


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_f32_against_float64_oracle(cuda, lib, oracle, rows, cols):
    x, g, b = _inputs(oracle, rows, cols)
    assert oracle.max_rel_err(_run_f32(cuda, lib, x, 1e-12, g, b), oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
    assert oracle.max_rel_err(_run_f32(cuda, lib, x, 1e-5, None, None, 1), oracle.layernorm_f64(x, 1e-5, None, None, 1)) <= TOL_REL
    assert oracle.max_rel_err(_run_f32(cuda, lib, x, 1e-5, g, None), oracle.layernorm_f64(x, 1e-5, g, None)) <= TOL_REL


def test_f32_is_not_the_reference_kernels_arithmetic(cuda, lib, oracle, golden):
    """The reference's kernel output on the same input (committed fixture) is not LayerNorm; the
    product follows the mathematical operator, the documented deviation."""
    x, _g, _b = _inputs(oracle, 8, 768)
    y = _run_f32(cuda, lib, x, 1e-4)
    assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-4)) <= TOL_REL
    assert np.abs(y - golden["layernorm_8x768_warp"]).max() > 10.0


GEOMETRIES = [dict(tier=1, rows_per_warp=1, block=64), dict(tier=1, rows_per_warp=2, block=128), dict(tier=1, block=256, grid_cap=5),
              dict(tier=1, rows_per_warp=2, grid_cap=1), dict(tier=4), dict(tier=4, rows_per_warp=1, stages=2),
              dict(tier=4, rows_per_warp=2, stages=3, ctas_per_sm=2), dict(tier=4, stage_rows=8, stages=2)]


@pytest.mark.parametrize("knobs", GEOMETRIES, ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items()))
def test_f32_warp_and_staged_tiers_give_the_same_rows(cuda, lib, oracle, knobs):
    for rows, cols in ((77, 128), (77, 256), (130, 512), (77, 768), (77, 1024), (40, 2048), (90, 772)):
        x, g, b = _inputs(oracle, rows, cols)
        y = _run_f32(cuda, lib, x, 1e-12, g, b, 0, **knobs)
        assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=1))
        assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL


@pytest.mark.parametrize("block", [128, 256, 512, 1024])
def test_f32_block_tier_thread_counts(cuda, lib, oracle, block):
    for cols in (768, 2048, 4096, 8192):
        x, g, b = _inputs(oracle, 19, cols)
        assert oracle.max_rel_err(_run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=2, block=block), oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL


@pytest.mark.parametrize("block", [0, 128, 256, 512, 1024])
def test_f32_resident_tier(cuda, lib, oracle, block):
    for rows, cols in ((19, 768), (300, 2048), (7, 2052), (5, 16384), (40, 4096)):
        if block and cols // 4 > block * 4:
            continue
        x, g, b = _inputs(oracle, rows, cols)
        for gg, bb in ((g, b), (None, None), (g, None)):
            y = _run_f32(cuda, lib, x, 1e-12, gg, bb, 0, tier=5, block=block, grid_cap=3 if rows > 100 else 0)
            assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-12, gg, bb)) <= TOL_REL


def test_resident_tier_with_768_and_896_threads(cuda, lib, oracle):
    """Rows of 2049..3072 vectors take 768 threads with four vectors each, rows of 3073..3584 vectors 896 (the default
    there, and block = 768 / 896 on request): exactly filled, partly filled, more rows than blocks, with and without
    the affine parameters, in place."""
    for block, rows, cols in ((768, 5, 12288), (768, 33, 9216), (768, 7, 8196), (768, 300, 10240), (768, 2, 12284),
                              (896, 5, 14336), (896, 40, 12292), (896, 300, 13312)):
        x, g, b = _inputs(oracle, rows, cols)
        for gg, bb in ((g, b), (None, None)):
            want = oracle.layernorm_f64(x, 1e-12, gg, bb)
            y = _run_f32(cuda, lib, x, 1e-12, gg, bb, 0, tier=5, block=block, grid_cap=3 if rows > 100 else 0)
            assert oracle.max_rel_err(y, want) <= TOL_REL
            assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, gg, bb))          # the default for such rows
            assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, gg, bb, 0, inplace=True, tier=5, block=block))
    # shorter rows fit too (threads without data), longer ones are refused
    x, g, b = _inputs(oracle, 9, 4096)
    assert oracle.max_rel_err(_run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=5, block=768), oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL


@pytest.mark.parametrize("lanes", [0, 4, 8, 16, 32])
@pytest.mark.parametrize("slots", [0, 1, 2, 4])
def test_lane_group_tier_for_short_rows(cuda, lib, oracle, lanes, slots):
    """tier 9: a row per group of 4 / 8 / 16 / 32 lanes (up to four vectors per lane), several row slots per group,
    persistent warps with gamma / beta unpacked once.  Rows that fill the group exactly, partly, or leave lanes idle;
    row counts that are not a multiple of the rows per warp step; one block walking every row (grid_cap = 1); with and
    without the affine parameters; ddof; FP32 and BF16; in place."""
    for rows, cols in ((1, 4), (7, 8), (1000, 32), (333, 64), (77, 96), (501, 128), (65, 200), (129, 256), (40, 512)):
        nvec = cols // 4
        if lanes and (lanes * 4 < nvec):
            continue
        x, g, b = _inputs(oracle, rows, cols)
        x += 2.0
        knobs = dict(tier=9, stage_rows=lanes, rows_per_warp=slots)
        y = _run_f32(cuda, lib, x, 1e-12, g, b, 0, **knobs)
        assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
        assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, 0, grid_cap=1, **knobs))
        assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, 0, inplace=True, **knobs))
        y = _run_f32(cuda, lib, x, 1e-5, None, None, 1, **knobs)
        assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-5, None, None, 1)) <= TOL_REL
        y = _run_f32(cuda, lib, x, 1e-5, None, b, 0, **knobs)
        assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-5, None, b)) <= TOL_REL
    for rows, cols in ((9, 8), (1001, 64), (77, 96), (300, 128), (65, 200), (129, 256), (33, 320), (40, 512), (17, 1024)):
        nvec = cols // 8
        if lanes and (lanes * 4 < nvec):
            continue
        x, g, b = _inputs(oracle, rows, cols)
        xb, gb, bb = oracle.to_bf16_bits(x), oracle.to_bf16_bits(g), oracle.to_bf16_bits(b)
        got = oracle.from_bf16_bits(_run_bf16(cuda, lib, xb, 1e-12, gb, bb, tier=9, stage_rows=lanes, rows_per_warp=slots))
        want = oracle.layernorm_f64(oracle.from_bf16_bits(xb), 1e-12, oracle.from_bf16_bits(gb), oracle.from_bf16_bits(bb))
        assert oracle.max_rel_err(got, want) <= 2.0 ** -8 * 1.01


def test_short_rows_default_to_the_lane_group_tier(cuda, lib, oracle):
    for rows, cols in ((1000, 32), (500, 64), (300, 192)):
        x, g, b = _inputs(oracle, rows, cols)
        assert np.array_equal(_run_f32(cuda, lib, x, 1e-12, g, b), _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=9))
    x, g, b = _inputs(oracle, 400, 512)
    xb, gb, bb = oracle.to_bf16_bits(x), oracle.to_bf16_bits(g), oracle.to_bf16_bits(b)
    assert np.array_equal(_run_bf16(cuda, lib, xb, 1e-12, gb, bb), _run_bf16(cuda, lib, xb, 1e-12, gb, bb, tier=9))


@pytest.mark.parametrize("block", [0, 128, 256, 512, 1024])
def test_resident_tier_row_ring_gives_the_bits_of_the_register_prefetch(cuda, lib, oracle, block):
    """stages = 3: the block's next rows are in flight into shared memory (cp.async, every thread copies the vectors it
    will consume); stages = 1: one row prefetched into registers.  Same arithmetic, so the same bits -- for rows that
    fill the threads exactly, partly, or leave whole warps without data; more rows than ring slots per block (the
    slots are refilled), fewer rows than slots, FP32 and BF16."""
    for rows, cols in ((19, 768), (300, 2048), (7, 2052), (40, 4096), (33, 2560), (50, 3072), (2, 1024), (101, 520)):
        if block and cols // 4 > block * 4:
            continue
        x, g, b = _inputs(oracle, rows, cols)
        for cap in (0, 3):
            ring = _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=5, block=block, stages=3, grid_cap=cap)
            assert oracle.max_rel_err(ring, oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
            assert np.array_equal(ring, _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=5, block=block, stages=1, grid_cap=cap))
        assert np.array_equal(_run_f32(cuda, lib, x, 1e-12, g, b, 0, inplace=True, tier=5, block=block, stages=3), ring)
    for rows, cols in ((21, 4096), (50, 5120), (33, 3072), (9, 8192), (300, 2304)):
        if block and cols // 8 > block * 4:
            continue
        x, g, b = _inputs(oracle, rows, cols)
        xb, gb, bb = oracle.to_bf16_bits(x), oracle.to_bf16_bits(g), oracle.to_bf16_bits(b)
        ring = _run_bf16(cuda, lib, xb, 1e-12, gb, bb, tier=5, block=block, stages=3, grid_cap=2)
        assert np.array_equal(ring, _run_bf16(cuda, lib, xb, 1e-12, gb, bb, tier=5, block=block, stages=1, grid_cap=2))
        want = oracle.layernorm_f64(oracle.from_bf16_bits(xb), 1e-12, oracle.from_bf16_bits(gb), oracle.from_bf16_bits(bb))
        assert oracle.max_rel_err(oracle.from_bf16_bits(ring), want) <= 2.0 ** -8 * 1.01


@pytest.mark.parametrize("cluster", [0, 2, 4, 8])
def test_cluster_tier_merges_triples_through_dsmem(cuda, lib, oracle, cluster):
    for rows, cols in ((5, 4096), (3, 40000), (37, 8192), (2, 131072), (300, 2048), (3, 1028)):
        x, g, b = _inputs(oracle, rows, cols)
        y = _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=6, cluster=cluster)
        assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
        assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=6, cluster=cluster, grid_cap=16))
    x, g, b = _inputs(oracle, 4, 65536)
    xb, gb, bb = oracle.to_bf16_bits(x), oracle.to_bf16_bits(g), oracle.to_bf16_bits(b)
    got = oracle.from_bf16_bits(_run_bf16(cuda, lib, xb, 1e-12, gb, bb, tier=6, cluster=cluster))
    want = oracle.layernorm_f64(oracle.from_bf16_bits(xb), 1e-12, oracle.from_bf16_bits(gb), oracle.from_bf16_bits(bb))
    assert oracle.max_rel_err(got, want) <= 2.0 ** -8 * 1.01


@pytest.mark.parametrize("block", [0, 256, 512, 1024])
@pytest.mark.parametrize("pair", [1, 2])
def test_reread_tier_two_passes_per_row(cuda, lib, oracle, block, pair):
    """tier 8: statistics in a first pass (chunked exact triples merged Chan-wise), the row again from the L2 in the
    second; rows_per_warp = 2 takes two rows at a time and loads gamma / beta once for both (an odd row count leaves
    the last block with one row).  Rows shorter than a step, rows ending inside a step, more rows than blocks."""
    for rows, cols in ((5, 4), (3, 4100), (7, 40000), (301, 36864), (3, 262144), (2, 524288 + 8)):
        x, g, b = _inputs(oracle, rows, cols)
        x += 3.0  # a mean well away from zero: a one-pass sum of squares would lose digits here
        y = _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=8, block=block, rows_per_warp=pair)
        assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
        assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=8, block=block, rows_per_warp=pair, grid_cap=3))
        assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, 0, inplace=True, tier=8, block=block, rows_per_warp=pair))
        y = _run_f32(cuda, lib, x, 1e-5, None, None, 1, tier=8, block=block, rows_per_warp=pair)
        assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-5, None, None, 1)) <= TOL_REL
        if pair == 1:
            # every row load through the per-thread shared-memory ring of (row, pass, chunk) items: the same chunks, so
            # the same bits as the direct loads
            ring = _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=8, block=block, rows_per_warp=1, stages=3)
            assert np.array_equal(ring, _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=8, block=block, rows_per_warp=1, stages=1))
            assert np.array_equal(ring, _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=8, block=block, rows_per_warp=1, stages=3, grid_cap=3))
            assert np.array_equal(ring, _run_f32(cuda, lib, x, 1e-12, g, b, 0, inplace=True, tier=8, block=block, rows_per_warp=1, stages=3))
    x, g, b = _inputs(oracle, 5, 65536 + 16)
    xb, gb, bb = oracle.to_bf16_bits(x), oracle.to_bf16_bits(g), oracle.to_bf16_bits(b)
    got = oracle.from_bf16_bits(_run_bf16(cuda, lib, xb, 1e-12, gb, bb, tier=8, block=block, rows_per_warp=pair))
    want = oracle.layernorm_f64(oracle.from_bf16_bits(xb), 1e-12, oracle.from_bf16_bits(gb), oracle.from_bf16_bits(bb))
    assert oracle.max_rel_err(got, want) <= 2.0 ** -8 * 1.01
    got = oracle.from_bf16_bits(_run_bf16(cuda, lib, xb, 1e-12, gb, bb, tier=8, block=block, rows_per_warp=1, stages=3))
    assert oracle.max_rel_err(got, want) <= 2.0 ** -8 * 1.01


def test_long_rows_default_to_the_reread_tier_or_the_cluster_tier(cuda, lib, oracle):
    """FP32 rows beyond 16384 columns take two passes per row unless there are fewer rows than SMs and a cluster can
    hold the row; rows of any length are served."""
    for rows, cols, knobs in ((3, 65536, dict(tier=6)), (200, 40000, dict(tier=8)), (300, 20480, dict(tier=8, block=256)),
                              (2, 600000, dict(tier=8)), (150, 131072, dict(tier=8, rows_per_warp=2))):
        x, g, b = _inputs(oracle, rows, cols)
        y = _run_f32(cuda, lib, x, 1e-12, g, b)
        assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
        assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, 0, **knobs))


def test_f32_stream_tier_and_staged_ring_wrap(cuda, lib, oracle):
    x, g, b = _inputs(oracle, 23, 768)
    assert oracle.max_rel_err(_run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=3), oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
    x, g, b = _inputs(oracle, 148 * 8 * 12 + 5, 256)
    y = _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=4, stage_rows=8, stages=2, rows_per_warp=1)
    assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, 0, tier=1))


def test_f32_edge_rows(cuda, lib, oracle):
    const = np.full((4, 768), 3.25, dtype=np.float32)
    assert np.array_equal(_run_f32(cuda, lib, const, 1e-12), np.zeros_like(const))      # var = 0
    x, g, b = _inputs(oracle, 300, 768)
    x += 10.0   # common offset of 10 sigma; FP32 statistics lose about |mean|/sigma * 2^-24 per unit of offset
    assert oracle.max_rel_err(_run_f32(cuda, lib, x, 1e-12, g, b), oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
    far = x + 990.0   # offset 1000 sigma: the mean itself is only representable to 6e-5
    assert oracle.max_rel_err(_run_f32(cuda, lib, far, 1e-12, g, b), oracle.layernorm_f64(far, 1e-12, g, b)) <= 5e-4
    y = _run_f32(cuda, lib, x, 1e-12, g, b)
    assert np.array_equal(_run_f32(cuda, lib, x, 1e-12, g, b, inplace=True), y)
    assert np.array_equal(_run_f32(cuda, lib, x, 1e-12, g, b), y)


def test_f32_full_bert_shape(cuda, lib, oracle, ko):
    """C2: [16384, 768], x ~ N(0,1), gamma ~ U(0.5,1.5), beta ~ N(0,0.1^2), eps 1e-12, seed 1: the whole
    tensor against the oracle, plus the property that un-affined output rows have mean 0 / variance 1."""
    rows, cols = 16384, 768
    x = ko.fill_normal((rows, cols), 1, 0, 0.0, 1.0)
    g, b = ko.fill_uniform((cols,), 1, 1, 0.5, 1.5), ko.fill_normal((cols,), 1, 2, 0.0, 0.1)
    assert oracle.max_rel_err(_run_f32(cuda, lib, x, 1e-12, g, b), oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
    y = _run_f32(cuda, lib, x, 1e-12).astype(np.float64)
    assert np.abs(y.mean(1)).max() <= 1e-6 and np.abs(y.var(1) - 1.0).max() <= 1e-5


BF16_SHAPES = [(3, 1), (5, 8), (7, 100), (100, 256), (1000, 768), (64, 2048), (9, 2056), (37, 4096), (11, 8192),
               (3, 40000)]


def test_cluster_tier_mailboxes_and_barriers_agree(cuda, lib, oracle):
    """The cluster tier exchanges (n, mean, M2) through peer mailboxes + mbarriers (default) or between cluster barriers
    (stages=2): same values in the same rank order, so the same bits."""
    for rows, cols in ((5, 65536), (40, 40000), (3, 262144), (37, 8192)):
        x, g, b = _inputs(oracle, rows, cols)
        y = _run_f32(cuda, lib, x, 1e-12, g, b, tier=6)
        assert oracle.max_rel_err(y, oracle.layernorm_f64(x, 1e-12, g, b)) <= TOL_REL
        assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, tier=6, stages=2))
        assert np.array_equal(y, _run_f32(cuda, lib, x, 1e-12, g, b, tier=6, grid_cap=8))   # one cluster, many rows: phases flip


@pytest.mark.parametrize("rows,cols", BF16_SHAPES)
def test_bf16_against_rounded_oracle(cuda, lib, oracle, rows, cols):
    x, g, b = _inputs(oracle, rows, cols)
    xb, gb, bb = oracle.to_bf16_bits(x), oracle.to_bf16_bits(g), oracle.to_bf16_bits(b)
    want = oracle.layernorm_f64(oracle.from_bf16_bits(xb), 1e-12, oracle.from_bf16_bits(gb), oracle.from_bf16_bits(bb))
    got_bits = _run_bf16(cuda, lib, xb, 1e-12, gb, bb)
    want_bits = oracle.to_bf16_bits(want.astype(np.float32))
    got, want_r = oracle.from_bf16_bits(got_bits), oracle.from_bf16_bits(want_bits)
    assert np.mean(got_bits != want_bits) <= 2e-3, "only rounding-boundary flips may differ"
    assert np.abs(got - want_r).max() <= np.abs(want_r).max() * 2.0 ** -7      # at most one BF16 ulp
    assert oracle.max_rel_err(got, want) <= 2.0 ** -8 * 1.01                    # half an ulp of BF16 rounding


@pytest.mark.parametrize("knobs", [dict(tier=1), dict(tier=2, block=128), dict(tier=2, block=256), dict(tier=2, block=512),
                                   dict(tier=2, block=1024), dict(tier=3), dict(tier=4), dict(tier=4, stages=2, ctas_per_sm=2),
                                   dict(tier=5), dict(tier=5, block=128), dict(tier=5, block=512, grid_cap=3), dict(tier=5, block=1024)],
                         ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items()))
def test_bf16_tiers_agree(cuda, lib, oracle, knobs):
    for rows, cols in ((21, 4096), (50, 1024), (33, 776)):
        x, g, b = _inputs(oracle, rows, cols)
        xb, gb, bb = oracle.to_bf16_bits(x), oracle.to_bf16_bits(g), oracle.to_bf16_bits(b)
        base = _run_bf16(cuda, lib, xb, 1e-12, gb, bb, tier=1)
        assert np.mean(_run_bf16(cuda, lib, xb, 1e-12, gb, bb, **knobs) != base) <= 2e-3


def test_bf16_scaled_shard_properties(cuda, lib, oracle, ko):
    """A slice of C5's LayerNorm: BF16 [32768, 4096] (1/8 of the rows), seed 4: sampled rows against the
    oracle, every row by mean/variance of the un-affined output."""
    rows, cols = 32768, 4096
    xb = ko.fill_normal((rows, cols), 4, 0, 0.0, 1.0, dtype=2)
    got = oracle.from_bf16_bits(_run_bf16(cuda, lib, xb, 1e-12))
    assert np.abs(got.mean(1, dtype=np.float64)).max() <= 2e-3 and np.abs(got.var(1, dtype=np.float64) - 1.0).max() <= 1e-2
    pick = np.r_[0:64, rows - 64:rows, np.random.default_rng(4).integers(0, rows, 512)]
    want = oracle.layernorm_f64(oracle.from_bf16_bits(xb[pick]), 1e-12)
    assert oracle.max_rel_err(got[pick], want) <= 2.0 ** -8 * 1.01
