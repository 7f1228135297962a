"""GPU parity of ko_sgemm_f32 (through the C ABI): relative Frobenius error <= 1e-6 against float64
(the benchmark's tolerance); without a K split also bit-identical to the FP32 oracle port (one FFMA per k in
ascending k, the reference's order) and to the committed outputs of the reference's own kernel."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_FRO = 1e-6


def _run(cuda, lib, a, b, c=None, variant=0, d_is_c=False, split_k=0):
    M, K = a.shape
    N = b.shape[1]
    ad, bd = cuda.from_numpy(a).cuda(), cuda.from_numpy(b).cuda()
    cd = None if c is None else cuda.from_numpy(c).cuda()
    dd = cd if d_is_c else cuda.empty((M, N), dtype=cuda.float32, device="cuda")
    rc = lib.ko_sgemm_f32_tuned(M, N, K, ad.data_ptr(), bd.data_ptr(), None if cd is None else cd.data_ptr(),
                                dd.data_ptr(), variant, split_k, cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert rc == 0, lib.ko_last_error_string()
    return dd.cpu().numpy()


SHAPES = [(1, 1, 1), (64, 64, 8), (100, 36, 52), (129, 65, 17), (256, 256, 256), (300, 200, 1000), (17, 513, 33),
          (128, 128, 1), (640, 384, 72)]


@pytest.mark.parametrize("variant", [1, 2, 3, 4, 6])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_unsplit_kernels_are_bit_identical_to_the_reference_order(cuda, lib, oracle, M, N, K, variant):
    a, b, c = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1), oracle.fill_uniform((M, N), 2, 2)
    for cc in (None, c):
        d = _run(cuda, lib, a, b, cc, variant, split_k=1)
        assert oracle.rel_frobenius(d, oracle.sgemm_f64(a, b, cc)) <= TOL_FRO
        assert np.array_equal(d, oracle.sgemm_f32(a, b, cc)), "same FFMA order as the reference => same bits"


@pytest.mark.parametrize("split_k", [0, 2, 3, 4, 8])
@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (300, 200, 1000), (129, 65, 170), (1024, 1024, 1024), (64, 64, 4096), (17, 513, 333),
                                   (2048, 1536, 512), (1920, 1152, 1000)])
def test_split_k_is_deterministic_and_within_tolerance(cuda, lib, oracle, M, N, K, split_k):
    a, b, c = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1), oracle.fill_uniform((M, N), 2, 2)
    for cc in (None, c):
        d = _run(cuda, lib, a, b, cc, 4, split_k=split_k)
        assert oracle.rel_frobenius(d, oracle.sgemm_f64(a, b, cc)) <= TOL_FRO
        assert np.array_equal(d, _run(cuda, lib, a, b, cc, 4, split_k=split_k)), "slices are added in a fixed order"
        # only the association of the K sum differs from the sequential order (whose own error grows with K)
        assert oracle.rel_frobenius(d, oracle.sgemm_f32(a, b, cc).astype(np.float64)) <= 3 * TOL_FRO


@pytest.mark.parametrize("variant", [7, 8])   # two groups of 4 warps on 128x128 tiles, four groups of 2 warps on 64x128 tiles
@pytest.mark.parametrize("split_k", [0, 1, 2, 3])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (128, 128, 16), (100, 36, 52), (129, 65, 17), (256, 256, 256), (300, 200, 1000),
                                   (17, 513, 33), (1024, 1024, 1024), (64, 64, 4096), (1920, 1152, 136)])
def test_warp_groups_split_k_inside_the_block(cuda, lib, oracle, M, N, K, variant, split_k):
    """The groups' K parts are added in K order through shared memory: deterministic, within the tolerance,
    and (a single K-tile has nothing to split) bit-identical to the reference order when K <= 16."""
    a, b, c = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1), oracle.fill_uniform((M, N), 2, 2)
    for cc in (None, c):
        d = _run(cuda, lib, a, b, cc, variant, split_k=split_k)
        assert oracle.rel_frobenius(d, oracle.sgemm_f64(a, b, cc)) <= TOL_FRO
        assert np.array_equal(d, _run(cuda, lib, a, b, cc, variant, split_k=split_k))
        seq = oracle.sgemm_f32(a, b, cc)
        assert oracle.rel_frobenius(d, seq.astype(np.float64)) <= 3 * TOL_FRO
        if K <= 16:
            assert np.array_equal(d, seq)


@pytest.mark.parametrize("M,N,K", [(2560, 2560, 256), (2304, 2432, 130), (1664, 1664, 512)])
def test_unit_ranges_that_straddle_tiles(cuda, lib, oracle, M, N, K):
    """More tiles than resident blocks but a partly empty last wave: blocks own equal ranges of (tile, K-tile)
    units and keep their two partial tiles in per-block workspace slots."""
    a, b, c = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1), oracle.fill_uniform((M, N), 2, 2)
    for cc in (None, c):
        d = _run(cuda, lib, a, b, cc, 6, split_k=0)
        assert oracle.rel_frobenius(d, oracle.sgemm_f64(a, b, cc)) <= TOL_FRO
        assert np.array_equal(d, _run(cuda, lib, a, b, cc, 6, split_k=0))    # counters are back at zero, same order
        assert np.array_equal(d, _run(cuda, lib, a, b, cc, 4, split_k=0))    # the default picks the same kernel here
        assert oracle.rel_frobenius(d, oracle.sgemm_f32(a, b, cc).astype(np.float64)) <= 3 * TOL_FRO


def test_default_dispatch(cuda, lib, oracle):
    # the second group exercises the launcher's choices: grouped shapes with a split across blocks, tails in M, N
    # and K, short K, a single tile row / column, more than two waves of tiles
    for M, N, K in SHAPES + [(100, 3000, 5000), (1000, 130, 700), (2000, 2000, 40), (64, 64, 10000), (65, 4000, 129),
                             (4000, 65, 1000), (3000, 3000, 24)]:
        a, b = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1)
        assert oracle.rel_frobenius(_run(cuda, lib, a, b), oracle.sgemm_f64(a, b)) <= TOL_FRO


def test_against_reference_kernel_outputs(cuda, lib, oracle, golden):
    a, b = oracle.fill_uniform((64, 64), 2, 0), oracle.fill_uniform((64, 64), 2, 1)
    for variant in (1, 2, 3, 4):
        assert np.array_equal(_run(cuda, lib, a, b, variant=variant, split_k=1), golden["sgemm_64x64x64"])
    a, b, c = oracle.fill_uniform((128, 256), 2, 0), oracle.fill_uniform((256, 64), 2, 1), oracle.fill_uniform((128, 64), 2, 2)
    for variant in (1, 2, 3, 4):
        assert np.array_equal(_run(cuda, lib, a, b, c, variant=variant, split_k=1), golden["sgemm_128x64x256_c"])
        assert np.array_equal(_run(cuda, lib, a, b, c, variant=variant, split_k=1, d_is_c=True), golden["sgemm_128x64x256_c"])   # D may alias C


def test_baseline_shape(cuda, lib, oracle, ko):
    """C3: M=N=K=1024, A and B ~ U(-1,1) seed 2, C overwritten (alpha=1, beta=0)."""
    a, b = ko.fill_uniform((1024, 1024), 2, 0), ko.fill_uniform((1024, 1024), 2, 1)
    d = _run(cuda, lib, a, b)
    assert oracle.rel_frobenius(d, oracle.sgemm_f64(a, b)) <= TOL_FRO
    assert np.array_equal(_run(cuda, lib, a, b, variant=4, split_k=1), oracle.sgemm_f32(a, b))
    # linearity: (2A)B == 2(AB) exactly in binary floating point, whatever the K split
    assert np.array_equal(_run(cuda, lib, 2 * a, b), 2 * d)


def test_k_zero_and_aliasing_rules(cuda, lib):
    s = cuda.cuda.current_stream().cuda_stream
    d = cuda.full((4, 4), 7.0, device="cuda")
    c = cuda.ones((4, 4), device="cuda")
    assert lib.ko_sgemm_f32(4, 4, 0, None, None, c.data_ptr(), d.data_ptr(), s) == 0
    cuda.cuda.synchronize()
    assert (d == 1).all()          # empty sum + C
    a = cuda.ones((4, 4), device="cuda")
    assert lib.ko_sgemm_f32(4, 4, 4, a.data_ptr(), a.data_ptr(), None, a.data_ptr(), s) == 1   # D aliases A
