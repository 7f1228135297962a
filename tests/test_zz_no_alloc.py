"""GPU: ko_sgemm_f32_no_alloc, the SGEMM entry point for hosts that must not allocate device memory.

Its split-K scratch is a fixed array inside the library instead of a cudaMalloc'ed buffer, so a
process whose own allocator owns the GPU (or one that cannot afford an allocation's synchronisation)
can still run the split kernel.  The file name keeps this test last in collection order: if it
fails, a run that stops at the first failure has already covered everything else.

The test calls the entry point through the C ABI twice in a row -- different shapes, so the second
call starts from the first call's left-over scratch -- and compares each result with the regular
entry point (same kernel, same K split: the outputs must agree bit for bit, far inside the 1e-6
relative Frobenius tolerance of the SGEMM tests) and with the float64 oracle.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_FRO = 1e-6


def _gemm(cuda, lib, entry, a, b, c, split_k):
    M, K = a.shape
    N = b.shape[1]
    s = cuda.cuda.current_stream().cuda_stream
    ad, bd = cuda.from_numpy(a).cuda(), cuda.from_numpy(b).cuda()
    cd = None if c is None else cuda.from_numpy(c).cuda()
    dd = cuda.full((M, N), float("nan"), dtype=cuda.float32, device="cuda")
    cp = None if cd is None else cd.data_ptr()
    if entry == "no_alloc":
        rc = lib.ko_sgemm_f32_no_alloc(M, N, K, ad.data_ptr(), bd.data_ptr(), cp, dd.data_ptr(), split_k, s)
    else:
        rc = lib.ko_sgemm_f32_tuned(M, N, K, ad.data_ptr(), bd.data_ptr(), cp, dd.data_ptr(), 4, split_k, s)
    cuda.cuda.synchronize()
    assert rc == 0, lib.ko_last_error_string()
    return dd.cpu().numpy()


def test_two_calls_in_a_row_match_the_allocating_entry_point(cuda, lib, oracle):
    cases = [((512, 384, 1024), 4, True), ((300, 200, 1000), 2, False), ((1024, 1024, 1024), 2, False)]
    for (M, N, K), split_k, with_c in cases:
        a, b = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1)
        c = oracle.fill_uniform((M, N), 2, 2) if with_c else None
        got = _gemm(cuda, lib, "no_alloc", a, b, c, split_k)
        want = _gemm(cuda, lib, "regular", a, b, c, split_k)
        assert oracle.rel_frobenius(got, want.astype(np.float64)) <= TOL_FRO
        assert np.array_equal(got, want), "same kernel and same K split: identical bits"
        assert oracle.rel_frobenius(got, oracle.sgemm_f64(a, b, c)) <= TOL_FRO
        # and once more on the scratch the call above just used
        assert np.array_equal(_gemm(cuda, lib, "no_alloc", a, b, c, split_k), want)


def test_defaults_and_the_size_limit(cuda, lib, oracle):
    a, b = oracle.fill_uniform((256, 512), 2, 0), oracle.fill_uniform((512, 256), 2, 1)
    want = oracle.sgemm_f64(a, b)
    assert oracle.rel_frobenius(_gemm(cuda, lib, "no_alloc", a, b, None, 0), want) <= TOL_FRO   # chosen split
    assert np.array_equal(_gemm(cuda, lib, "no_alloc", a, b, None, 1), oracle.sgemm_f32(a, b))  # no split, no scratch
    # 1024 x 1024 outputs are 64 tiles: 4 slices would need 4 Mi scratch floats, twice what the library holds
    s = cuda.cuda.current_stream().cuda_stream
    big = cuda.zeros((1024, 1024), dtype=cuda.float32, device="cuda")
    out = cuda.full((1024, 1024), 7.0, dtype=cuda.float32, device="cuda")
    rc = lib.ko_sgemm_f32_no_alloc(1024, 1024, 1024, big.data_ptr(), big.data_ptr(), None, out.data_ptr(), 4, s)
    cuda.cuda.synchronize()
    assert rc == 3 and b"scratch" in lib.ko_last_error_string()
    assert bool((out == 7.0).all()), "a refused call must not launch anything"


def test_the_limit_is_128_partial_tiles(cuda, lib):
    """tiles * split_k <= 128: 64 output tiles in 2 slices are accepted, 65 tiles in 2 slices are refused before
    anything is launched (the limit the header states)."""
    s = cuda.cuda.current_stream().cuda_stream
    K = 256
    for (M, N), accepted in (((1024, 1024), True), ((1024 + 1, 1024), False), ((128 * 5, 128 * 13), False)):
        a = cuda.zeros((M, K), dtype=cuda.float32, device="cuda")
        b = cuda.zeros((K, N), dtype=cuda.float32, device="cuda")
        out = cuda.full((M, N), 7.0, dtype=cuda.float32, device="cuda")
        rc = lib.ko_sgemm_f32_no_alloc(M, N, K, a.data_ptr(), b.data_ptr(), None, out.data_ptr(), 2, s)
        cuda.cuda.synchronize()
        if accepted:
            assert rc == 0, lib.ko_last_error_string()
            assert bool((out == 0.0).all())
        else:
            assert rc == 3 and b"scratch" in lib.ko_last_error_string()
            assert bool((out == 7.0).all())


def test_a_warmed_call_leaves_device_memory_untouched(cuda, lib, oracle):
    """What the entry point exists for: once its one-time set-up has run, a call allocates nothing -- the free-memory
    figure the driver reports is the same before and after, and so is the caching allocator's reservation."""
    M, N, K = 512, 512, 2048
    a, b = oracle.fill_uniform((M, K), 2, 0), oracle.fill_uniform((K, N), 2, 1)
    ad, bd = cuda.from_numpy(a).cuda(), cuda.from_numpy(b).cuda()
    dd = cuda.empty((M, N), dtype=cuda.float32, device="cuda")
    s = cuda.cuda.current_stream().cuda_stream

    def call():
        rc = lib.ko_sgemm_f32_no_alloc(M, N, K, ad.data_ptr(), bd.data_ptr(), None, dd.data_ptr(), 4, s)
        assert rc == 0, lib.ko_last_error_string()

    call()  # set-up (symbol address, shared-memory limit) happens here at the latest
    cuda.cuda.synchronize()
    free_before, _total = cuda.cuda.mem_get_info()
    reserved_before = cuda.cuda.memory_reserved()
    for _ in range(3):
        call()
    cuda.cuda.synchronize()
    free_after, _total = cuda.cuda.mem_get_info()
    assert free_after == free_before, f"device memory changed by {free_before - free_after} bytes across warmed calls"
    assert cuda.cuda.memory_reserved() == reserved_before
    assert oracle.rel_frobenius(dd.cpu().numpy(), oracle.sgemm_f64(a, b)) <= TOL_FRO
