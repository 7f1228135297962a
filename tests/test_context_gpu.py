"""GPU: the explicit context (ko_context_create / ko_context_destroy and the *_ctx entry points) that owns the SGEMM's
split-K scratch lanes and the tensor-core GEMM's cache of TMA descriptors; scratch that never moves once handed out
(a captured graph stays valid when a later, larger eager call on the same stream needs more); and the status poll
seeing a kernel on a non-blocking side stream."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _stats(lib, ctx):
    vals = [C.c_size_t() for _ in range(4)]
    assert lib.ko_context_stats(ctx, *[C.byref(v) for v in vals]) == 0
    return tuple(v.value for v in vals)  # device bytes, maps, hits, misses


def test_context_owns_scratch_and_descriptors(cuda, lib, oracle):
    s = cuda.cuda.current_stream().cuda_stream
    ctx = C.c_void_p()
    assert lib.ko_context_create(-1, C.byref(ctx)) == 0 and ctx.value
    assert _stats(lib, ctx) == (0, 0, 0, 0)  # creating a context allocates nothing
    # SGEMM 512^3 splits K across blocks: the first call allocates this stream's lane, the second reuses it
    a, b = oracle.fill_uniform((512, 512), 2, 0), oracle.fill_uniform((512, 512), 2, 1)
    ad, bd = cuda.from_numpy(a).cuda(), cuda.from_numpy(b).cuda()
    d_ctx, d_def = cuda.empty((512, 512), device="cuda"), cuda.empty((512, 512), device="cuda")
    assert lib.ko_sgemm_f32_ctx(ctx, 512, 512, 512, ad.data_ptr(), bd.data_ptr(), None, d_ctx.data_ptr(), s) == 0, lib.ko_last_error_string()
    held = _stats(lib, ctx)[0]
    assert held > 0
    assert lib.ko_sgemm_f32_ctx(ctx, 512, 512, 512, ad.data_ptr(), bd.data_ptr(), None, d_ctx.data_ptr(), s) == 0
    assert _stats(lib, ctx)[0] == held
    assert lib.ko_sgemm_f32(512, 512, 512, ad.data_ptr(), bd.data_ptr(), None, d_def.data_ptr(), s) == 0
    cuda.cuda.synchronize()
    assert cuda.equal(d_ctx, d_def)
    assert oracle.rel_frobenius(d_ctx.cpu().numpy(), oracle.sgemm_f64(a, b)) <= 1e-6
    # tensor-core GEMM: three descriptors encoded once, then served from the cache
    a16 = (cuda.rand((256, 128), device="cuda") * 2 - 1).bfloat16()
    b16 = (cuda.rand((192, 128), device="cuda") * 2 - 1).bfloat16()
    d1, d2 = cuda.empty((256, 192), device="cuda"), cuda.empty((256, 192), device="cuda")
    for _ in range(3):
        assert lib.ko_gemm_tc_ctx(ctx, 1, 0, 0, 256, 192, 128, a16.data_ptr(), b16.data_ptr(), None, d1.data_ptr(), s) == 0, lib.ko_last_error_string()
    _, maps, hits, misses = _stats(lib, ctx)
    assert (maps, misses, hits) == (3, 3, 6)
    assert lib.ko_gemm_tc(1, 0, 0, 256, 192, 128, a16.data_ptr(), b16.data_ptr(), None, d2.data_ptr(), s) == 0
    cuda.cuda.synchronize()
    assert cuda.equal(d1, d2)
    want = a16.double().cpu().numpy() @ b16.double().cpu().numpy().T
    assert oracle.rel_frobenius(d1.cpu().numpy(), want) <= 1e-3
    # another buffer at the same shape is a new key
    d3 = cuda.empty((256, 192), device="cuda")
    assert lib.ko_gemm_tc_ctx(ctx, 1, 0, 0, 256, 192, 128, a16.data_ptr(), b16.data_ptr(), None, d3.data_ptr(), s) == 0
    assert _stats(lib, ctx)[1] == 4
    free_before, _ = cuda.cuda.mem_get_info()
    assert lib.ko_context_destroy(ctx) == 0
    free_after, _ = cuda.cuda.mem_get_info()
    assert free_after - free_before >= held  # the lane went back to the driver
    assert lib.ko_context_destroy(None) == 0
    assert lib.ko_context_create(-1, None) == 1


def test_a_captured_sgemm_survives_a_larger_eager_call_on_its_stream(cuda, lib, oracle):
    """The scratch a captured launch points at is never freed or moved while its context lives: capture a small split
    SGEMM, then run eagerly, on the same stream, a call whose explicit split needs a lane several times the first
    one's size (the context adds a block and keeps the old one), replay the graph and compare bits."""
    a, b = oracle.fill_uniform((256, 1024), 2, 0), oracle.fill_uniform((1024, 256), 2, 1)
    ad, bd = cuda.from_numpy(a).cuda(), cuda.from_numpy(b).cuda()
    d = cuda.empty((256, 256), device="cuda")
    side = cuda.cuda.Stream()
    with cuda.cuda.stream(side):
        s = side.cuda_stream

        def small():
            assert lib.ko_sgemm_f32(256, 256, 1024, ad.data_ptr(), bd.data_ptr(), None, d.data_ptr(), s) == 0, lib.ko_last_error_string()

        small()  # warm-up: allocates this stream's lane in the device's default context
        side.synchronize()
        eager = d.clone()
        held = _stats(lib, None)[0]
        assert held > 0
        graph = cuda.cuda.CUDAGraph()
        with cuda.cuda.graph(graph, stream=side):
            small()
        # 48 x 48 tiles of 128 x 128 in 2 K-slices: 4608 partial tiles, far beyond the lane's first size
        big_n = 128 * 48
        ab = cuda.rand((big_n, 64), device="cuda")
        bb = cuda.rand((64, big_n), device="cuda")
        db = cuda.empty((big_n, big_n), device="cuda")
        assert lib.ko_sgemm_f32_tuned(big_n, big_n, 64, ab.data_ptr(), bb.data_ptr(), None, db.data_ptr(), 6, 2, s) == 0, lib.ko_last_error_string()
        side.synchronize()
        assert _stats(lib, None)[0] >= held + 4608 * 128 * 128 * 4, "the larger split needed a new block"
        assert cuda.allclose(db, ab @ bb, rtol=1e-5, atol=1e-5)
        for _ in range(2):
            d.fill_(float("nan"))
            graph.replay()
            side.synchronize()
            assert cuda.equal(d, eager)
    cuda.cuda.synchronize()
    assert oracle.rel_frobenius(d.cpu().numpy(), oracle.sgemm_f64(a, b)) <= 1e-6


def test_growth_is_refused_inside_a_capture_and_nothing_breaks(cuda, lib, oracle):
    """A stream that has no lane yet cannot get one while it is being captured: the call reports it and launches nothing;
    the same call made eagerly first, then captured, works."""
    ctx = C.c_void_p()
    assert lib.ko_context_create(-1, C.byref(ctx)) == 0
    ad = cuda.rand((256, 1024), device="cuda")
    bd = cuda.rand((1024, 256), device="cuda")
    d = cuda.full((256, 256), 7.0, device="cuda")
    side = cuda.cuda.Stream()
    refused = []
    with cuda.cuda.stream(side):
        s = side.cuda_stream
        graph = cuda.cuda.CUDAGraph()
        with cuda.cuda.graph(graph, stream=side):
            bd.add_(0.0)  # something to capture besides the refused call
            refused.append(lib.ko_sgemm_f32_ctx(ctx, 256, 256, 1024, ad.data_ptr(), bd.data_ptr(), None, d.data_ptr(), s))
            refused.append(lib.ko_last_error_string())
        graph.replay()
        side.synchronize()
    assert refused[0] == 1 and b"capture" in refused[1]
    assert bool((d == 7.0).all())
    assert _stats(lib, ctx)[0] == 0
    assert lib.ko_context_destroy(ctx) == 0


def test_status_poll_sees_a_kernel_on_a_non_blocking_stream(cuda, lib):
    """ko_poll_device_status waits for every stream of the device: a wait that runs out in a kernel on a non-blocking
    side stream is reported by a poll made right after the launch."""
    assert lib.ko_poll_device_status() == 0
    side = cuda.cuda.Stream()  # torch side streams are created non-blocking
    assert lib.ko_selftest_bounded_wait(1 << 20, side.cuda_stream) == 0   # about a millisecond of polling
    assert lib.ko_poll_device_status() == 5
    assert lib.ko_poll_device_status() == 0
