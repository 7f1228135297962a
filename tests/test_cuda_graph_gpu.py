"""GPU: the launchers are safe to capture into a CUDA graph once their per-device set-up has run (no allocation, no
synchronisation and no host-side state change happens in a warmed call), and a replayed graph gives the bits of the
eager calls.  Kernels are launched with programmatic stream serialization; inside a capture that becomes a
programmatic dependency edge of the graph."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_operator_sequence_replays_from_a_cuda_graph(cuda, lib, ko, oracle):
    dev = "cuda"
    x = cuda.from_numpy(oracle.fill_normal((4096, 128), 0, 0, 0.0, 2.0)).to(dev)
    xl = cuda.from_numpy(oracle.fill_normal((2048, 768), 1, 0)).to(dev)
    g = cuda.from_numpy(oracle.fill_uniform((768,), 1, 1, 0.5, 1.5)).to(dev)
    b = cuda.from_numpy(oracle.fill_normal((768,), 1, 2, 0.0, 0.1)).to(dev)
    a32, b32 = cuda.rand((512, 512), device=dev) * 2 - 1, cuda.rand((512, 512), device=dev) * 2 - 1
    a16 = (cuda.rand((512, 256), device=dev) * 2 - 1).bfloat16()
    b16 = (cuda.rand((384, 256), device=dev) * 2 - 1).bfloat16()
    y, yl = cuda.empty_like(x), cuda.empty_like(xl)
    d32 = cuda.empty((512, 512), device=dev)
    dtc = cuda.empty((512, 384), device=dev)

    def sequence():
        ko.softmax(x, out=y)
        ko.layernorm(xl, 1e-12, g, b, out=yl)
        ko.sgemm(a32, b32, out=d32)          # 512^3: K split inside and across blocks (scratch from the warm-up call)
        ko.gemm_tc(a16, b16, out=dtc)

    side = cuda.cuda.Stream()
    with cuda.cuda.stream(side):
        sequence()                           # warm-up on the capture stream: per-(device, stream) set-up happens here
        side.synchronize()
        eager = [t.clone() for t in (y, yl, d32, dtc)]
        graph = cuda.cuda.CUDAGraph()
        for t in (y, yl, d32, dtc):
            t.fill_(float("nan"))
        with cuda.cuda.graph(graph, stream=side):
            sequence()
    for _ in range(3):
        for t in (y, yl, d32, dtc):
            t.fill_(float("nan"))
        graph.replay()
        cuda.cuda.synchronize()
        for got, want in zip((y, yl, d32, dtc), eager):
            assert cuda.equal(got, want)
    assert lib.ko_poll_device_status() == 0
    assert oracle.max_abs_err(y.cpu().numpy(), oracle.softmax_f64(x.cpu().numpy())) <= 1e-6


def test_sliced_gemm_in_a_graph_and_capture_without_a_scratch_lane(cuda, lib, ko, oracle):
    """A GEMM of few tiles and long K is cut into K slices, which need the stream's scratch lane: warmed, it replays
    from a graph bit for bit; captured on a stream that has no lane yet it may not allocate and runs unsliced."""
    dev = "cuda"
    a = (cuda.rand((128, 8192), device=dev) * 2 - 1).bfloat16()
    b = (cuda.rand((128, 8192), device=dev) * 2 - 1).bfloat16()
    d = cuda.empty((128, 128), device=dev)
    want = a.double() @ b.double().t()
    side = cuda.cuda.Stream()
    with cuda.cuda.stream(side):
        ko.gemm_tc(a, b, out=d)              # allocates this stream's lane
        side.synchronize()
        eager = d.clone()
        graph = cuda.cuda.CUDAGraph()
        with cuda.cuda.graph(graph, stream=side):
            ko.gemm_tc(a, b, out=d)
    d.fill_(float("nan"))
    graph.replay()
    cuda.cuda.synchronize()
    assert cuda.equal(d, eager)
    assert float((eager.double() - want).norm() / want.norm()) <= 1e-5
    fresh = cuda.cuda.Stream()
    with cuda.cuda.stream(fresh):
        graph2 = cuda.cuda.CUDAGraph()
        with cuda.cuda.graph(graph2, stream=fresh):
            ko.gemm_tc(a, b, out=d)
    d.fill_(float("nan"))
    graph2.replay()
    cuda.cuda.synchronize()
    assert float((d.double() - want).norm() / want.norm()) <= 1e-5
    assert lib.ko_poll_device_status() == 0
