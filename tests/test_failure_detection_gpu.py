"""GPU: failure detection without a GPU fault.  Every device-side wait in this library is bounded; one
that runs out records a code in a device status word and the kernel returns normally.  The self-test
kernel waits (briefly) on an mbarrier that nothing ever arrives at, so the wait must run out: the host
sees KO_ERR_TIMEOUT once, the words are cleared, and the context stays fully usable."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(cuda, lib, oracle):
    s = cuda.cuda.current_stream().cuda_stream
    assert lib.ko_poll_device_status() == 0
    assert lib.ko_selftest_bounded_wait(2000, s) == 0
    assert lib.ko_poll_device_status() == 5                      # KO_ERR_TIMEOUT
    assert b"bounded device-side wait ran out" in lib.ko_last_error_string()
    assert lib.ko_poll_device_status() == 0                      # reported once, then cleared
    # the device is still healthy: a real operator runs and matches the oracle
    x = oracle.fill_normal((300, 128), 0, 0, 0.0, 2.0)
    xd = cuda.from_numpy(x).cuda()
    yd = cuda.empty_like(xd)
    assert lib.ko_softmax_f32(xd.data_ptr(), yd.data_ptr(), 300, 128, s) == 0
    cuda.cuda.synchronize()
    assert oracle.max_abs_err(yd.cpu().numpy(), oracle.softmax_f64(x)) <= 1e-6
    assert lib.ko_selftest_bounded_wait(0, s) == 1               # argument check


def test_healthy_pipelines_leave_the_status_clean(cuda, lib, oracle):
    from kernel_optimization_b200.native import RowKnobs

    s = cuda.cuda.current_stream().cuda_stream
    x = cuda.from_numpy(oracle.fill_normal((5000, 256), 0, 0, 0.0, 2.0)).cuda()
    y = cuda.empty_like(x)
    assert lib.ko_softmax_f32_tuned(x.data_ptr(), y.data_ptr(), 5000, 256, RowKnobs(tier=4), s) == 0   # TMA ring
    a = cuda.zeros((512, 256), dtype=cuda.bfloat16, device="cuda")
    d = cuda.empty((512, 512), dtype=cuda.float32, device="cuda")
    assert lib.ko_gemm_bf16_f32(512, 512, 256, a.data_ptr(), a.data_ptr(), None, d.data_ptr(), s) == 0  # tcgen05 pipeline
    assert lib.ko_poll_device_status() == 0
