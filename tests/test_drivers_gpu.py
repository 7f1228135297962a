"""GPU: the stand-alone C++ drivers (kernel_optimization_b200/nn_operators/*/main.cu, built by CMake into
kernel_optimization_b200/bin/) run, time their operator and pass their built-in checks."""
import json

import numpy as np
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(name, *args):
    exe = os.path.join(ROOT, "kernel_optimization_b200", "bin", name)
    assert os.path.exists(exe), f"{exe} is missing: build with cmake (KO_BUILD_DRIVERS=ON)"
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.join(ROOT, "kernel_optimization_b200", "lib") + ":" + env.get("LD_LIBRARY_PATH", "")
    proc = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "Passed." in proc.stdout
    return json.loads(proc.stdout.strip().splitlines()[-1])


def test_softmax_driver():
    assert _run("softmax_driver", "--iters", 10)["gbs"] > 1000
    _run("softmax_driver", "--rows", 4096, "--cols", 512, "--causal", "--iters", 5, "--sets", 2)


def test_layernorm_driver():
    assert _run("layernorm_driver", "--iters", 10)["gbs"] > 1000
    _run("layernorm_driver", "--rows", 2048, "--cols", 4096, "--bf16", "--iters", 5, "--sets", 2)
    _run("layernorm_driver", "--rows", 1000, "--cols", 1024, "--ddof", 1, "--iters", 3, "--sets", 1)


def test_gemm_driver():
    assert _run("gemm_driver", "--iters", 5)["tflops"] > 5
    _run("gemm_driver", "--bf16", "--m", 1024, "--n", 1024, "--k", 512, "--iters", 3)
    _run("gemm_driver", "--f16", "--m", 1000, "--n", 520, "--k", 200, "--iters", 3)


@pytest.mark.parametrize("chunks", [0, 1, 3, 64])
def test_host_tensor_pipeline_matches_the_device_call(cuda, lib, ko, oracle, chunks):
    """ko_softmax_f32_host / ko_layernorm_f32_host: chunked copy-in / kernel / copy-out over three streams gives the
    bits of the plain device call (rows are independent), for any chunk count, also more chunks than rows."""
    for rows, cols in ((1000, 128), (37, 768), (5, 1024)):
        x = oracle.fill_normal((rows, cols), 9, 0, 0.0, 2.0)
        g, b = oracle.fill_uniform((cols,), 9, 1, 0.5, 1.5), oracle.fill_normal((cols,), 9, 2, 0.0, 0.1)
        gd, bd = cuda.from_numpy(g).cuda(), cuda.from_numpy(b).cuda()
        t_in, t_out = ko.Tensor(x.nbytes), ko.Tensor(x.nbytes)
        t_in.host_ref(np.float32)[:] = x.reshape(-1)
        xd = cuda.from_numpy(x).cuda()
        for op in ("softmax", "layernorm"):
            t_out.host_ref(np.float32)[:] = np.nan
            if op == "softmax":
                ko.softmax_host(t_in, t_out, rows, cols, chunks)
                want = ko.softmax(xd).cpu().numpy()
            else:
                ko.layernorm_host(t_in, t_out, rows, cols, 1e-5, gd, bd, 0, chunks)
                want = ko.layernorm(xd, 1e-5, gd, bd).cpu().numpy()
            cuda.cuda.current_stream().synchronize()   # the call is ordered on the current stream
            assert np.array_equal(t_out.host_ref(np.float32).reshape(rows, cols), want)
    bad = ko.Tensor(16)
    assert lib.ko_softmax_f32_host(bad._h, bad._h, 100, 100, 0, None) == 3   # larger than the tensors
