"""GPU: the stand-alone C++ drivers (kernel_optimization_b200/nn_operators/*/main.cu, built by CMake into
kernel_optimization_b200/bin/) run, time their operator and pass their built-in checks."""
import json
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
