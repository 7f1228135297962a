"""CPU: a translation unit that uses every helper name of the reference's common.h / functors.h / layernorm.h
(and the operator templates with the reference drivers' launch syntax) compiles for sm_100a against this
repository's headers.  nvcc cross-compiles without a GPU; nothing is run."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_helper_names_compile(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is not installed")
    src = os.path.join(ROOT, "tests", "compile", "reference_helper_names.cu")
    cmd = [nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "kernel_optimization_b200"),
           "-I", os.path.join(ROOT, "include"), "-c", src, "-o", str(tmp_path / "names.o")]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert proc.returncode == 0, proc.stdout[-6000:]
