"""Shared fixtures.  ``-m gpu`` tests need a B200; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import ko_oracle

    return ko_oracle


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_kernels_b200.npz"))


@pytest.fixture(scope="session")
def ko():
    import kernel_optimization_b200

    return kernel_optimization_b200


@pytest.fixture(scope="session")
def lib(ko):
    return ko.native.lib()


@pytest.fixture(scope="session")
def cuda():
    """torch handle for device memory; GPU tests fail (not skip) when CUDA is absent."""
    import torch

    assert torch.cuda.is_available(), "a CUDA device is required for -m gpu tests"
    torch.cuda.set_device(0)
    return torch
