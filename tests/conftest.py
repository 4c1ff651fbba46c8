"""Shared fixtures.  GPU tests are marked `gpu`; everything else must pass on a CPU-only box."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "cutlass-kernels_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import CfkOracle
    return CfkOracle()


@pytest.fixture(scope="session")
def lib():
    import cfk_b200
    return cfk_b200.load()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a gpu-marked test was collected on a box without a CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
