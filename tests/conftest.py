import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle

    return Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU GEMM, where oracle/_ref was built (it travels to the GPU box as a prebuilt file)."""
    from oracle.oracle import Ref

    if not Ref.available():
        pytest.skip("oracle/_ref/libsepal_ref.so is not built here")
    return Ref()


@pytest.fixture(scope="session")
def ref_gpu():
    """The reference's own GPU multiplies and cuBLAS call, where oracle/_ref was built (a prebuilt file on the GPU box)."""
    from oracle.oracle import RefGpu

    if not RefGpu.available():
        pytest.skip("oracle/_ref/libsepal_ref_gpu.so is not built here")
    return RefGpu()


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    path = os.path.join(ROOT, "tests", "golden", "golden.npz")
    return np.load(path)


@pytest.fixture(scope="session")
def ctx():
    """One context on cuda:0 for the GPU tests. Fails (does not skip) when the library or the device is missing."""
    import torch

    import sepal_runner_b200 as sb

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    c = sb.Context(0)
    yield c
    c.close()
