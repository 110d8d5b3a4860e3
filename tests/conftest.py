import importlib
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PKG_NAME = "hunyuan3d-tools_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def pkg():
    """The product package (its directory name has a hyphen, hence importlib)."""
    return importlib.import_module(PKG_NAME)


@pytest.fixture(scope="session")
def qu(pkg):
    return importlib.import_module(PKG_NAME + ".quantize_utils")


@pytest.fixture(scope="session")
def build_mod(pkg):
    return importlib.import_module(PKG_NAME + ".csrc.build")


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "reference_cpu.npz")
    return dict(np.load(path))


def as_half(arr: np.ndarray) -> torch.Tensor:
    """Golden fp16 tensors are stored as raw 16-bit patterns."""
    return torch.from_numpy(arr.copy()).view(torch.float16)


@pytest.fixture(scope="session")
def tc(build_mod):
    return build_mod.load_tc_gemm()


@pytest.fixture(scope="session")
def sp(build_mod):
    return build_mod.load_sparse_tc()


@pytest.fixture(scope="session")
def ik(build_mod):
    return build_mod.load_int8_kernels()


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test the device-side error word must still be zero: a kernel whose
    bounded wait ran out would have left a code there."""
    yield
    if request.node.get_closest_marker("gpu") and torch.cuda.is_available():
        mod = importlib.import_module(PKG_NAME + ".csrc.build").load_tc_gemm()
        assert mod.device_status() == 0
