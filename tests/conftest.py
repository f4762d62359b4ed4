import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "qwen3-27b-thor-runner_b200"), os.path.join(ROOT, "oracle"),
          os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    import oracle_binding
    oracle_binding.load()
    return oracle_binding


@pytest.fixture(scope="session")
def handle():
    """A library handle on cuda:0 with room for the debug prefill path of the test shapes."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import nvfp4
    h = nvfp4.Handle(0, 512 << 20)
    yield h
    h.close()


@pytest.fixture(scope="module")
def big_handle():
    """A handle whose workspace holds the activation copy of 8192 tokens x 17408 columns."""
    import ctypes
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import nvfp4
    need = ctypes.c_size_t()
    assert nvfp4.load().nvfp4_workspace_bytes(8192, 34816, 17408, ctypes.byref(need)) == 0
    h = nvfp4.Handle(0, need.value)
    yield h
    h.close()
