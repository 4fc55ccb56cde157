import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for path in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests", "golden"),
             os.path.join(ROOT, "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device with compute capability 10.x")


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran on a machine without CUDA")
    if torch.cuda.get_device_capability()[0] != 10:
        pytest.fail("the kernels need compute capability 10.x")
    import nvfp4_attn_kernel_b200._lib as lib

    lib.load()  # raises loudly when the extension is missing
    return torch.device("cuda", torch.cuda.current_device())
