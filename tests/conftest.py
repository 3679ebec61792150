import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    with open(os.path.join(ROOT, "tests", "golden", "matmul_family.json")) as fh:
        data = json.load(fh)

    def arr(bits, shape):
        return np.array(bits, dtype=np.uint32).view(np.float32).reshape(shape)

    for c in data["cases"]:
        c["a"] = arr(c["a_bits"], c["a_shape"])
        c["b"] = arr(c["b_bits"], c["b_shape"])
        c["c"] = arr(c["c_bits"], c["c_shape"])
        c["w"] = arr(c["w_bits"], c["c_shape"])
        c["grad_a"] = arr(c["grad_a_bits"], c["a_shape"])
        c["grad_b"] = arr(c["grad_b_bits"], c["b_shape"])
    return data


@pytest.fixture(scope="session")
def built_library():
    """libfastnn_b200.so, built in-tree if it is not there yet (nvcc cross-compiles)."""
    from fastnn_b200 import build as b
    return b.build()


@pytest.fixture(scope="session")
def gpu(built_library):
    """Initialised device 0 through the C ABI; torch is used for device memory only."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import fastnn_b200 as f
    torch.cuda.set_device(0)
    f.cuda_init(0)
    f.set_policy(0, 0, 0)
    yield f
    f.set_policy(0, 0, 0)
    assert f.device_status() == 0, "a kernel reported a bounded-wait timeout during the session"
