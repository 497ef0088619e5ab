import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_golden.npz"))


@pytest.fixture(scope="session")
def built_libs():
    """The sm_100a libraries, built in-tree if missing (nvcc cross-compiles without a GPU)."""
    from goml_b200 import build
    build.build_all()
    return build.LIBS


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def fa_ctx(cuda, built_libs):
    from goml_b200 import fa_forward
    ctx = fa_forward.FACreate()
    yield ctx
    ctx.Destroy()
