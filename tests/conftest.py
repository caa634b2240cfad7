import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def built_library():
    """The CUDA library is built in-tree; (re)build it when missing or stale and a compiler is
    at hand, so that a fresh checkout can run the suite directly."""
    import shutil
    from executorch_b200 import build as b
    if b.needs_build() and (shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc")):
        b.build()
    return b.LIB


@pytest.fixture(scope="session")
def restatement():
    import oracle
    return oracle.Restatement()


@pytest.fixture(scope="session")
def golden():
    import json
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "sampler_golden.npz")
    z = np.load(path)
    meta = json.loads(bytes(z["meta"]).decode())
    return z, meta


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
