import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def golden():
    """The committed golden vectors (tests/golden/make_golden.py wrote them from PyTorch's CPU
    kernels, which is what the reference's CPU device runs)."""
    import numpy as np

    with np.load(ROOT / "tests" / "golden" / "hotpath.npz") as data:
        return {key: data[key] for key in data.files}
