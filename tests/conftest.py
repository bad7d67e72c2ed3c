import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def golden_cases():
    """QVB8 fixtures (outputs of the reference's Python pack decoders)."""
    return sorted(f[:-4] for f in os.listdir(GOLDEN) if f.endswith(".npz") and f.startswith(("qvbd_", "legacy_")))


def golden_qvb8r_cases():
    """QVB8R fixtures (files written and decoded by the reference's container.py + qvb8r_cpu.cpp)."""
    return sorted(f[:-4] for f in os.listdir(GOLDEN) if f.endswith(".npz") and f.startswith("qvb8r_"))


@pytest.fixture(scope="session")
def cuda_lib():
    """The built kernel library on a machine with a GPU; GPU tests fail (not skip) if it is missing."""
    import torch
    assert torch.cuda.is_available(), "GPU test selected without a CUDA device"
    from qvb8_b200 import lib
    return lib.load()
