"""pytest configuration: the ``gpu`` marker and shared helpers."""

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with `-m gpu` on a B200")


def load_golden(name):
    return torch.load(GOLDEN / name, weights_only=False)


@pytest.fixture(scope="session")
def cuda_dev():
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device; select CPU tests with -m 'not gpu'")
    return torch.device("cuda", 0)
