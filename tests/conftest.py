import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def cuda():
    """torch with a CUDA device; GPU tests request this fixture."""
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="session")
def built_library():
    """The in-tree CUDA library, built if this checkout has not built it yet."""
    from qwencore_b200 import build

    return build.build()
