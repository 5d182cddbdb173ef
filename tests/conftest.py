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


def pytest_terminal_summary(terminalreporter):
    """bf16 comparisons are allowed one bf16 grid step on top of 1e-2 * RMS: say how often that was needed."""
    import sys

    module = sys.modules.get("test_gpu_kernels")
    used = getattr(module, "GRID_TERM_USE", None)
    if not used:
        return
    needed = sum(count for _, count, _ in used)
    total = sum(size for _, _, size in used)
    terminalreporter.write_line(f"bf16 grid term: needed by {needed} of {total} compared elements "
                                f"({len([u for u in used if u[1]])} of {len(used)} comparisons)")
    for what, count, size in sorted(used, key=lambda u: -u[1] / max(u[2], 1))[:5]:
        if count:
            terminalreporter.write_line(f"  {what}: {count} of {size}")
