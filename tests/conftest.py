import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def cuda():
    """torch with a usable CUDA device and the native library loaded; GPU tests never fall back."""
    import torch
    assert torch.cuda.is_available(), "GPU test selected but no CUDA device is visible"
    import clblast_b200
    clblast_b200.lib()  # raises when the library is missing
    torch.cuda.init()
    torch.zeros(1, device="cuda")
    return torch
