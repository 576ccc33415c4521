"""pytest configuration: the `gpu` marker, repo-root imports and shared helpers."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from metal_candle_b200 import _lib

    _lib.init(0)  # raises when the library is missing: GPU tests never pass on a fallback
    return torch.device("cuda", 0)
