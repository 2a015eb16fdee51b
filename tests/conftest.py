import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return ROOT / "tests" / "golden"


@pytest.fixture(scope="session")
def cuda_ctx():
    """One context per test process, as in the reference (one device, one queue)."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ferrotensor_b200.engine import CudaContext
    ctx = CudaContext(0)
    yield ctx
    ctx.synchronize()
