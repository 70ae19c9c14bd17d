import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _gpu_count() -> int:
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


@pytest.fixture(scope="session")
def gpu_count():
    return _gpu_count()


@pytest.fixture(scope="session")
def ctx():
    """One libreCu context on device 0 for the whole session (the API has a process-global current context)."""
    from librecuda_b200 import api

    c = api.Context(0, api.CU_CTX_SCHED_YIELD)
    yield c
    c.set_current()


@pytest.fixture()
def stream(ctx):
    from librecuda_b200 import api

    ctx.set_current()
    s = api.Stream()
    yield s
    s.destroy()


FIXTURE_CUBIN = ROOT / "tests" / "fixtures" / "_bin" / "fixture_kernels.cubin"
