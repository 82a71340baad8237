import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "flaggems-sglang_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def built_lib():
    """The shared object must exist; CPU tests only load it and look at symbols."""
    from flaggems_sglang_b200 import _build, _lib
    if _build.needs_build():
        _build.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def pytest_sessionfinish(session, exitstatus):
    """With B200MOE_PARITY_REPORT=<file>: one line per floating-point comparison of the run
    (fraction within the strict bound, worst element, bit-equal fraction)."""
    path = os.environ.get("B200MOE_PARITY_REPORT")
    if not path:
        return
    import json
    from parity import RESULTS
    with open(path, "a") as f:
        for r in RESULTS:
            f.write(json.dumps(r) + "\n")
