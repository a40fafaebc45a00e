import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    # A fresh checkout has no built libraries (they are not tracked): build them once, as
    # `__graft_entry__.build()` does, so that the suite can be run directly.
    if not os.path.exists(os.path.join(ROOT, "pegaflow_b200", "libpegaflow_b200.so")):
        import __graft_entry__

        __graft_entry__.build()


@pytest.fixture(scope="session")
def kats():
    import json

    with open(os.path.join(GOLDEN, "reference_kats.json")) as f:
        return json.load(f)
