import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def bridge():
    from browsergrad_b200 import CudaBridge
    b = CudaBridge(0)
    yield b
    b.close()


def pytest_sessionfinish(session, exitstatus):
    """When BG_PARITY_REPORT names a file, leaves the measured error of every parity comparison of this run there
    as JSON."""
    import json
    from tests import util
    path = os.environ.get("BG_PARITY_REPORT")
    if not path or not util.ERROR_LOG:
        return
    import numpy as np
    with open(path, "w") as fh:
        json.dump({"numpy": np.__version__, "floor_bits": {"pointwise": util.FLOOR_BITS_POINTWISE, "contraction": util.FLOOR_BITS_CONTRACTION},
                   "comparisons": util.ERROR_LOG}, fh, indent=1)
