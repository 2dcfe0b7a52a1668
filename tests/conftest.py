import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden():
    import json

    import numpy as np

    here = os.path.join(ROOT, "tests", "golden")
    arrays = np.load(os.path.join(here, "mxfp8_golden.npz"))
    with open(os.path.join(here, "mxfp8_golden.json")) as f:
        manifest = json.load(f)
    return arrays, manifest


@pytest.fixture(scope="session")
def native_lib():
    """Build (if stale) and load librtxb; building needs only nvcc, not a GPU."""
    from rtx_b200 import _native, build

    build.build()
    return _native.load()
