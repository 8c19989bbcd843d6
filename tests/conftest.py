import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    """Reference outputs recorded by tests/golden/make_golden.py."""
    path = os.path.join(ROOT, "tests", "golden", "reference_vectors.npz")
    data = np.load(path)
    S = data["q"].shape[2]

    class G:
        q, k, v = data["q"], data["k"], data["v"]

        @staticmethod
        def mask(kind):
            return np.unpackbits(data[f"mask_{kind}"], axis=-1)[..., :S].astype(bool)

        @staticmethod
        def get(key):
            return data[key]

        cases = [("random_128x32", "random", 128, 32), ("random_32x32", "random", 32, 32),
                 ("random_32x128", "random", 32, 128), ("document_64x64", "document", 64, 64),
                 ("document_128x32", "document", 128, 32)]

    return G


@pytest.fixture(scope="session")
def native_lib():
    """Builds (if stale) and loads the C-ABI library."""
    from sparseattention_b200 import build, _native
    build.build()
    return _native.load_library()
