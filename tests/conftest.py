import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")
if GOLDEN not in sys.path:
    sys.path.insert(0, GOLDEN)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    class _Store:
        def __init__(self):
            self._files = {}

        def __call__(self, fname):
            if fname not in self._files:
                self._files[fname] = dict(np.load(os.path.join(GOLDEN, fname), allow_pickle=False))
            return self._files[fname]

    return _Store()
