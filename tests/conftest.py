"""Shared pytest configuration: marker registration and repo-root imports."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Loader for the vectors in tests/golden/ produced by make_golden.py from the reference."""
    import numpy as np

    def load(name):
        path = os.path.join(ROOT, "tests", "golden", f"{name}.npz")
        with np.load(path) as data:
            return {key: data[key] for key in data.files}
    return load
