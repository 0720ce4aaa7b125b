import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu")


@pytest.fixture(scope="session")
def manifest():
    with open(os.path.join(GOLDEN, "manifest.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def fq_cases():
    return np.load(os.path.join(GOLDEN, "fq_cases.npz"))


@pytest.fixture(scope="session")
def linear_cases():
    return np.load(os.path.join(GOLDEN, "linear_cases.npz"))


@pytest.fixture(scope="session")
def tables():
    return np.load(os.path.join(GOLDEN, "tables.npz"))
