import json
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
    with open(os.path.join(ROOT, "tests", "golden", "gemm_hashes.json")) as f:
        recs = json.load(f)
    return {(r["name"], r["S"]): r for r in recs}


@pytest.fixture(scope="session")
def scalar_vectors():
    with open(os.path.join(ROOT, "tests", "golden", "scalar_vectors.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def conv_golden():
    with open(os.path.join(ROOT, "tests", "golden", "conv_hashes.json")) as f:
        recs = json.load(f)
    return {(r["name"], r["S"]): r for r in recs}
