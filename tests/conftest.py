import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 and the built libh3b200.so")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the reference's own Python code on seeded inputs (tests/golden/make_golden.py)."""
    return np.load(os.path.join(GOLDEN_DIR, "ref_golden.npz"))


@pytest.fixture(scope="session")
def ref_dispatch():
    with open(os.path.join(GOLDEN_DIR, "ref_dispatch.json")) as fh:
        return json.load(fh)


@pytest.fixture(scope="session")
def gpu():
    """One context for the whole GPU session. Fails loudly (no skip) when the device or the library is missing:
    a GPU test that silently ran nothing would be worse than a red one."""
    from h3metal_b200.gpu import Gpu
    g = Gpu()
    yield g
    g.close()


def rel_fro(got, want) -> float:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-300))
