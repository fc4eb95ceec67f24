import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_package():
    """The package directory is named 'salt-core_b200' (not an identifier);
    import it by path name and alias it as salt_core_b200."""
    if "salt_core_b200" not in sys.modules:
        sys.modules["salt_core_b200"] = importlib.import_module("salt-core_b200")
    return sys.modules["salt_core_b200"]


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def synth():
    return importlib.import_module("salt-core_b200.synth")


@pytest.fixture(scope="session")
def orc():
    import oracle
    return oracle.Oracle()


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a


def assert_bits_equal(a, b, what=""):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    ne = bits(a) != bits(b)
    if ne.any():
        i = np.argwhere(ne)[0]
        raise AssertionError(f"{what}: {int(ne.sum())} of {ne.size} differ; first at {tuple(i)}: "
                             f"{a[tuple(i)]!r} vs {b[tuple(i)]!r}")
