import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PKG = "axiom-compute_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def load_pkg(sub: str = ""):
    return importlib.import_module(PKG + (("." + sub) if sub else ""))


@pytest.fixture(scope="session")
def axc():
    return load_pkg()


@pytest.fixture(scope="session")
def ffi():
    return load_pkg("_ffi")


@pytest.fixture(scope="session")
def ops():
    return load_pkg("ops")


@pytest.fixture(scope="session")
def synth():
    return load_pkg("synth")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The shared library is built in-tree; build it if this checkout has none yet."""
    load_pkg("build").build_library()


@pytest.fixture(scope="session")
def golden():
    import json
    d = os.path.join(ROOT, "tests", "golden")
    with open(os.path.join(d, "reference_known_answers.json")) as f:
        known = json.load(f)
    with open(os.path.join(d, "lcg_fixture_outputs.json")) as f:
        lcg = json.load(f)
    return {"known": known, "lcg": lcg}
