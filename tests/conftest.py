import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_package():
    """Import the in-tree package (its directory name has a hyphen) as gopherence_b200."""
    if "gopherence_b200" in sys.modules:
        return sys.modules["gopherence_b200"]
    pkg_dir = os.path.join(ROOT, "go-pherence_b200")
    spec = importlib.util.spec_from_file_location(
        "gopherence_b200", os.path.join(pkg_dir, "__init__.py"),
        submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["gopherence_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def gpu(pkg):
    """The runtime bound to cuda:0; fails loudly if the CUDA library is missing."""
    rt = pkg.runtime
    rt.init(0)
    return rt
