import importlib
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    """The package directory name is not a Python identifier, so it is imported by string."""
    return importlib.import_module("ai_framework-dev_b200")


@pytest.fixture(scope="session")
def oracle():
    return importlib.import_module("oracle.dense_oracle")


@pytest.fixture(scope="session")
def lib(pkg):
    from __graft_entry__ import build
    build()
    return pkg.load_library()


@pytest.fixture(scope="session")
def conv_oracle():
    return importlib.import_module("oracle.conv2d_oracle")
