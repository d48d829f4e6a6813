import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built_lib():
    """The native library, built in-tree if needed."""
    from aluminum_b200 import _build
    lib = ROOT / "aluminum_b200" / "lib" / "libal_b200.so"
    tools = ROOT / "aluminum_b200" / "bin" / "test_ops"
    if lib.exists() and tools.exists() and not os.environ.get("AL_REBUILD"):
        return lib  # built artefacts travel with the tree; rebuild only on request
    return _build.build(tools=True)


@pytest.fixture(scope="session")
def bin_dir(built_lib):
    return ROOT / "aluminum_b200" / "bin"
