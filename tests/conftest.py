import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # files named test_zz_* run last, whatever the order of collection
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)).startswith("test_zz_"),))


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session into a temporary folder."""
    from tiny_configs import TINY, write_tiny
    root = tmp_path_factory.mktemp("models")
    dirs = {name: write_tiny(name, str(root / name)) for name in TINY}
    # queries and keys x8: scores spread over several units instead of hundredths, so attention is far
    # from uniform and a wrong or missing key moves the logits
    dirs["Bsharp"] = write_tiny("B", str(root / "Bsharp"), sharpen=8.0)
    return dirs
