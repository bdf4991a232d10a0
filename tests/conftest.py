import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    # Files named test_zz_* run last whatever the order on the command line.
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)).startswith("test_zz_"),))
