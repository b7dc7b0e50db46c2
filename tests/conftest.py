import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a) and the built extension")


def pytest_collection_modifyitems(config, items):
    # keep the file whose name sorts last (the allocation-free entry point) at the very end
    items.sort(key=lambda it: (Path(str(it.fspath)).name.startswith("test_zz"),))
