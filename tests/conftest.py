import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import nvfp4_oracle
    nvfp4_oracle.build()
    return nvfp4_oracle


@pytest.fixture(scope="session")
def lib():
    from eval_test_b200 import _lib
    return _lib.load()
