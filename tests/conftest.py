import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a B200 (sm_100a) GPU; run with -m gpu')


@pytest.fixture(scope='session')
def kvm_lib():
    """The built shared library (compiled on demand; nvcc cross-compiles without a GPU)."""
    from kvm_b200 import build
    return build.build()
