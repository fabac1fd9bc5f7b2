import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(autouse=True)
def _fresh_table_registry():
    """Table names are process-wide unique; every test starts from an empty registry."""
    from recis_b200.nn.modules.hashtable import HashtableRegister
    HashtableRegister().clear()
    yield
    HashtableRegister().clear()
