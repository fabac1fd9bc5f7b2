"""recis_b200: a Blackwell-native (sm_100a) sparse + dense recommendation training framework."""
__version__ = "0.1.0"

from . import _ext  # noqa: F401


def native():
    """The compiled extension module (built on first use)."""
    return _ext.load()
