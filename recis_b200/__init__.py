"""recis_b200: a Blackwell-native (sm_100a) sparse + dense recommendation training framework."""
__version__ = "0.2.0"

from . import _ext  # noqa: F401


def native():
    """The compiled extension module (built on first use)."""
    return _ext.load()


def get_build_info() -> dict:
    """Version, target architecture and whether the native extension is built (``recis.get_build_info`` in the reference)."""
    return {"version": __version__, "cuda_arch": "sm_100a", "native_built": _ext.is_built(), "source_hash": _ext.source_hash()[:16]}


def is_internal_enabled() -> bool:
    """The reference gates proprietary storage back-ends behind this flag; there are none here."""
    return False
