"""Build information (``recis/info.py`` is generated at build time in the reference; ``recis/__info__.py`` is its template)."""
from . import __version__, get_build_info, is_internal_enabled

__all__ = ["__version__", "get_build_info", "is_internal_enabled"]
