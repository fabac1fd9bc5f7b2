"""Filesystem selection by path scheme through fsspec (``recis/framework/filesystem.py:18-64``)."""
from __future__ import annotations

import fsspec


def get_file_system(path: str):
    scheme = path.split("://", 1)[0] if "://" in path else "file"
    return fsspec.filesystem(scheme)
