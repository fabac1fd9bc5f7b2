"""Process-wide JSON configuration (``recis/common/common_config.py:27-45``)."""
from __future__ import annotations

import json

_CONFIG = {}


def set_config(conf):
    """Replace the global configuration with a dict or a JSON string."""
    global _CONFIG
    _CONFIG = dict(json.loads(conf) if isinstance(conf, str) else conf)


def get_config(key=None, default=None):
    return _CONFIG if key is None else _CONFIG.get(key, default)
