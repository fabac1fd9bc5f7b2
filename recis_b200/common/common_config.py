"""Process-wide JSON configuration (``recis/common/common_config.py:12-78``).

``set_config(path, transforms)`` loads a JSON file (also accepted here: a dict or a JSON string) and replaces every string value
that is a key of ``transforms`` by its mapped value, at any depth of dicts and lists; ``get_config("a", "b", default=...)`` walks
nested keys. ``get_access_id`` / ``get_access_key`` decode credentials passed through the environment with the RSA helpers.
"""
from __future__ import annotations

import json
import os
from typing import Optional, Union

_CONFIG: dict = {}


def _substitute(node, transforms):
    if isinstance(node, dict):
        for k, v in node.items():
            node[k] = _substitute(v, transforms)
        return node
    if isinstance(node, list):
        for i, v in enumerate(node):
            node[i] = _substitute(v, transforms)
        return node
    if isinstance(node, str) and node in transforms:
        return transforms[node]
    return node


def set_config(path: Optional[Union[str, dict]] = None, transforms: Optional[dict] = None) -> dict:
    global _CONFIG
    if path is None:
        conf = {}
    elif isinstance(path, dict):
        conf = json.loads(json.dumps(path))           # private deep copy
    elif os.path.exists(path):
        with open(path) as fh:
            conf = json.load(fh)
    else:
        conf = json.loads(path)                       # a JSON document passed as text
    if transforms:
        _substitute(conf, transforms)
    _CONFIG = conf
    return _CONFIG


def get_config(*keys, **kwargs):
    """``get_config()`` -> the whole configuration; ``get_config("a", "b", default=x)`` -> ``conf["a"]["b"]`` or ``x``."""
    default = kwargs.pop("default", None)
    value = _CONFIG
    for k in keys:
        if not isinstance(value, dict) or k not in value:
            return default
        value = value[k]
    return value


def _decoded_env(name: str):
    encoded = os.getenv(name)
    key = os.getenv("XDL_AK_PRIVATE_KEY_INTERNAL")
    if encoded and key:
        from . import crypto_utils
        return crypto_utils.decode(encoded, key)
    return None


def get_access_id():
    return _decoded_env("ENCODED_ODPS_ACCESS_ID")


def get_access_key():
    return _decoded_env("ENCODED_ODPS_ACCESS_KEY")
