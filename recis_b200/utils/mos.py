"""Model store: checkpoints addressed by ``model.<project>.<name>[/version=<v>[/ckpt_id=<id>]]`` instead of by path.

The reference resolves such URIs through a proprietary model-management service (``recis/utils/mos.py:13-340``, client
library ``nebula.mos``) and uses them in two places: as the ``output_dir`` of a run (``recis/framework/checkpoint_manager.py:
75-78``; every saved or removed checkpoint is reported with ``ckpt_update``, ``:214-219``) and as the ``path`` of a model-bank
entry (``:490-492``). Here the store is a directory tree on any file system, so the same URIs work on a workstation, on
shared storage, or on whatever ``RECIS_MODEL_STORE`` points to::

    <root>/<project>/<model_name>/version=<version>/            output directory of one run
    <root>/<project>/<model_name>/version=<version>/ckpts.json  {"ckpts": {ckpt_id: {"path": ..., "time": ...}}, "order": [...]}

* a model-level URI used for output gets a fresh time-stamped version (as the reference's ``auto_version``);
* a model-level or version-level URI used as a model bank resolves to the newest version / the newest checkpoint listed;
  ``version=max_pt`` means the newest version as well;
* the registry file is rewritten atomically (temporary file + rename), so a reader never sees half of it.
"""
from __future__ import annotations

import json
import os
import re
import tempfile
import time
from typing import Optional

from .logger import Logger

logger = Logger(__name__)

_URI = re.compile(r"^model\.([^./\s]+)\.([^/\s]+?)(?:/version=([^/\s]+))?(?:/ckpt_id=([^/\s]+))?$")
_REGISTRY = "ckpts.json"


def store_root() -> str:
    """Directory under which all models live: ``$RECIS_MODEL_STORE``, else ``~/.recis_model_store``."""
    return os.environ.get("RECIS_MODEL_STORE") or os.path.join(os.path.expanduser("~"), ".recis_model_store")


def parse_uri(uri: str, auto_version: bool = False) -> dict:
    """Split a model URI into ``project, model_name, version, ckpt_id`` and its ``level`` (``model`` / ``version`` /
    ``ckpt_id``). With ``auto_version`` a model-level URI gets a ``%Y%m%d%H%M%S`` version appended
    (``recis/utils/mos.py:13-88``). A version that names a moving target (``max_pt``) keeps the URI at version level even when
    a checkpoint id follows."""
    m = _URI.match(uri or "")
    if not m:
        raise ValueError(f"[MOS] uri is invalid : {uri}")
    project, model_name, version, ckpt_id = m.groups()
    level = "model"
    if version is not None:
        level = "version"
    if ckpt_id is not None:
        if "max_pt" in version:
            ckpt_id = None
        else:
            level = "ckpt_id"
    if level == "model" and auto_version:
        version = time.strftime("%Y%m%d%H%M%S", time.localtime())
        uri = f"{uri}/version={version}"
    return dict(uri=uri, project=project, model_name=model_name, version=version, ckpt_id=ckpt_id, level=level)


def _model_dir(info: dict, root: Optional[str] = None) -> str:
    return os.path.join(root or store_root(), info["project"], info["model_name"])


def _versions(model_dir: str):
    if not os.path.isdir(model_dir):
        return []
    names = [d[len("version="):] for d in os.listdir(model_dir) if d.startswith("version=") and os.path.isdir(os.path.join(model_dir, d))]
    # newest first by registry / directory time, names as the tie-break (time-stamped names sort the same way)
    return sorted(names, key=lambda v: (os.path.getmtime(os.path.join(model_dir, f"version={v}")), v), reverse=True)


def _read_registry(version_dir: str) -> dict:
    path = os.path.join(version_dir, _REGISTRY)
    if not os.path.exists(path):
        return {"ckpts": {}, "order": []}
    with open(path) as f:
        return json.load(f)


def _write_registry(version_dir: str, reg: dict):
    os.makedirs(version_dir, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=version_dir, prefix=".ckpts.", suffix=".tmp")
    with os.fdopen(fd, "w") as f:
        json.dump(reg, f, indent=1, sort_keys=True)
    os.replace(tmp, os.path.join(version_dir, _REGISTRY))


def render_uri_to_output_dir(uri: str, root: Optional[str] = None) -> str:
    """Directory a run writes into. A model-level URI gets a new time-stamped version; the directory is created
    (``recis/utils/mos.py:159-212``)."""
    info = parse_uri(uri, auto_version=True)
    path = os.path.join(_model_dir(info, root), f"version={info['version']}")
    os.makedirs(path, exist_ok=True)
    return path


def render_uri_to_model_bank_path(uri: str, user_id: Optional[str] = None, root: Optional[str] = None):
    """``(path, info)`` of an existing checkpoint to load from. Missing parts resolve to the newest: the newest version of the
    model, the checkpoint saved last in that version (``recis/utils/mos.py:90-156``). ``user_id`` is accepted for the
    reference's signature; access control is the file system's."""
    info = parse_uri(uri)
    model_dir = _model_dir(info, root)
    version = info["version"]
    if version is None or "max_pt" in version:
        versions = _versions(model_dir)
        if not versions:
            raise FileNotFoundError(f"[MOS] no version of {uri} under {model_dir}")
        version = versions[0]
    version_dir = os.path.join(model_dir, f"version={version}")
    reg = _read_registry(version_dir)
    ckpt_id = info["ckpt_id"]
    if ckpt_id is None:
        if not reg["order"]:
            raise FileNotFoundError(f"[MOS] version {version} of {uri} lists no checkpoint")
        ckpt_id = reg["order"][-1]
    entry = reg["ckpts"].get(ckpt_id)
    path = entry["path"] if entry else os.path.join(version_dir, ckpt_id)
    if not os.path.isdir(path):
        raise FileNotFoundError(f"[MOS] checkpoint {ckpt_id} of {uri} not found at {path}")
    info = dict(info, version=version, ckpt_id=ckpt_id)
    return path, info


class Mos:
    """Resolves a model URI to a directory and keeps the version's checkpoint registry
    (``recis/utils/mos.py:215-340``). ``model_bank_path=True`` resolves an existing checkpoint to load;
    otherwise the URI names where a run saves."""

    def __init__(self, uri: str, model_bank_path: bool = False, root: Optional[str] = None):
        if not str(uri).startswith("model."):
            raise ValueError(f"[MOS] uri is invalid : {uri}")
        self.uri = uri
        self.root = root or store_root()
        self.user_id = os.environ.get("USER_ID")
        if model_bank_path:
            self.real_physical_path, self.uri_info = render_uri_to_model_bank_path(uri, self.user_id, self.root)
            self._version_dir = os.path.join(_model_dir(self.uri_info, self.root), f"version={self.uri_info['version']}")
        else:
            self.uri_info = parse_uri(uri, auto_version=True)
            self.real_physical_path = render_uri_to_output_dir(self.uri_info["uri"], self.root)
            self._version_dir = self.real_physical_path
        self.version_uri = "model.{}.{}/version={}".format(self.uri_info["project"], self.uri_info["model_name"], self.uri_info["version"])

    def ckpt_update(self, ckpt_id: str, path: Optional[str] = None, is_delete: bool = False):
        """Record (or, with ``is_delete``, forget) one checkpoint of this version."""
        reg = _read_registry(self._version_dir)
        if is_delete:
            reg["ckpts"].pop(ckpt_id, None)
            reg["order"] = [c for c in reg["order"] if c != ckpt_id]
            logger.warning(f"[MOS] delete ckpt_id = {ckpt_id}")
        else:
            reg["ckpts"][ckpt_id] = {"path": os.path.abspath(path or os.path.join(self._version_dir, ckpt_id)), "time": time.time()}
            reg["order"] = [c for c in reg["order"] if c != ckpt_id] + [ckpt_id]
        _write_registry(self._version_dir, reg)

    def list_ckpts(self):
        """Checkpoint ids of this version, oldest first."""
        return list(_read_registry(self._version_dir)["order"])
