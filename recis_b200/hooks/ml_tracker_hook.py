"""Experiment tracking: values named during a step are logged against the global step.

The reference logs to a proprietary tracking service (``recis/hooks/ml_tracker_hook.py:15-153``: ``add_to_ml_tracker`` fills
a global map, ``MLTrackerHook.after_step`` calls ``tracker.log(map, global_step)``, ``end`` calls ``tracker.finish()``). The
same interface here over a tracker object with ``log(data, step)`` / ``finish()``:

* the ``ml_tracker`` package, when it is installed (``ml_tracker.init(project=, name=, id=, config=)``);
* otherwise ``FileTracker``: one run directory ``<root>/<project>/<name>-<id>/`` with ``config.json`` and ``metrics.jsonl``
  (one JSON object per step: ``{"step": n, "time": t, ...values}``), ``root`` being ``$RECIS_TRACKER_DIR`` or
  ``./ml_tracker``. Any fsspec URL works as the root (on stores without append the log is written in parts, flushed every few
  steps). Only rank 0 writes unless ``all_ranks=True``.

Scalars on the GPU are read in ``after_step`` (one small device-to-host copy per named value and step); tensors with more than
one element are logged as lists.
"""
from __future__ import annotations

import json
import os
import time
import uuid
from typing import Dict, Optional

import numpy as np
import torch

from ..utils.logger import Logger
from .hook import Hook

logger = Logger(__name__)

TRACE_MAP: Dict[str, object] = {}


def get_trace_map():
    return TRACE_MAP


def clear_trace_map():
    global TRACE_MAP
    TRACE_MAP = {}


def add_to_ml_tracker(name: str, data):
    """Name a value to log with this step (``recis/hooks/ml_tracker_hook.py:49-79``). Tensors are detached; they are brought to
    the host when the step is logged."""
    TRACE_MAP[name] = data.detach() if isinstance(data, torch.Tensor) else data


def _plain(v):
    """A JSON-serialisable form: scalars as numbers, arrays as lists."""
    if isinstance(v, torch.Tensor):
        v = v.float().cpu().numpy() if v.dtype in (torch.bfloat16, torch.float16) else v.cpu().numpy()
    if isinstance(v, np.ndarray):
        return v.item() if v.size == 1 else v.tolist()
    if isinstance(v, np.generic):
        return v.item()
    if isinstance(v, dict):
        return {str(k): _plain(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    return v


class FileTracker:
    """A run as files: ``config.json`` once, ``metrics.jsonl`` appended per step, ``finished`` at the end."""

    def __init__(self, project: str, name: str, id: Optional[str] = None, config: Optional[Dict] = None, root: Optional[str] = None):
        import fsspec
        self.id = str(id) if id is not None else uuid.uuid4().hex[:8]
        root = root or os.environ.get("RECIS_TRACKER_DIR") or "./ml_tracker"
        self.fs, base = fsspec.core.url_to_fs(str(root))
        self.dir = "/".join([base.rstrip("/"), project, f"{name}-{self.id}"])
        self.fs.makedirs(self.dir, exist_ok=True)
        with self.fs.open(self.dir + "/config.json", "w") as f:
            json.dump({"project": project, "name": name, "id": self.id, "config": _plain(config or {}), "started": time.time()}, f, indent=1)
        # Real file systems append a line per step. Object stores cannot append: there the log is written in parts of
        # ``part_lines`` lines (``metrics-00000.jsonl``, ...), the part in progress being rewritten every ``flush_every`` steps
        # and at the end, so the cost per step does not grow with the length of the run.
        self._append = getattr(self.fs, "protocol", "file") in ("file", ("file", "local"), "local")
        self._lines, self._part, self._dirty = [], 0, 0
        self.part_lines, self.flush_every = 10_000, 20
        self.steps = 0

    def log(self, data: Dict, step: int):
        rec = {"step": int(step), "time": time.time()}
        rec.update({k: _plain(v) for k, v in data.items()})
        line = json.dumps(rec) + "\n"
        if self._append:
            with self.fs.open(self.dir + "/metrics.jsonl", "a") as f:
                f.write(line)
        else:
            self._lines.append(line)
            self._dirty += 1
            if self._dirty >= self.flush_every or len(self._lines) >= self.part_lines:
                self._write_part()
        self.steps += 1

    def _part_name(self):
        # the first part keeps the plain name, so that short runs look the same on every file system
        return "/metrics.jsonl" if self._part == 0 else f"/metrics-{self._part:05d}.jsonl"

    def _write_part(self):
        if self._lines:
            with self.fs.open(self.dir + self._part_name(), "w") as f:
                f.writelines(self._lines)
        self._dirty = 0
        if len(self._lines) >= self.part_lines:
            self._lines, self._part = [], self._part + 1

    def finish(self):
        if not self._append:
            self._write_part()
        with self.fs.open(self.dir + "/finished", "w") as f:
            f.write(json.dumps({"steps": self.steps, "time": time.time()}))


class _NullTracker:
    def log(self, data, step):
        pass

    def finish(self):
        pass


def init_tracker(project: str, name: str, id=None, config: Optional[Dict] = None, root: Optional[str] = None):
    """The tracking service's client when its package is installed, else a ``FileTracker``."""
    try:
        import ml_tracker
    except ImportError:
        return FileTracker(project, name, id, config, root)
    return ml_tracker.init(project=project, name=name, id=id, config=config)


class MLTrackerHook(Hook):
    """Log what ``add_to_ml_tracker`` collected, once per step (``recis/hooks/ml_tracker_hook.py:82-153``). With
    ``log_metrics=True`` the step's metric dict from the trainer is logged as well."""

    def __init__(self, project: str, name: str, config: Dict, id=None, root: Optional[str] = None, all_ranks: bool = False,
                 log_metrics: bool = False) -> None:
        rank = int(os.environ.get("RANK", "0"))
        self.log_metrics = log_metrics
        self.tracker = init_tracker(project, name, id, config, root) if (rank == 0 or all_ranks) else _NullTracker()

    def after_step(self, metric=None, global_step=0):
        data = dict(get_trace_map())
        if self.log_metrics and isinstance(metric, dict):
            for k, v in metric.items():
                data.setdefault(k, v)
        if data:
            self.tracker.log(data, int(global_step))
        clear_trace_map()

    def end(self):
        self.tracker.finish()
