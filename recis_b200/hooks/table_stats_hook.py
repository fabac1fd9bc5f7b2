"""Publishes the occupancy of every dynamic table as metrics (rows, load factors, probation, evictions), every ``interval``
steps. The counters are read with one small device-to-host copy per table, so the interval should match the logging interval.
The reference has no such hook; its tables expose only their size."""
from __future__ import annotations

from ..framework.metrics import add_metric
from ..nn.modules.hashtable import HashTable
from .hook import Hook


class TableStatsHook(Hook):
    def __init__(self, model=None, interval: int = 100, prefix: str = "table"):
        self.interval = max(int(interval), 1)
        self.prefix = prefix
        self._tables = []
        self._steps = 0
        self._last_rows = {}
        if model is not None:
            self.attach(model)

    def attach(self, model):
        self._tables = [(m.name if hasattr(m, "name") else f"t{i}", m) for i, m in enumerate(mm for mm in model.modules() if isinstance(mm, HashTable))]
        return self

    def collect(self) -> dict:
        out = {}
        for i, (name, table) in enumerate(self._tables):
            st = table.impl.stats()
            key = f"{self.prefix}{i}"
            out[f"{key}/rows"] = st["rows"]
            out[f"{key}/row_load"] = st["row_load"]
            out[f"{key}/index_load"] = st["index_load"]
            out[f"{key}/probation"] = st["probation"]
            out[f"{key}/status"] = st["status"]
            out[f"{key}/rows_delta"] = st["rows"] - self._last_rows.get(i, 0)
            self._last_rows[i] = st["rows"]
        return out

    def after_step(self, metrics=None, global_step=0):
        self._steps += 1
        if self._steps % self.interval:
            return
        for k, v in self.collect().items():
            add_metric(k, v)
            if metrics is not None:
                metrics[k] = v
