"""Drives table eviction from the training loop (``recis/hooks/filter_hook.py:82-117``): every step the global step of
each table's filter advances; every ``filter_interval`` steps rows not seen for longer than the filter's TTL are erased."""
from __future__ import annotations

from ..nn.modules.hashtable import HashTable
from ..utils.logger import Logger
from .hook import Hook


class HashTableFilterHook(Hook):
    def __init__(self, filter_interval: int = 100, model=None):
        self.filter_interval = max(int(filter_interval), 1)
        self._filters = []
        self._steps = 0
        self.evicted = 0
        self.logger = Logger("HashTableFilterHook")
        if model is not None:
            self.attach(model)

    def reset_filter_interval(self, interval: int = 100):
        self.filter_interval = max(int(interval), 1)

    def attach(self, model):
        """Collect the filter of every table inside ``model``."""
        self._filters = [m._filter_hook_impl for m in model.modules() if isinstance(m, HashTable) and m._filter_hook_impl is not None]
        return self

    def _live_filters(self):
        """The attached model's filters, or - when the hook was built without a model, as in the reference - the filter of every
        table alive in the process (``HashtableHookFactory().get_filters()``, ``recis/hooks/filter_hook.py:60-80``)."""
        if self._filters:
            return self._filters
        from ..nn.modules.hashtable_hook_impl import HashtableHookFactory
        return list(HashtableHookFactory().get_filters().values())

    def after_step(self, metrics=None, global_step=0):
        self._steps += 1
        filters = self._live_filters()
        for f in filters:
            f.update_step()
        if self._steps % self.filter_interval == 0:
            n = sum(f.do_filter() for f in filters)
            self.evicted += n
            if n:
                self.logger.info(f"evicted {n} rows at step {self._steps}")
