"""Admission and eviction policies attached to a table.

Same two descriptor classes as the reference (``recis/nn/hashtable_hook.py:52,163``): a hook is a
``(name, params)`` pair; the implementation is looked up by name when the table is built. Policies:

* ``AdmitHook("ReadOnly")``            lookups never insert; unknown ids read as zeros.
* ``AdmitHook("CountAdmit", {"threshold": n})``  an id gets a row only once it has been seen ``n`` times
  (an addition: the reference has no count-based admission). A sighting is one step in which the id was asked for, by any
  number of ranks (the owning shard dedups what the requesters send before it counts, on every exchange path).
* ``FilterHook("GlobalStepFilter", {"filter_step": n})``  rows not seen for more than ``n`` global steps
  are evicted.
"""
from __future__ import annotations

import json


class BaseHook:
    """``(name, params)`` descriptor; ``type`` tells the two kinds apart (``recis/nn/hashtable_hook.py:10-50``)."""
    type = "base"

    def __init__(self, name: str, params: dict | None = None, **kwargs):
        self.name = name
        self.params = dict(params or {})
        self.params.update(kwargs)

    def __str__(self):
        return json.dumps({"name": self.name, "params": self.params}, sort_keys=True)

    __repr__ = __str__

    def __eq__(self, other):
        return isinstance(other, type(self)) and str(self) == str(other)

    def __hash__(self):
        return hash(str(self))


class AdmitHook(BaseHook):
    """Admission policy descriptor."""
    type = "admit"


class FilterHook(BaseHook):
    """Eviction policy descriptor."""
    type = "filter"


_Hook = BaseHook          # earlier private name
