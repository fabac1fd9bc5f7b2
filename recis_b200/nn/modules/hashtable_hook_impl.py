"""Implementations behind ``AdmitHook`` / ``FilterHook`` descriptors.

Reference: ``recis/nn/modules/hashtable_hook_impl.py:14-590`` (``ReadOnlyHookImpl``,
``GlobalStepFilterHookImpl``, factory + registry). Differences: the last-seen step of a row is written by the
table's own lookup kernel (no separate slot-update launch per forward), expiry is one native scan over the
index, and a count-based admission policy exists (``CountAdmit``).
"""
from __future__ import annotations

import weakref

import torch

from ..hashtable_hook import AdmitHook, FilterHook


class BaseAdmitHookImpl:
    """Base of admission policies (``recis/nn/modules/hashtable_hook_impl.py:193-210``). A policy is two attributes that the
    table's lookup reads: ``readonly`` (never insert) and ``threshold`` (occurrences before an id is given a row)."""

    readonly = False
    threshold = 1

    def __init__(self, **kwargs) -> None:
        pass


class BaseFilterHookImpl:
    """Base of eviction policies (``recis/nn/modules/hashtable_hook_impl.py:259-290``): ``before_lookup`` sees the ids of a
    lookup, ``do_filter`` removes what has expired."""

    def before_lookup(self, *args, **kwargs):
        pass

    def do_filter(self, *args, **kwargs):
        pass


class ReadOnlyHookImpl(BaseAdmitHookImpl):
    """Lookups do not insert; unknown ids read as zeros and receive no gradient."""

    readonly = True
    threshold = 1

    def __init__(self, table=None, **params):
        pass


class CountAdmitHookImpl(BaseAdmitHookImpl):
    """An id is given a row at its ``threshold``-th occurrence; before that it reads as zeros."""

    readonly = False

    def __init__(self, table=None, threshold: int = 2, **params):
        self.threshold = int(threshold)


def admit_params(hook):
    """``(readonly, admit_threshold)`` for an ``AdmitHook`` descriptor, an impl, or None."""
    if hook is None:
        return False, 1
    if isinstance(hook, AdmitHook):
        hook = HashtableHookFactory().create_admit_hook(None, hook)
    return bool(hook.readonly), int(hook.threshold)


class GlobalStepFilterHookImpl(torch.nn.Module, BaseFilterHookImpl):
    """TTL eviction: a row is expired when ``last_seen < global_step - filter_step``.

    ``update_step`` advances the global step (a device scalar the lookup kernel reads, and a host mirror so
    that nothing is read back); ``do_filter`` erases expired rows. Erased rows go back on the free stack, their
    optimizer slots are reset, and a re-inserted id starts from a fresh initializer draw.
    """

    def __init__(self, table, filter_step: int = 100, **params):
        super().__init__()
        object.__setattr__(self, "_table", table)   # plain reference: the table is this module's parent, not a child
        self._filter_step = int(filter_step)
        dev = table.impl.device if hasattr(table, "impl") else table.device
        self.register_buffer("_global_step", torch.zeros(1, dtype=torch.int64, device=dev))
        self._host_step = 0
        self._one = torch.ones(1, dtype=torch.int64, device=dev)

    def step_tensor(self):
        return self._global_step

    def forward(self, rows):  # kept for API symmetry: stamping happens inside the lookup kernel
        return rows

    def update_step(self):
        self._global_step.add_(self._one)
        self._host_step += 1

    def reset_step(self, step: int):
        self._global_step.fill_(int(step))
        self._host_step = int(step)

    @property
    def global_step(self) -> int:
        return self._host_step

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        key = prefix + "_global_step"
        if key in state_dict:
            self._host_step = int(state_dict[key].item())

    def expired_ids(self) -> torch.Tensor:
        impl = self._table.impl if hasattr(self._table, "impl") else self._table
        ids, _rows = impl.store.snapshot(True, self._host_step - self._filter_step)
        return ids

    def do_filter(self) -> int:
        impl = self._table.impl if hasattr(self._table, "impl") else self._table
        ids = self.expired_ids()
        if ids.numel():
            impl.store.erase(ids.contiguous())
        return int(ids.numel())


def _table_key(table) -> str:
    for attr in ("_name", "name"):
        v = getattr(table, attr, None)
        if isinstance(v, str):
            return v
    return str(id(table))


class HashtableHookFactory:
    """Name -> implementation registry (singleton)."""

    _instance = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
            cls._instance._admit = {"ReadOnly": ReadOnlyHookImpl, "CountAdmit": CountAdmitHookImpl}
            cls._instance._filter = {"GlobalStepFilter": GlobalStepFilterHookImpl}
            cls._instance._filters, cls._instance._admits = {}, {}
        return cls._instance

    # names used by the reference (recis/nn/modules/hashtable_hook_impl.py:61-75,153-200)
    def regist_admit(self, name, impl):
        if name in self._admit:
            raise ValueError(f"admit hook {name} already registered")
        self._admit[name] = impl

    def regist_filter(self, name, impl):
        if name in self._filter:
            raise ValueError(f"filter hook {name} already registered")
        self._filter[name] = impl

    def get_filters(self):
        """Filter hook instances of the tables that are alive, by table name (held weakly: a table that is gone drops out)."""
        return {k: r() for k, r in list(self._filters.items()) if r() is not None}

    def get_admits(self):
        return {k: r() for k, r in list(self._admits.items()) if r() is not None}

    def register_admit_hook(self, name, impl):
        self._admit[name] = impl

    def register_filter_hook(self, name, impl):
        self._filter[name] = impl

    def create_admit_hook(self, table, hook: AdmitHook):
        if hook.name not in self._admit:
            raise ValueError(f"unknown admit hook {hook.name}; known: {sorted(self._admit)}")
        inst = self._admit[hook.name](table, **hook.params)
        self._admits[_table_key(table)] = weakref.ref(inst)
        return inst

    def create_filter_hook(self, table, hook: FilterHook):
        if hook.name not in self._filter:
            raise ValueError(f"unknown filter hook {hook.name}; known: {sorted(self._filter)}")
        inst = self._filter[hook.name](table, **hook.params)
        self._filters[_table_key(table)] = weakref.ref(inst)
        return inst
