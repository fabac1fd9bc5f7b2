"""Training-loop hooks: base class, metric logging, profiler traces, table eviction and table statistics."""
import importlib as _importlib

_WHERE = {"Hook": "hook", "LoggerHook": "logger_hook", "ProfilerHook": "profiler_hook", "HashTableFilterHook": "filter_hook",
          "TableStatsHook": "table_stats_hook"}
for _name, _module in _WHERE.items():
    globals()[_name] = getattr(_importlib.import_module(f"{__name__}.{_module}"), _name)
__all__ = list(_WHERE)
