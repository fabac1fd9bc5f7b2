"""Training-loop hooks: base class, metric logging, profiler traces, table eviction and table statistics, sample-level traces
into a columnar table, experiment tracking."""
import importlib as _importlib
import sys as _sys

_WHERE = {"Hook": "hook", "LoggerHook": "logger_hook", "ProfilerHook": "profiler_hook", "HashTableFilterHook": "filter_hook",
          "TableStatsHook": "table_stats_hook", "TraceToOdpsHook": "trace_hook", "TraceHook": "trace_hook", "add_to_trace": "trace_hook",
          "MLTrackerHook": "ml_tracker_hook", "add_to_ml_tracker": "ml_tracker_hook"}
for _name, _module in _WHERE.items():
    globals()[_name] = getattr(_importlib.import_module(f"{__name__}.{_module}"), _name)
__all__ = list(_WHERE)

# the reference's module name for the trace hook resolves to the same module
_sys.modules.setdefault(__name__ + ".trace_to_odps_hook", _importlib.import_module(f"{__name__}.trace_hook"))
