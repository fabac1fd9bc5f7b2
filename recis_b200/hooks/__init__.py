from .filter_hook import HashTableFilterHook
from .hook import Hook
from .logger_hook import LoggerHook
from .profiler_hook import ProfilerHook
from .table_stats_hook import TableStatsHook

__all__ = ["Hook", "LoggerHook", "ProfilerHook", "HashTableFilterHook", "TableStatsHook"]
