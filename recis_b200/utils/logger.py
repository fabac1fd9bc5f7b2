"""Logger with rank-0 helpers: INFO to stdout, everything above to stderr (``recis/utils/logger.py:51-196``)."""
from __future__ import annotations

import logging
import os
import sys


class _MaxLevel(logging.Filter):
    def __init__(self, level):
        super().__init__()
        self.level = level

    def filter(self, record):
        return record.levelno <= self.level


class SingleLevelFilter(logging.Filter):
    """Passes only records of ``passlevel``, or with ``reject`` everything but them (``recis/utils/logger.py:6-48``)."""

    def __init__(self, passlevel, reject):
        super().__init__()
        self.passlevel, self.reject = passlevel, reject

    def filter(self, record):
        return (record.levelno != self.passlevel) if self.reject else (record.levelno == self.passlevel)


class Logger:
    _FMT = "%(asctime)s %(levelname)s [%(name)s] %(message)s"

    def __init__(self, name: str = "recis_b200", level=logging.INFO):
        self._logger = logging.getLogger(name)
        if not self._logger.handlers:
            out = logging.StreamHandler(sys.stdout)
            out.addFilter(_MaxLevel(logging.INFO))
            err = logging.StreamHandler(sys.stderr)
            err.setLevel(logging.WARNING)
            for h in (out, err):
                h.setFormatter(logging.Formatter(self._FMT))
                self._logger.addHandler(h)
            self._logger.propagate = False
        self._logger.setLevel(level)

    @staticmethod
    def _rank0():
        return int(os.environ.get("RANK", "0")) == 0

    def set_level(self, level):
        self._logger.setLevel(level)

    def debug(self, msg, *a, **k): self._logger.debug(msg, *a, **k)
    def info(self, msg, *a, **k): self._logger.info(msg, *a, **k)
    def warning(self, msg, *a, **k): self._logger.warning(msg, *a, **k)
    def error(self, msg, *a, **k): self._logger.error(msg, *a, **k)
    def critical(self, msg, *a, **k): self._logger.critical(msg, *a, **k)

    def info_rank0(self, msg, *a, **k):
        if self._rank0():
            self._logger.info(msg, *a, **k)

    def error_rank0(self, msg, *a, **k):
        if self._rank0():
            self._logger.error(msg, *a, **k)

    def warning_rank0(self, msg, *a, **k):
        if self._rank0():
            self._logger.warning(msg, *a, **k)
