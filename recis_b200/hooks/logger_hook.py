"""Periodic metric logging: ``<gstep=..> <lstep=..> <qps=..> <k=v>...`` (``recis/hooks/logger_hook.py:67-96``).
``qps`` is steps per second over the last interval. Tensor metrics are read back only when a line is printed."""
from __future__ import annotations

import time

import torch

from ..utils.logger import Logger
from .hook import Hook


class LoggerHook(Hook):
    def __init__(self, log_step: int = 10):
        self.log_step = max(int(log_step), 1)
        self.steps = 0
        self.start_time = time.time()
        self.logger = Logger("LoggerHook")
        self.last_line = ""

    @staticmethod
    def format_metrics(metrics) -> str:
        out = ""
        for k, v in (metrics or {}).items():
            if isinstance(v, torch.Tensor) and v.numel() == 1:
                v = v.item()
            out += f" <{k}={v}>"
        return out

    def after_step(self, metrics=None, global_step=0):
        if self.steps % self.log_step == 0:
            spent = max(time.time() - self.start_time, 1e-9)
            gs = int(global_step.item()) if isinstance(global_step, torch.Tensor) else global_step
            self.last_line = f"<gstep={gs}> <lstep={self.steps}> <qps={self.log_step / spent:.4f}>" + self.format_metrics(metrics)
            self.logger.info(self.last_line)
            self.start_time = time.time()
        self.steps += 1
