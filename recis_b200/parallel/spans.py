"""CUDA-event spans around the communication phases of a step ("exposed all-to-all" accounting).

The embedding exchange runs on the stream that also runs the model, so the device time between the start and the end of an
exchange phase on that stream - transfer kernels plus the time spent waiting for peers - is time the step cannot hide behind
compute. ``recorder`` brackets those phases with CUDA events (recorded on the launching stream, as all timing here is) when it
is switched on; switched off (the default) a phase costs one attribute test. The reference has no such accounting; its
all-to-alls are blocking calls between its kernels (``recis/nn/modules/embedding.py:518-533,73-80,110-116``).

Labels used by the package: ``ids`` (requester signal -> owner has pulled the ids), ``emb`` (row push -> rows have arrived),
``grad_push`` (per-unique gradient reduce + push / gradient all-to-all), ``grad_wait`` (owner waits for the gradients),
``dense_allreduce_wait`` (main stream blocked on the dense gradient all-reduce of the side stream).
"""
from __future__ import annotations

from collections import defaultdict
from typing import Dict, Optional

import torch


class SpanRecorder:
    def __init__(self, event_cls=None):
        self.enabled = False
        self._spans = []
        self._event_cls = event_cls          # tests inject a fake; None -> torch.cuda.Event

    def _event(self):
        cls = self._event_cls or torch.cuda.Event
        ev = cls(enable_timing=True)
        ev.record()
        return ev

    def open(self, label: str):
        """Record the start of a phase on the current stream; returns a token for ``close`` (None when switched off)."""
        if not self.enabled:
            return None
        return (label, self._event())

    def close(self, token) -> None:
        if token is None:
            return
        self._spans.append((token[0], token[1], self._event()))

    def start(self) -> None:
        self._spans = []
        self.enabled = True

    def stop(self, steps: int = 1, synchronize=None) -> Dict[str, float]:
        """Switch off and return milliseconds per step and label (plus ``total``). Waits for the recorded events."""
        self.enabled = False
        (synchronize or torch.cuda.synchronize)()
        out: Dict[str, float] = defaultdict(float)
        for label, e0, e1 in self._spans:
            out[label] += e0.elapsed_time(e1)
        self._spans = []
        res = {k: v / max(steps, 1) for k, v in out.items()}
        res["total"] = sum(res.values())
        return res


recorder = SpanRecorder()


def span_open(label: str):
    return recorder.open(label) if recorder.enabled else None


def span_close(token: Optional[tuple]) -> None:
    if token is not None:
        recorder.close(token)
