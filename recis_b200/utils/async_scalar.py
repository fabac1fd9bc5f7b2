"""Reading a scalar (a loss, a metric) from the device without draining the stream that produced it.

``float(loss)`` right after a training step waits for everything queued on the model's stream: the backward pass and both
optimizer steps. The GPU then sits idle while the host prepares and launches the next step. The loss itself has been known
since the end of the forward pass, so ``post(loss)`` copies it to pinned host memory on a side stream that waits only for the
forward pass; ``get(ticket)`` at the end of the step waits only for that copy, which finished long before. The host keeps its
lead over the GPU and every step's value is still read in that step. (The reference logs ``loss.item()`` from its logger hook,
``recis/hooks/logger_hook.py``, and pays the drain on every logged step.)
"""
from __future__ import annotations

import torch


class AsyncScalarReader:
    def __init__(self, device, slots: int = 16, dtype=torch.float32):
        self.device = torch.device(device)
        self.on_gpu = self.device.type == "cuda"
        self.slots = int(slots)
        self.host = torch.zeros(self.slots, dtype=dtype)
        self.events = [None] * self.slots
        self.stream = None
        if self.on_gpu:
            self.host = self.host.pin_memory()
            self.stream = torch.cuda.Stream(device=self.device)
        self.head = 0

    def post(self, value: torch.Tensor) -> int:
        """Start copying the 0-d tensor ``value`` (as produced so far on the current stream) to the host; returns a ticket."""
        ticket = self.head
        self.head += 1
        k = ticket % self.slots
        value = value.detach()
        if not self.on_gpu:
            self.host[k] = value
            return ticket
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            self.host[k:k + 1].copy_(value.reshape(1), non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.stream)
        value.record_stream(self.stream)
        self.events[k] = done
        return ticket

    def get(self, ticket: int) -> float:
        """The value behind ``ticket`` (one of the last ``slots`` posts); waits for its copy only."""
        assert self.head - ticket <= self.slots, "the ticket's slot has been reused: read values sooner or use more slots"
        k = ticket % self.slots
        if self.on_gpu:
            self.events[k].synchronize()
        return float(self.host[k])
