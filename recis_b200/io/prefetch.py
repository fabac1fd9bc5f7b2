"""Host-to-device prefetch: the next batches are copied on a side stream while the current step computes.

The reference gets the same overlap from its native packer, which can emit batches directly into GPU memory on a private
stream, followed by a prefetch stage (``third_party/column-io``: ``dataset/packer.cc:61-113,382-413`` and
``PrefetchDataset``). Here the copy stream and the hand-over are explicit:

* ``depth`` batches are in flight; each is copied from (ideally pinned) host memory with non-blocking copies on the copy
  stream and fenced by a CUDA event;
* ``prefetch()`` (called by the training loop once the current step is queued) issues the copies of the next batches;
* ``next()`` makes the consumer's stream wait for that event (no host synchronisation) and tells the caching allocator that
  the consumer's stream uses the memory (``record_stream``), so the buffers are not recycled under a running kernel.
"""
from __future__ import annotations

from collections import deque

import torch

from ..ragged import RaggedTensor
from ..utils.data_utils import copy_data_to_device


def _tensors(obj):
    if isinstance(obj, torch.Tensor):
        yield obj
    elif isinstance(obj, RaggedTensor):
        yield obj.values()
        for o in obj.offsets():
            yield o
        if obj.weight() is not None:
            yield obj.weight()
    elif isinstance(obj, dict):
        for v in obj.values():
            yield from _tensors(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _tensors(v)


class DevicePrefetcher:
    """Iterate over ``source`` (batches on the host) yielding the same batches on ``device``, copied ahead of use."""

    def __init__(self, source, device, depth: int = 2):
        self.source = iter(source)
        self.device = torch.device(device)
        self.depth = max(int(depth), 1)
        self.on_gpu = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device) if self.on_gpu else None
        self.queue = deque()
        self.exhausted = False

    def _issue(self):
        try:
            host = next(self.source)
        except StopIteration:
            self.exhausted = True
            return
        if not self.on_gpu:
            self.queue.append((host, None))
            return
        with torch.cuda.stream(self.stream):
            dev = copy_data_to_device(host, self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.queue.append((dev, ev))

    def __iter__(self):
        return self

    def __next__(self):
        while len(self.queue) < self.depth and not self.exhausted:
            self._issue()
        if not self.queue:
            raise StopIteration
        batch, ev = self.queue.popleft()
        if ev is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(ev)
            for t in _tensors(batch):
                if t.is_cuda:
                    t.record_stream(cur)
        return batch

    def prefetch(self):
        """Top the pipeline up. Call it right after the current step's kernels have been queued: the host then issues the
        copies of the next batches while the GPU is busy, instead of delaying the start of the next step."""
        while len(self.queue) < self.depth and not self.exhausted:
            self._issue()
