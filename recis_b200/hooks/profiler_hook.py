"""torch.profiler schedule driven from the step hook; writes a chrome trace per active window
(``recis/hooks/profiler_hook.py:46-116``). ``output_dir`` may be a local directory or any URL that fsspec understands
(``hdfs://``, ``s3://``, ``memory://`` ...): the trace is exported to a local temporary file and put there through the
file system of the URL, as the reference does with its own file-system lookup (``recis/hooks/profiler_hook.py:71-116``).
Sparse-path kernels show up under their own names; NVTX ranges can be added around steps with ``nvtx=True``."""
from __future__ import annotations

import os
import tempfile

import torch

from .hook import Hook


class ProfilerHook(Hook):
    def __init__(self, wait=1, warmup=48, active=1, repeat=4, output_dir="./", record_shapes=True, profile_memory=False,
                 with_stack=False, with_flops=False, nvtx=False):
        self.output_dir = output_dir
        self.app_id = os.environ.get("APP_ID", "recis_b200")
        self.remote = "://" in str(output_dir) and not str(output_dir).startswith("file://")
        if self.remote:
            import fsspec
            self.fs, self.root = fsspec.core.url_to_fs(output_dir)
            self.fs.makedirs(self.root, exist_ok=True)
        else:
            self.fs, self.root = None, str(output_dir)[7:] if str(output_dir).startswith("file://") else output_dir
            os.makedirs(self.root, exist_ok=True)
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self.traces = []
        self._step = 0
        self.nvtx = nvtx and torch.cuda.is_available()
        self.prof = torch.profiler.profile(
            activities=acts, schedule=torch.profiler.schedule(wait=wait, warmup=warmup, active=active, repeat=repeat),
            on_trace_ready=self.get_trace_handler(), record_shapes=record_shapes, profile_memory=profile_memory, with_stack=with_stack,
            with_flops=with_flops)
        self.prof.start()
        if self.nvtx:
            torch.cuda.nvtx.range_push("step 0")

    def get_trace_handler(self):
        """The ``on_trace_ready`` callback: writes ``<APP_ID>-timeline-<step>.json`` into ``output_dir``
        (``recis/hooks/profiler_hook.py:71-116``)."""
        return self._on_trace

    def _on_trace(self, prof):
        name = f"{self.app_id}-timeline-{self._step}.json"
        if not self.remote:
            path = os.path.join(self.root, name)
            prof.export_chrome_trace(path)
        else:
            path = self.root.rstrip("/") + "/" + name
            with tempfile.TemporaryDirectory() as tmp:
                local = os.path.join(tmp, name)
                prof.export_chrome_trace(local)
                self.fs.put_file(local, path)
        self.traces.append(path)

    def after_step(self, metrics=None, global_step=0):
        self._step += 1
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
            torch.cuda.nvtx.range_push(f"step {self._step}")
        self.prof.step()

    def end(self):
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
            self.nvtx = False
        if self.prof is not None:
            self.prof.stop()
            self.prof = None
