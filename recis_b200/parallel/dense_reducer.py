"""Data-parallel gradient averaging for the dense tower.

All dense gradients live in ONE flat fp32 buffer (each ``param.grad`` is a view into it), so averaging is a single
operation over a few MB instead of one per parameter. The reference gets bucketing from HF accelerate ->
``DistributedDataParallel`` (``recis/framework/trainer.py:170-184``).

On CUDA with more than one rank the buffer is peer-mapped and the average is our own two-shot all-reduce kernel
(``csrc/kernels/comm.cu``): every rank reduces 1/W of the buffer from all peers over NVLink and writes the averaged slice
back into every peer's buffer. It runs on a side stream, so it overlaps with whatever the main stream does next (the
sparse optimizer's embedding update); ``wait()`` joins it before the dense optimizer step. ``RECIS_COMM=nccl`` (or CPU
tensors) selects a plain ``all_reduce`` instead.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import native

CH_AR0, CH_AR1, N_CH = 3, 4, 8


class DenseGradReducer:
    def __init__(self, params, world: int, pg=None, p2p=None):
        self.params = [p for p in params if p.requires_grad]
        self.world = world
        self.pg = pg
        n = sum(p.numel() for p in self.params)
        dev = self.params[0].device
        mode = os.environ.get("RECIS_COMM", "auto")
        if p2p is None:
            # CUDA: our all-reduce unless NCCL is asked for. CPU ranks of one machine: only when asked for (RECIS_COMM=fused),
            # over shared memory with the kernels' host twins
            from .symmetric import single_node
            p2p = world > 1 and world <= native().MAX_PEERS and single_node(world) and ((dev.type == "cuda" and mode != "nccl") or (dev.type == "cpu" and mode == "fused"))
        self.p2p = p2p
        self.host = dev.type != "cuda"
        self.n = n
        self.epoch = 0
        if p2p:
            from .symmetric import SymmetricHeap
            quantum = 4 * world
            self.n_pad = (n + quantum - 1) // quantum * quantum
            self.heap = SymmetricHeap({"flags": (torch.int64, N_CH * world), "grads": (torch.float32, self.n_pad)}, dev, pg)
            self.flat = self.heap["grads"].tensor[:n]
            self.status = torch.zeros(1, dtype=torch.int64, device=dev)
            self.stream = torch.cuda.Stream(device=dev) if not self.host else None
            self.rank = dist.get_rank(pg)
            self.spin_limit = int(float(os.environ.get("RECIS_WAIT_TIMEOUT_S", "20")) * 1e6)  # microseconds
        else:
            self.flat = torch.zeros(n, dtype=torch.float32, device=dev)
        off = 0
        for p in self.params:
            assert p.dtype == torch.float32, "dense master weights are fp32"
            p.grad = self.flat[off:off + p.numel()].view_as(p)
            off += p.numel()

    def all_reduce_async(self):
        """Start averaging the gradients (call after backward)."""
        if self.world == 1:
            return
        if not self.p2p:
            from .spans import span_close, span_open
            tok = span_open("dense_allreduce_wait")          # a collective on the model's stream: all of it is exposed
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.pg)
            self.flat.mul_(1.0 / self.world)
            span_close(tok)
            return
        C = native()
        self.epoch += 1
        e, h, W, me = self.epoch, self.heap, self.world, self.rank
        if self.host:                      # no streams on the host: the two phases run here and now
            self._phases(C, h, W, me, e)
            return
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            self._phases(C, h, W, me, e)

    def _phases(self, C, h, W, me, e):
        C.comm_signal(h["flags"].ptrs, CH_AR0, me, e, self.host)
        C.comm_wait(h["flags"].tensor, CH_AR0, W, e, self.spin_limit, self.status)
        C.comm_allreduce_slice(h["grads"].ptrs, me, self.n_pad, 1.0 / W, self.host)
        C.comm_signal(h["flags"].ptrs, CH_AR1, me, e, self.host)
        C.comm_wait(h["flags"].tensor, CH_AR1, W, e, self.spin_limit, self.status)

    def wait(self):
        """Make the main stream wait for the averaged gradients (call before the dense optimizer step)."""
        if self.world > 1 and self.p2p and not self.host:
            from .spans import span_close, span_open
            tok = span_open("dense_allreduce_wait")
            torch.cuda.current_stream().wait_stream(self.stream)
            span_close(tok)

    def all_reduce(self):
        self.all_reduce_async()
        self.wait()

    def check(self):
        if self.p2p and int(self.status.item()) != 0:
            raise RuntimeError("dense all-reduce: a peer did not signal within the wait limit")
