"""Data-parallel gradient averaging for the dense tower.

All dense gradients live in ONE flat fp32 buffer (each ``param.grad`` is a view into it), so averaging is a single
collective over a few MB instead of one per parameter. The reference gets the same effect from HF accelerate ->
``DistributedDataParallel`` buckets (``recis/framework/trainer.py:170-184``).

Backends: ``p2p`` (our two-shot all-reduce kernel over peer-mapped memory, see ``fused_exchange``/``comm.cu``) when a
symmetric buffer is available, else ``nccl``/``gloo`` ``all_reduce``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class DenseGradReducer:
    def __init__(self, params, world: int, pg=None, symmetric=None):
        self.params = [p for p in params if p.requires_grad]
        self.world = world
        self.pg = pg
        n = sum(p.numel() for p in self.params)
        dev = self.params[0].device
        self.symmetric = symmetric
        if symmetric is not None:
            self.flat = symmetric.alloc_flat(n)
        else:
            self.flat = torch.zeros(n, dtype=torch.float32, device=dev)
        off = 0
        for p in self.params:
            assert p.dtype == torch.float32, "dense master weights are fp32"
            p.grad = self.flat[off:off + p.numel()].view_as(p)
            off += p.numel()

    def all_reduce(self):
        """Average gradients over ranks in place (call after backward, before the optimizer step)."""
        if self.world == 1:
            return
        if self.symmetric is not None:
            self.symmetric.all_reduce_mean(self.flat)
            return
        dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.pg)
        self.flat.mul_(1.0 / self.world)
