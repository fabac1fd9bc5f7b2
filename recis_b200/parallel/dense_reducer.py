"""Data-parallel gradient averaging for the dense tower, started bucket by bucket while backward still runs.

All dense gradients live in ONE flat fp32 buffer (each ``param.grad`` is a view into it). The buffer is cut into buckets of
whole parameters in reverse registration order, which is roughly the order in which backward produces them. Every parameter
carries a post-accumulate hook; when the last gradient of a bucket has landed (and every earlier bucket has been started, so
that all ranks start them in the same order), the bucket's average is launched on a side stream and overlaps the rest of
backward. The first step only records which parameters receive a gradient at all (the others are not waited for afterwards)
and starts everything after backward. ``all_reduce_async()`` after backward starts whatever is left,
``wait()`` joins before the dense optimizer step. The reference gets the same overlap from HF accelerate ->
``DistributedDataParallel`` (``recis/framework/trainer.py:170-184``).

On CUDA with more than one rank the buffer is peer-mapped and a bucket's average is our own two-shot all-reduce kernel
(``csrc/kernels/comm.cu``): every rank reduces 1/W of the bucket from all peers over NVLink and writes the averaged slice
back into every peer's buffer. ``RECIS_COMM=nccl`` (or CPU tensors) selects an asynchronous ``all_reduce`` per bucket
instead. ``RECIS_DENSE_BUCKET_MB`` (default 4) is the bucket size; 0 keeps one bucket that starts after backward.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import native

CH_AR0, CH_AR1, N_CH = 3, 4, 8


class _Bucket:
    __slots__ = ("start", "length", "n_params", "pending", "launched", "work")

    def __init__(self, start):
        self.start, self.length, self.n_params, self.pending, self.launched, self.work = start, 0, 0, 0, False, None


class DenseGradReducer:
    def __init__(self, params, world: int, pg=None, p2p=None, bucket_mb: float = None):
        self.params = [p for p in params if p.requires_grad]
        self.world = world
        self.pg = pg
        dev = self.params[0].device
        mode = os.environ.get("RECIS_COMM", "auto")
        if p2p is None:
            # CUDA: our all-reduce unless NCCL is asked for. CPU ranks of one machine: only when asked for (RECIS_COMM=fused),
            # over shared memory with the kernels' host twins
            from .symmetric import single_node
            p2p = world > 1 and world <= native().MAX_PEERS and single_node(world) and ((dev.type == "cuda" and mode != "nccl") or (dev.type == "cpu" and mode == "fused"))
        self.p2p = p2p
        self.host = dev.type != "cuda"
        self.epoch = 0
        self.armed = True          # False: hooks do nothing (a micro-batch that is not an accumulation boundary)
        self.grad_scale = 1.0      # folded into the average (1 / accumulation steps)
        if bucket_mb is None:
            bucket_mb = float(os.environ.get("RECIS_DENSE_BUCKET_MB", "4"))
        cap = int(bucket_mb * (1 << 20) / 4) if bucket_mb > 0 and world > 1 else 0
        # every bucket starts on a multiple of 4 * world floats: the all-reduce kernel splits a bucket into W slices of float4
        quantum = 4 * max(world, 1)
        self.buckets, placement, off = [], [], 0
        cur = _Bucket(0)
        for p in reversed(self.params):
            assert p.dtype == torch.float32, "dense master weights are fp32"
            if cap and cur.length and cur.length + p.numel() > cap:
                off = (cur.start + cur.length + quantum - 1) // quantum * quantum
                cur.length = off - cur.start
                self.buckets.append(cur)
                cur = _Bucket(off)
            placement.append((p, cur.start + cur.length, len(self.buckets)))
            cur.length += p.numel()
            cur.n_params += 1
        self.n = cur.start + cur.length
        self.n_pad = (self.n + quantum - 1) // quantum * quantum
        cur.length = self.n_pad - cur.start
        self.buckets.append(cur)
        if p2p:
            from .symmetric import SymmetricHeap
            self.heap = SymmetricHeap({"flags": (torch.int64, N_CH * world), "grads": (torch.float32, self.n_pad)}, dev, pg)
            self.flat = self.heap["grads"].tensor
            self.flat.zero_()
            self.status = torch.zeros(1, dtype=torch.int64, device=dev)
            self.stream = torch.cuda.Stream(device=dev) if not self.host else None
            self.rank = dist.get_rank(pg)
            self.spin_limit = int(float(os.environ.get("RECIS_WAIT_TIMEOUT_S", "20")) * 1e6)  # microseconds
        else:
            self.flat = torch.zeros(self.n_pad, dtype=torch.float32, device=dev)
        self._hooks = []
        self._placement = [(p, start) for p, start, _ in placement]
        self._used = [False] * len(placement)
        self._bucket_of = [b for _, _, b in placement]
        self._learned = False
        for k, (p, start, b) in enumerate(placement):
            p.grad = self.flat[start:start + p.numel()].view_as(p)
            if world > 1 and cap:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(b, k)))
        self._reset()

    # ---- bucket bookkeeping
    def _reset(self):
        for b in self.buckets:
            b.pending, b.launched, b.work = b.n_params, False, None
        self._next = 0

    def _make_hook(self, index, k):
        def hook(_param):
            if not self.armed:              # other micro-batches only accumulate
                return
            b = self.buckets[index]
            if not self._learned:           # the first step finds out which parameters take part in the graph
                self._used[k] = True
                return
            if not self._used[k]:           # a parameter that joined the graph later: counted from the next step on
                if b.launched:
                    raise RuntimeError("dense reducer: a parameter that had no gradient in the first step got one after its "
                                       "bucket's average had started; build the reducer with bucket_mb=0 for such a model")
                self._used[k] = True
                b.n_params += 1
                return
            b.pending -= 1
            self._launch_ready()
        return hook

    def _launch_ready(self, force=False):
        while self._next < len(self.buckets) and (force or self.buckets[self._next].pending <= 0):
            self._launch(self.buckets[self._next])
            self._next += 1

    def _launch(self, b):
        b.launched = True
        if not self.p2p:
            b.work = dist.all_reduce(self.flat[b.start:b.start + b.length], op=dist.ReduceOp.SUM, group=self.pg, async_op=True)
            return
        C = native()
        self.epoch += 1
        if self.host:                      # no streams on the host: the phases run here and now
            self._phases(C, b, self.epoch)
            return
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            self._phases(C, b, self.epoch)

    def _phases(self, C, b, e):
        h, W, me = self.heap, self.world, self.rank
        bufs = [p + 4 * b.start for p in h["grads"].ptrs]
        C.comm_signal(h["flags"].ptrs, CH_AR0, me, e, self.host)
        C.comm_wait(h["flags"].tensor, CH_AR0, W, e, self.spin_limit, self.status)
        C.comm_allreduce_slice(bufs, me, b.length, self.grad_scale / W, self.host)
        C.comm_signal(h["flags"].ptrs, CH_AR1, me, e, self.host)
        C.comm_wait(h["flags"].tensor, CH_AR1, W, e, self.spin_limit, self.status)

    # ---- the calls of a training step
    def all_reduce_async(self):
        """Start averaging whatever backward's hooks have not started yet (call after backward)."""
        if self.world == 1:
            if self.grad_scale != 1.0:
                self.flat.mul_(self.grad_scale)
            return
        self._launch_ready(force=True)

    def wait(self):
        """Make the main stream wait for the averaged gradients (call before the dense optimizer step)."""
        if self.world == 1:
            return
        from .spans import span_close, span_open
        tok = span_open("dense_allreduce_wait")
        if not self.p2p:
            for b in self.buckets:
                if b.work is not None:
                    b.work.wait()
            self.flat.mul_(self.grad_scale / self.world)
        elif not self.host:
            torch.cuda.current_stream().wait_stream(self.stream)
        span_close(tok)
        if not self._learned and self._hooks:
            self._learned = True
            for b in self.buckets:
                b.n_params = 0
            for k, used in enumerate(self._used):
                self.buckets[self._bucket_of[k]].n_params += int(used)
        self._reset()

    def all_reduce(self):
        self.all_reduce_async()
        self.wait()

    def check(self):
        if self.p2p and int(self.status.item()) != 0:
            raise RuntimeError("dense all-reduce: a peer did not signal within the wait limit")
