"""Fused embedding exchange: the all-to-alls of a sharded lookup done by our own kernels over peer-mapped memory.

Replaces, per table group and step, the reference's counts / ids / embeddings / gradients ``all_to_all_single`` calls and
the host read of split sizes between them (``recis/nn/modules/embedding.py:498-624``). Protocol (kernels in
``csrc/kernels/comm.cu``):

forward   requester  dedup + bucket ids by owner straight into its symmetric window ............ signal IDS
          owner      wait IDS; pull the ids bucketed for it from every requester (peer loads); table lookup-or-insert;
                     push each row into the requester's unique-embedding buffer (peer stores) .. signal EMB
          requester  wait EMB; pool from its (local) unique-embedding buffer
backward  requester  ONE kernel reduces the pooled gradient to one gradient per unique id and stores it straight into the
                     gradient window of the rank that owns the id (peer stores) ................. signal GRAD
optimizer owner      wait GRAD; ONE kernel adds the contributions of every touched row (duplicates across requesters are
                     chained) and applies the row-wise optimizer update, reading only local memory

No split size ever reaches the host; windows are sized for the worst case (``exchange_capacity`` unique ids per rank).
The same code drives CPU ranks of one machine (``RECIS_COMM=fused`` with CPU tables): the windows then live in POSIX shared
memory and the kernels' host twins (``csrc/cpu/cpu_comm.cc``) do the work - the oracle of this path in the multi-rank tests.
Every (table, runtime group) pair owns one *lane*: its own windows, flag pad and epoch counter, so that the epochs written
to a flag only ever grow and a gradient window is never rewritten before its owner consumed it.
All flag waits are time-bounded; a timeout or a window overflow sets a bit in ``status`` which ``check()`` turns into an
exception.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import native
from .spans import span_close, span_open
from .symmetric import SymmetricHeap

CH_IDS, CH_EMB, CH_GRAD, N_CH = 0, 1, 2, 8
STATUS_TIMEOUT, STATUS_OVERFLOW = 4, 8


class _Lane:
    """Windows + flags of one (table, runtime group) pair."""

    def __init__(self, ex: "FusedExchange", nnz: int):
        # every rank must lay its windows out identically (peers address them by offset): the capacity is agreed on here, once,
        # as the maximum over ranks of the configured value or of twice the first batch's id count
        want = ex.send_cap if ex.send_cap else max(int(nnz) * 2, 1024)
        t = torch.tensor([want], dtype=torch.int64, device=ex.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ex.pg)
        cap = int(t.item())
        W, D = ex.world, ex.D
        self.send_cap = cap
        self.in_cap = min(W, 2) * cap
        self.heap = SymmetricHeap({
            "flags": (torch.int64, N_CH * W),
            "offsets": (torch.int32, W + 1),
            "ids": (torch.int64, cap),
            "uemb": (torch.float32, cap * D),
            "gin": (torch.float32, self.in_cap * D),
        }, ex.device, ex.pg)
        self.ids_in = torch.empty(self.in_cap, dtype=torch.int64, device=ex.device)
        self.prefix = torch.zeros(3 * W + 1, dtype=torch.int32, device=ex.device)
        self.n_in = torch.zeros(1, dtype=torch.int32, device=ex.device)
        self.epoch = 0
        self.pending_grad_epoch = 0      # a staged, not yet consumed gradient window
        self.warned = False
        self.last_train_epoch = 0        # epoch of the newest forward that will be back-propagated


class FusedExchange:
    @staticmethod
    def create(emb_opt, pg, world, rank):
        if emb_opt.embedding_dim % 4 != 0 or emb_opt.embedding_dim > 512 or emb_opt.dtype != torch.float32:
            return None
        if world > native().MAX_PEERS:
            return None
        return FusedExchange(emb_opt, pg, world, rank)

    def __init__(self, emb_opt, pg, world, rank):
        self.opt = emb_opt
        self.pg, self.world, self.rank = pg, world, rank
        self.device = torch.device(emb_opt.device)
        self.D = emb_opt.embedding_dim
        self.host = self.device.type != "cuda"       # CPU ranks: windows in shared memory, the exchange runs in csrc/cpu/cpu_comm.cc
        self.lanes = {}
        self.send_cap = int(os.environ.get("RECIS_EXCHANGE_CAPACITY", "0")) or int(getattr(emb_opt, "exchange_capacity", 0) or 0)
        # time limit of every flag wait; a dead peer then surfaces as an error, never as a hang
        self.wait_us = int(float(os.environ.get("RECIS_WAIT_TIMEOUT_S", "20")) * 1e6)
        self.status = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.immediate_reduce = False
        self.multi_stream = False          # set by the engine when lanes run on separate streams: table lookups are then chained
        self._store_event = None
        self.owner_unroll = int(os.environ.get("RECIS_OWNER_UNROLL", "2"))
        # RECIS_WAIT_STATS=1: flag waits go through the accounting kernel; wait_stats holds nanoseconds per (channel, peer)
        self.wait_stats = (torch.zeros(N_CH * world + N_CH, dtype=torch.int64, device=self.device)
                           if os.environ.get("RECIS_WAIT_STATS") == "1" else None)
        self._head = None
        # RECIS_STAGE_EXCHANGE=1: the engine may issue the id phase of all of a model's groups before the first wait (prepare())
        self.stage_enabled = os.environ.get("RECIS_STAGE_EXCHANGE") == "1"
        self.staged_serves = 0             # how many lookups had their owner side issued ahead of the first wait (serve())

    def _wait(self, flags, channel, epoch):
        C = native()
        if self.wait_stats is None:
            C.comm_wait(flags, channel, self.world, epoch, self.wait_us, self.status)
        else:
            C.comm_wait_timed(flags, channel, self.world, epoch, self.wait_us, self.status, self.wait_stats)

    def exposed_wait_ms(self) -> dict:
        """With RECIS_WAIT_STATS=1: per channel, the mean time of a wait until its last peer arrived (ms), since creation."""
        if self.wait_stats is None:
            return {}
        s = self.wait_stats.cpu()
        W = self.world
        out = {}
        for name, ch in (("ids", CH_IDS), ("emb", CH_EMB), ("grad", CH_GRAD)):
            n = int(s[N_CH * W + ch])
            if n:
                out[name] = float(s[ch * W:(ch + 1) * W].max()) / n / 1e6
        return out

    def table_storage(self):
        return None           # rows are pushed by their owner: the table arena itself need not be peer-visible

    def attach(self, emb_mod):
        self.emb_mod = emb_mod

    def check(self):
        """Raise if a bounded wait timed out or a window overflowed (one host read; call at step boundaries / in tests)."""
        s = int(self.status.item())
        if s & STATUS_TIMEOUT:
            raise RuntimeError("fused exchange: a peer did not signal within the wait limit (rank missing or stalled)")
        if s & STATUS_OVERFLOW:
            raise RuntimeError("fused exchange: receive window overflow; raise exchange_capacity / RECIS_EXCHANGE_CAPACITY")

    def _head_for(self, store):
        cap = store.capacity()
        if self._head is None or self._head.numel() < cap:
            self._head = torch.full((cap,), -1, dtype=torch.int32, device=self.device)
        return self._head

    # ------------------------------------------------------------------ forward
    def forward(self, emb_mod, lane_key, ids, offsets, weights, combiner, tile_len, mode, perm_b, perm_f, train, readonly, threshold,
                step, prepared=None):
        with torch.profiler.record_function("recis_b200/exchange_forward"):
            return self._forward(emb_mod, lane_key, ids, offsets, weights, combiner, tile_len, mode, perm_b, perm_f, train, readonly,
                                 threshold, step, prepared)

    def prepare(self, emb_mod, lane_key, ids, train=True):
        """Requester half of the id phase only (dedup + bucket into the window, signal IDS). A model with several (table, runtime
        group) pairs calls this for all of them before the first ``forward``: every rank's ids are then on offer before anybody
        waits, as the reference issues all of its id all-to-alls before the first wait
        (``recis/nn/modules/embedding_engine.py:739-801``). Pass the result to ``serve`` and / or ``forward(..., prepared=...)``."""
        with torch.profiler.record_function("recis_b200/exchange_prepare"):
            lane, e, rev = self._begin(emb_mod, lane_key, ids)
            return {"lane": lane, "e": e, "rev": rev, "served": None}

    def serve(self, emb_mod, prepared, readonly, threshold, step):
        """Owner half of a prepared lookup: wait for the ids, pull them, look the rows up (inserting unless ``readonly``), push
        them to the requesters and signal EMB - without waiting for the other owners. Calling this for all groups before the
        first ``forward`` leaves one rank-wide synchronisation point for the embedding phase of the whole model instead of one
        per group."""
        with torch.profiler.record_function("recis_b200/exchange_serve"):
            prepared["served"] = self._serve(emb_mod, prepared["lane"], prepared["e"], readonly, threshold, step)
            self.staged_serves += 1
        return prepared

    def _begin(self, emb_mod, lane_key, ids):
        C = native()
        lane = self.lanes.get(lane_key)
        if lane is None:                       # collective: every rank meets here at its first forward of this lane
            lane = self.lanes[lane_key] = _Lane(self, ids.numel())
        if lane.pending_grad_epoch and not self.immediate_reduce:
            # the previous backward of this lane is still staged (gradient accumulation without set_grad_accum_steps):
            # consume it now, before this step's backward rewrites the gradient window
            self._flush_pending(emb_mod.impl, lane)
        h = lane.heap
        lane.epoch += 1
        e = lane.epoch
        if ids.numel() > lane.send_cap and not lane.warned:
            # the id count bounds the unique count from above: beyond the capacity an overflow becomes possible (not certain)
            lane.warned = True
            import warnings
            warnings.warn(f"fused exchange '{lane_key}': a batch of {ids.numel()} ids meets windows sized for {lane.send_cap} unique ids per "
                          "rank; if more of them are distinct the step is flagged as an overflow (raise exchange_capacity / "
                          "RECIS_EXCHANGE_CAPACITY)", RuntimeWarning, stacklevel=3)
        # more unique ids than the window holds sets the overflow bit in self.status (see check()); nothing is written out of bounds
        _uniq, rev, _counts, _offs = C.dedup_partition(ids, self.world, h["ids"].tensor, h["offsets"].tensor, self.status)
        C.comm_signal(h["flags"].ptrs, CH_IDS, self.rank, e, self.host)
        return lane, e, rev

    def _serve(self, emb_mod, lane, e, readonly, threshold, step):
        C = native()
        h, me = lane.heap, self.rank
        store = emb_mod.impl.store
        count_admit = (not readonly) and threshold > 1
        if count_admit:
            # The tail past this step's ids must not hold ids of earlier steps (see below). It is filled with -2, the table's
            # tombstone value: the dedup treats it as one ordinary key (one claim, then plain re-reads of one cell), the table
            # ignores it. (-1, the dedup's own reserved key, would send every tail element through one atomic.)
            lane.ids_in.fill_(-2)
        tok = span_open("ids")
        self._wait(h["flags"].tensor, CH_IDS, e)
        C.comm_pull_ids(h["ids"].ptrs, h["offsets"].ptrs, me, lane.ids_in, lane.prefix, lane.n_in, self.status)
        span_close(tok)
        if self.multi_stream and self._store_event is not None:
            # lanes on separate streams share one table: its lookups (which allocate rows) run one after the other
            torch.cuda.current_stream(self.device).wait_event(self._store_event)
        if readonly:
            rows_in = store.find(lane.ids_in, lane.n_in)
        elif count_admit:
            # Count-based admission counts ONE sighting per id and step, whoever asks (as a single rank and the collective
            # exchange do, where the owner dedups first): the incoming ids are deduplicated before the table sees them. The whole
            # window goes through the dedup (its size is fixed, the valid count lives on the device); the tail is one more "id"
            # that resolves to no row.
            o_uniq, o_rev, _c, o_offs = C.dedup_partition(lane.ids_in, 1)
            o_rows = store.lookup_or_insert(o_uniq, o_offs[1:2], step, threshold)
            rows_in = o_rows[o_rev.long()].contiguous()
        else:
            rows_in = store.lookup_or_insert(lane.ids_in, lane.n_in, step, threshold)
        if self.multi_stream:
            self._store_event = torch.cuda.Event()
            self._store_event.record(torch.cuda.current_stream(self.device))
        prefix = lane.prefix.clone()
        # the offsets window is rewritten by this lane's next forward; the backward needs this step's boundaries
        offsets_now = h["offsets"].tensor.clone()
        tok = span_open("emb")
        C.comm_push_emb(store.emb(), rows_in, prefix, h["uemb"].ptrs, me, lane.in_cap)
        C.comm_signal(h["flags"].ptrs, CH_EMB, me, e, self.host)
        span_close(tok)
        return rows_in, prefix, offsets_now

    def _forward(self, emb_mod, lane_key, ids, offsets, weights, combiner, tile_len, mode, perm_b, perm_f, train, readonly, threshold,
                 step, prepared=None):
        C = native()
        if prepared is None:
            lane, e, rev = self._begin(emb_mod, lane_key, ids)
            served = None
        else:
            lane, e, rev, served = prepared["lane"], prepared["e"], prepared["rev"], prepared["served"]
        if served is None:
            served = self._serve(emb_mod, lane, e, readonly, threshold, step)
        rows_in, prefix, offsets_now = served
        h, D = lane.heap, self.D
        tok = span_open("emb")
        self._wait(h["flags"].tensor, CH_EMB, e)
        span_close(tok)
        uemb = h["uemb"].tensor.view(lane.send_cap, D)
        if combiner == "tile":
            out, gsrc, gscale = C.tile_forward(uemb, None, rev, offsets, weights, tile_len, train)
        else:
            out, gsrc, gscale = C.pool_forward(uemb, None, rev, offsets, weights, mode, perm_b, perm_f, train)
        saved = dict(rev=rev, gsrc=gsrc, gscale=gscale, rows_in=rows_in, prefix=prefix, epoch=e, lane=lane,
                     offsets=offsets_now) if train else None
        if train:
            lane.last_train_epoch = e
        return out, saved

    # ------------------------------------------------------------------ backward (requester side) + staging
    def backward(self, emb_mod, s, grad_out, worker_scale):
        with torch.profiler.record_function("recis_b200/exchange_backward"):
            self._backward(emb_mod, s, grad_out, worker_scale)

    def _backward(self, emb_mod, s, grad_out, worker_scale):
        C = native()
        lane = s["lane"]
        if s["epoch"] != lane.last_train_epoch:
            # A newer TRAINING forward of this (table, runtime group) owns the lane's gradient window and flag epochs now: this
            # older forward's gradients can no longer be exchanged through them (a read-only forward in between is harmless).
            # Every rank gets here in the same step.
            raise RuntimeError(
                "fused exchange: the same feature group of a table was looked up again before the gradients of an earlier lookup "
                "were back-propagated (two training lookups per step share one set of exchange windows); call the embedding "
                "engine once per step for these features, or run with RECIS_COMM=nccl")
        h, me, D = lane.heap, self.rank, self.D
        csr_u, csr_elem, start = C.build_csr(s["rev"])
        tok = span_open("grad_push")
        C.comm_grad_reduce_push(grad_out, s["gsrc"], s["gscale"], csr_u, csr_elem, start, D, s["offsets"], s["prefix"],
                                h["gin"].ptrs, lane.in_cap)
        C.comm_signal(h["flags"].ptrs, CH_GRAD, me, s["epoch"], self.host)
        span_close(tok)
        rec = dict(rows_in=s["rows_in"], prefix=s["prefix"], epoch=s["epoch"], scale=worker_scale, exchange=self, lane=lane,
                   mean_by_id=emb_mod.option.grad_reduce_by == "id",
                   stream=torch.cuda.current_stream(self.device) if self.multi_stream else None)
        if self.immediate_reduce:
            rows, grads = self.owner_reduce(emb_mod.impl, rec, apply=False)
            emb_mod.impl.accept_grad(rows, grads)
        else:
            rec["kind"] = "peer"
            lane.pending_grad_epoch = s["epoch"]
            emb_mod.impl.records().append(rec)

    def _flush_pending(self, impl, lane):
        keep = []
        for rec in impl.records():
            if rec.get("kind") == "peer" and rec["lane"] is lane:
                rows, grads = self.owner_reduce(impl, rec, apply=False)
                keep.append({"kind": "rows", "rows": rows, "grad": grads})
            else:
                keep.append(rec)
        impl.records()[:] = keep

    # ------------------------------------------------------------------ owner side: pull + reduce (+ update)
    def owner_reduce(self, impl, rec, apply, kind=2, lr=0.0, b1=0.0, b2=0.0, eps=0.0, decay=1.0, alpha=0.0, grad_scale=1.0,
                     w=None, s1=None, s2=None):
        with torch.profiler.record_function("recis_b200/owner_reduce_update"):
            return self._owner_reduce(impl, rec, apply, kind, lr, b1, b2, eps, decay, alpha, grad_scale, w, s1, s2)

    def _owner_reduce(self, impl, rec, apply, kind, lr, b1, b2, eps, decay, alpha, grad_scale, w, s1, s2):
        C = native()
        lane = rec["lane"]
        h = lane.heap
        tok = span_open("grad_wait")
        self._wait(h["flags"].tensor, CH_GRAD, rec["epoch"])
        span_close(tok)
        head = self._head_for(impl.store)
        rows, grads = C.comm_owner_reduce(rec["rows_in"], head, rec["prefix"], h["gin"].tensor, self.world, self.D,
                                          rec["mean_by_id"], apply, kind, lr, b1, b2, eps, decay, alpha, rec["scale"] * grad_scale,
                                          w, s1, s2, lane.in_cap, self.owner_unroll)
        if lane.pending_grad_epoch == rec["epoch"]:
            lane.pending_grad_epoch = 0
        return rows, grads
