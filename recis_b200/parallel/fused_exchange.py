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

No split size ever reaches the host. The same code drives CPU ranks of one machine (``RECIS_COMM=fused`` with CPU tables):
the windows then live in POSIX shared memory and the kernels' host twins (``csrc/cpu/cpu_comm.cc``) do the work - the
oracle of this path in the multi-rank tests.

Lanes. Every (table, runtime group, lane) owns its own windows, flag pad and epoch counter, so that the epochs written to a
flag only ever grow and a gradient window is never rewritten before its owner consumed it. A runtime group with several
features can be split into lanes (``forward_group``): a lane is a set of features that share no table row with the other
lanes, and the lanes run as a software pipeline over two CUDA streams chosen by the resource a kernel is bound by - the
NVLink-bound kernels (row push, gradient push) of every lane go to a *link stream* with small grids, everything else (dedup,
table lookup, pooling, owner update) stays on the model's stream - so that lane i's transfer runs under lane i+1's
memory-bound work instead of in front of it.

Windows. They are sized from the first batch (the unique counts per owner are measured once, at lane creation, which is a
collective anyway) with half as much again on top, and they grow: every owner sees all requesters' counts, so every rank
computes the same "largest demand so far" on the device; that number comes back to the host asynchronously and is looked at
``GROW_LAG`` steps later, by which time it has long landed, so all ranks take the same decision at the same step without a
collective or a stall. A window that turns out too small anyway drops ids, never memory safety: the kernels clamp every
published boundary, set a status bit, and ``check()`` raises. ``RECIS_EXCHANGE_STRICT=1`` reads the demand of every step
before it is used (one host read per lookup) and repeats the id phase with larger windows instead of dropping anything.
All flag waits are time-bounded; a timeout sets a bit in ``status`` which ``check()`` turns into an exception.
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
GROW_LAG = 2            # steps between a demand measurement on the device and the host acting on it
GROW_RING = 4           # pinned slots the measurements come back through (> GROW_LAG)
GROW_AT = 0.8           # grow when the demand exceeds this fraction of a window
HEADROOM = 1.5          # new size = demand * HEADROOM


# element size of the row types the exchange carries; the wire format of a row is its storage format
_ROW_BYTES = {torch.float32: 4, torch.float16: 2, torch.bfloat16: 2, torch.int8: 1}


def _round_up(x: int, q: int = 1024) -> int:
    return (int(x) + q - 1) // q * q


class _Lane:
    """Windows + flags of one (table, runtime group, lane)."""

    def __init__(self, ex: "FusedExchange", ids: torch.Tensor):
        self.ex = ex
        W = ex.world
        # Every rank must lay its windows out identically (peers address them by offset). The sizes are agreed on here, once:
        # each rank measures what its first batch sends to every owner, the W x W matrix is gathered, and the largest row sum
        # (ids one requester sends) and column sum (ids one owner receives) size the windows.
        C = native()
        _u, _r, counts, _o = C.dedup_partition(ids, W)
        mine = counts.to(torch.int64)
        rows = [torch.zeros_like(mine) for _ in range(W)]
        dist.all_gather(rows, mine, group=ex.pg)
        m = torch.stack(rows).cpu()
        need_out, need_in = int(m.sum(1).max()), int(m.sum(0).max())
        want = torch.tensor([ex.send_cap], dtype=torch.int64, device=ex.device)
        dist.all_reduce(want, op=dist.ReduceOp.MAX, group=ex.pg)
        explicit = int(want.item())
        if explicit:
            cap = explicit
            in_cap = max(cap, min(W * cap, _round_up(need_in * HEADROOM)))
        else:
            cap = _round_up(max(need_out * HEADROOM, 1024))
            in_cap = _round_up(max(need_in * HEADROOM, 1024))
        self.warned = False
        self.grown = 0
        self.heap = None
        self.native = None               # the C++ twin of this object: windows, peer pointers, counters, demand ring
        self.children = None             # child tables this lane's ids belong to (None: unknown)
        self._alloc(cap, in_cap)

    def _alloc(self, cap: int, in_cap: int):
        ex = self.ex
        W, D = ex.world, ex.D
        self.send_cap, self.in_cap = int(cap), int(in_cap)
        self.heap = SymmetricHeap({
            "flags": (torch.int64, N_CH * W),
            "offsets": (torch.int32, W + 1),
            "counts": (torch.int32, W),
            "ids": (torch.int64, self.send_cap),
            "uemb": (ex.opt.dtype, self.send_cap * D),
            "gin": (torch.float32, self.in_cap * D),
        }, ex.device, ex.pg)
        counters = (0, 0, 0, 0) if self.native is None else (self.epoch, self.steps, self.last_train_epoch, self.pending_grad_epoch)
        h = self.heap
        self.native = native().ExLane(W, ex.rank, D, self.send_cap, self.in_cap, {k: h[k].tensor for k in h.regions},
                                      {k: h[k].ptrs for k in h.regions})
        self.epoch, self.steps, self.last_train_epoch, self.pending_grad_epoch = counters     # flag epochs only ever grow
        self.ids_in, self.n_in, self.demand = self.native.ids_in, self.native.n_in, self.native.demand
        self.prefix = torch.zeros(4 * W + 2, dtype=torch.int32, device=ex.device)

    # counters shared with the native executor
    epoch = property(lambda self: self.native.epoch, lambda self, v: setattr(self.native, "epoch", int(v)))
    steps = property(lambda self: self.native.steps, lambda self, v: setattr(self.native, "steps", int(v)))
    last_train_epoch = property(lambda self: self.native.last_train_epoch, lambda self, v: setattr(self.native, "last_train_epoch", int(v)))
    pending_grad_epoch = property(lambda self: self.native.pending_grad_epoch,
                                  lambda self, v: setattr(self.native, "pending_grad_epoch", int(v)))

    # ---- demand mirror: the device's "largest demand so far" comes back without anybody waiting for it
    def post_demand(self):
        self.native.post_demand()

    def demand_of(self, step: int):
        """(out, in) demand as measured at lookup ``step`` of this lane, or None when that slot has been reused."""
        d = self.native.demand_of(int(step))
        return None if d[0] < 0 else d

    def grow(self, need_out: int, need_in: int):
        """Collective: every rank calls this at the same lookup with the same numbers. Nothing of this lane is in flight when the
        old windows go: the device is drained first and the peers' mappings are closed before the memory is freed."""
        ex = self.ex
        cap = max(self.send_cap, _round_up(need_out * HEADROOM)) if need_out > GROW_AT * self.send_cap else self.send_cap
        in_cap = max(self.in_cap, _round_up(need_in * HEADROOM)) if need_in > GROW_AT * self.in_cap else self.in_cap
        if ex.device.type == "cuda":
            torch.cuda.synchronize(ex.device)
        dist.barrier(group=ex.pg)
        old = self.heap
        self._alloc(cap, in_cap)                  # ends with a barrier: every rank has mapped the new windows
        old.close()
        dist.barrier(group=ex.pg)                 # every rank has unmapped my old windows
        del old
        self.grown += 1


class FusedExchange:
    @staticmethod
    def create(emb_opt, pg, world, rank):
        if emb_opt.dtype not in _ROW_BYTES or emb_opt.embedding_dim % 4 != 0 or emb_opt.embedding_dim > 512:
            return None
        if (emb_opt.embedding_dim * _ROW_BYTES[emb_opt.dtype]) % 16 != 0:
            return None                  # rows travel in 16-byte pieces
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
        self.owner_unroll = int(os.environ.get("RECIS_OWNER_UNROLL", "2"))
        # RECIS_WAIT_STATS=1: flag waits go through the accounting kernel; wait_stats holds nanoseconds per (channel, peer)
        self.wait_stats = (torch.zeros(N_CH * world + N_CH, dtype=torch.int64, device=self.device)
                           if os.environ.get("RECIS_WAIT_STATS") == "1" else None)
        self._head = None
        # RECIS_STAGE_EXCHANGE=1: the engine may issue the id phase of all of a model's groups before the first wait (prepare())
        self.stage_enabled = os.environ.get("RECIS_STAGE_EXCHANGE") == "1"
        self.staged_serves = 0             # how many lookups had their owner side issued ahead of the first wait (serve())
        self.strict = os.environ.get("RECIS_EXCHANGE_STRICT") == "1" or bool(getattr(emb_opt, "exchange_strict", False))
        # grid caps of the two NVLink-bound kernels when they run on the link stream next to other work (0: fill the GPU)
        self.push_blocks = int(os.environ.get("RECIS_PUSH_BLOCKS", "296"))
        self.grad_push_blocks = int(os.environ.get("RECIS_GRAD_PUSH_BLOCKS", "592"))
        self._link = None                  # the link stream (created with the first multi-lane lookup)
        # RECIS_EXCHANGE_NATIVE=0 issues the lane pipeline from Python instead of the native executor (same launches, same order)
        self.native_executor = os.environ.get("RECIS_EXCHANGE_NATIVE", "1") != "0"
        # lane key -> frozenset of child-table indices whose rows the lane can touch (set by the engine); two staged gradient
        # records may be applied one after the other only when their lanes are known to share no row
        self.lane_children = {}

    # ------------------------------------------------------------------ small helpers
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
                out[name + "_waits"] = n
        return out

    def table_storage(self):
        return None           # rows are pushed by their owner: the table arena itself need not be peer-visible

    def attach(self, emb_mod):
        self.emb_mod = emb_mod

    def check(self):
        """Raise if a bounded wait timed out or a window overflowed (one host read; call at step boundaries / in tests). The
        overflow bit is cleared by the report: the windows have grown (or will, from the recorded demand), so a caller that
        chooses to go on is told once per incident, not forever."""
        s = int(self.status.item())
        if s & STATUS_TIMEOUT:
            raise RuntimeError("fused exchange: a peer did not signal within the wait limit (rank missing or stalled)")
        if s & STATUS_OVERFLOW:
            self.status.bitwise_and_(~STATUS_OVERFLOW)
            raise RuntimeError("fused exchange: receive window overflow (ids were dropped in an earlier step); the windows grow from "
                               "the measured demand, raise exchange_capacity / RECIS_EXCHANGE_CAPACITY or set RECIS_EXCHANGE_STRICT=1 "
                               "to rule it out")

    def window_bytes(self) -> int:
        return sum(l.heap.nbytes for l in self.lanes.values())

    def _head_for(self, store):
        cap = store.capacity()
        if self._head is None or self._head.numel() < cap:
            self._head = torch.full((cap,), -1, dtype=torch.int32, device=self.device)
        return self._head

    def _link_stream(self):
        if self._link is None:
            self._link = torch.cuda.Stream(device=self.device)
        return self._link

    # ------------------------------------------------------------------ forward, one lane
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
            return {"lane": lane, "e": e, "rev": rev, "served": None, "ids": ids, "key": lane_key}

    def serve(self, emb_mod, prepared, readonly, threshold, step):
        """Owner half of a prepared lookup: wait for the ids, pull them, look the rows up (inserting unless ``readonly``), push
        them to the requesters and signal EMB - without waiting for the other owners. Calling this for all groups before the
        first ``forward`` leaves one rank-wide synchronisation point for the embedding phase of the whole model instead of one
        per group."""
        with torch.profiler.record_function("recis_b200/exchange_serve"):
            prepared["served"] = self._serve(emb_mod, prepared, readonly, threshold, step)
            self.staged_serves += 1
        return prepared

    def _lane(self, lane_key, ids):
        lane = self.lanes.get(lane_key)
        if lane is None:                       # collective: every rank meets here at its first forward of this lane
            lane = self.lanes[lane_key] = _Lane(self, ids)
            lane.children = self.lane_children.get(lane_key)
        return lane

    def _begin(self, emb_mod, lane_key, ids):
        C = native()
        lane = self._lane(lane_key, ids)
        if lane.pending_grad_epoch and not self.immediate_reduce:
            # the previous backward of this lane is still staged (gradient accumulation without set_grad_accum_steps):
            # consume it now, before this step's backward rewrites the gradient window
            self._flush_pending(emb_mod.impl, lane)
        if not self.strict:
            # the demand measured GROW_LAG lookups ago (the same number on every rank): grow before the windows get tight
            d = lane.demand_of(lane.steps - GROW_LAG)
            if d is not None and (d[0] > GROW_AT * lane.send_cap or d[1] > GROW_AT * lane.in_cap):
                lane.grow(d[0], d[1])
        h = lane.heap
        lane.epoch += 1
        e = lane.epoch
        # more unique ids than the window holds sets the overflow bit in self.status (see check()); the published boundaries are
        # clamped, nothing is written out of bounds
        _uniq, rev, _counts, _offs = C.dedup_partition(ids, self.world, h["ids"].tensor, h["offsets"].tensor, self.status,
                                                       h["counts"].tensor)
        C.comm_signal(h["flags"].ptrs, CH_IDS, self.rank, e, self.host)
        return lane, e, rev

    def _pull(self, lane, e, count_admit):
        """Owner: wait for every requester's ids of epoch ``e`` and gather the ones bucketed for this rank."""
        C = native()
        h = lane.heap
        if count_admit:
            # The tail past this step's ids must not hold ids of earlier steps (see _lookup). It is filled with -2, the table's
            # tombstone value: the dedup treats it as one ordinary key (one claim, then plain re-reads of one cell), the table
            # ignores it. (-1, the dedup's own reserved key, would send every tail element through one atomic.)
            lane.ids_in.fill_(-2)
        tok = span_open("ids")
        self._wait(h["flags"].tensor, CH_IDS, e)
        C.comm_pull_ids(h["ids"].ptrs, h["offsets"].ptrs, h["counts"].ptrs, self.rank, lane.ids_in, lane.prefix, lane.n_in, lane.demand,
                        self.status)
        span_close(tok)
        lane.post_demand()
        lane.steps += 1

    def _lookup(self, emb_mod, lane, readonly, threshold, step):
        C = native()
        store = emb_mod.impl.store
        count_admit = (not readonly) and threshold > 1
        if readonly:
            rows_in = store.find(lane.ids_in, lane.n_in)
        elif count_admit:
            # Count-based admission counts ONE sighting per id and step, whoever asks (as a single rank and the collective
            # exchange do, where the owner dedups first): the incoming ids are deduplicated before the table sees them. The whole
            # window goes through the dedup (its size is fixed, the valid count lives on the device); the tail is one more "id"
            # that resolves to no row.
            o_uniq, o_rev, _c, o_offs = C.dedup_partition(lane.ids_in, 1)
            o_rows = store.lookup_or_insert(o_uniq, o_offs[1:2], step, threshold, True)
            rows_in = o_rows[o_rev.long()].contiguous()
        else:
            rows_in = store.lookup_or_insert(lane.ids_in, lane.n_in, step, threshold)
        return rows_in

    def _id_phase(self, emb_mod, prepared, readonly, threshold, step):
        """Owner: ids in, rows looked up. In strict mode the demand of THIS lookup is read first and, when a window is too
        small, the windows grow and the requester half is repeated (nothing was consumed yet), on every rank alike."""
        lane, e = prepared["lane"], prepared["e"]
        count_admit = (not readonly) and threshold > 1
        self._pull(lane, e, count_admit)
        if self.strict:
            for _ in range(4):
                need_out, need_in = (int(x) for x in lane.demand.cpu())
                if need_out <= lane.send_cap and need_in <= lane.in_cap:
                    break
                lane.grow(max(need_out, 1), max(need_in, 1))
                self.status.bitwise_and_(~STATUS_OVERFLOW)
                lane2, e2, rev2 = self._begin(emb_mod, prepared["key"], prepared["ids"])
                prepared.update(lane=lane2, e=e2, rev=rev2)
                lane, e = lane2, e2
                self._pull(lane, e, count_admit)
        rows_in = self._lookup(emb_mod, lane, readonly, threshold, step)
        prefix = lane.prefix.clone()
        # the offsets window is rewritten by this lane's next forward; the backward needs this step's boundaries, which the pull
        # kernel copied behind the prefix sums
        offsets_now = prefix[3 * self.world + 1:]
        return rows_in, prefix, offsets_now

    def _push(self, emb_mod, lane, e, rows_in, prefix, blocks=0):
        C = native()
        h = lane.heap
        tok = span_open("emb")
        C.comm_push_emb(emb_mod.impl.store.emb(), rows_in, prefix, h["uemb"].ptrs, self.rank, lane.in_cap, blocks)
        C.comm_signal(h["flags"].ptrs, CH_EMB, self.rank, e, self.host)
        span_close(tok)

    def _serve(self, emb_mod, prepared, readonly, threshold, step):
        rows_in, prefix, offsets_now = self._id_phase(emb_mod, prepared, readonly, threshold, step)
        self._push(emb_mod, prepared["lane"], prepared["e"], rows_in, prefix)
        return rows_in, prefix, offsets_now

    def _forward(self, emb_mod, lane_key, ids, offsets, weights, combiner, tile_len, mode, perm_b, perm_f, train, readonly, threshold,
                 step, prepared=None):
        C = native()
        if prepared is None:
            lane, e, rev = self._begin(emb_mod, lane_key, ids)
            prepared = {"lane": lane, "e": e, "rev": rev, "served": None, "ids": ids, "key": lane_key}
        if prepared["served"] is None:
            prepared["served"] = self._serve(emb_mod, prepared, readonly, threshold, step)
        lane, e, rev = prepared["lane"], prepared["e"], prepared["rev"]
        rows_in, prefix, offsets_now = prepared["served"]
        h, D = lane.heap, self.D
        tok = span_open("emb")
        self._wait(h["flags"].tensor, CH_EMB, e)
        span_close(tok)
        uemb = h["uemb"].tensor.view(lane.send_cap, D)
        if combiner == "tile":
            out, gsrc, gscale = C.tile_forward(uemb, None, rev, offsets, weights, tile_len, train)
        else:
            out, gsrc, gscale = C.pool_forward(uemb, None, rev, offsets, weights, mode, perm_b, perm_f, train)
        saved = dict(rev=rev, gsrc=gsrc, gscale=gscale, rows_in=rows_in, prefix=prefix, epoch=e, lane=lane, heap=h,
                     offsets=offsets_now) if train else None
        if train:
            lane.last_train_epoch = e
        return out, saved

    # ------------------------------------------------------------------ forward, several lanes of one runtime group
    def forward_group(self, emb_mod, parts, mode, perm_b, perm_total, n_rows, train, readonly, threshold, step):
        """Lookup of one runtime group split into lanes. ``parts``: one dict per lane with ``key``, ``ids``, ``offsets``,
        ``weights``, and where its pooled rows go in the shared output: ``perm_f`` features starting at feature ``perm_off`` of a
        ``[perm_b, perm_total, D]`` cube (interleaved layout), or ``n_seg`` rows starting at row ``perm_off`` (plain layout,
        ``perm_total == 0``). Returns the shared output ``[n_rows, D]`` and what the backward needs.

        Launch order: the requester half of lane i+1 is issued before the owner half of lane i waits for its ids; every lane's
        row push goes to the link stream behind an event; the pooling of all lanes follows on the model's stream. On CPU ranks
        there are no streams and the same calls simply run in this order."""
        with torch.profiler.record_function("recis_b200/exchange_forward_group"):
            C = native()
            D = self.D
            cuda = not self.host
            if not self.strict and self.native_executor:
                return self._forward_group_native(emb_mod, parts, mode, perm_b, perm_total, n_rows, train, readonly, threshold, step)
            main = torch.cuda.current_stream(self.device) if cuda else None
            link = self._link_stream() if cuda and len(parts) > 1 else None
            out = torch.empty(n_rows, D, dtype=torch.float32, device=self.device)
            preps = [None] * len(parts)
            p0 = parts[0]
            lane, e, rev = self._begin(emb_mod, p0["key"], p0["ids"])
            preps[0] = {"lane": lane, "e": e, "rev": rev, "served": None, "ids": p0["ids"], "key": p0["key"]}
            for i, part in enumerate(parts):
                if i + 1 < len(parts):
                    nxt = parts[i + 1]
                    lane, e, rev = self._begin(emb_mod, nxt["key"], nxt["ids"])
                    preps[i + 1] = {"lane": lane, "e": e, "rev": rev, "served": None, "ids": nxt["ids"], "key": nxt["key"]}
                pr = preps[i]
                rows_in, prefix, offsets_now = self._id_phase(emb_mod, pr, readonly, threshold, step)
                pr["served"] = (rows_in, prefix, offsets_now)
                if link is not None:
                    ev = torch.cuda.Event()
                    ev.record(main)
                    with torch.cuda.stream(link):
                        link.wait_event(ev)
                        self._push(emb_mod, pr["lane"], pr["e"], rows_in, prefix, self.push_blocks)
                else:
                    self._push(emb_mod, pr["lane"], pr["e"], rows_in, prefix)
            saved = []
            for part, pr in zip(parts, preps):
                lane, e, rev = pr["lane"], pr["e"], pr["rev"]
                h = lane.heap
                tok = span_open("emb")
                self._wait(h["flags"].tensor, CH_EMB, e)
                span_close(tok)
                uemb = h["uemb"].tensor.view(lane.send_cap, D)
                _o, gsrc, gscale = C.pool_forward(uemb, None, rev, part["offsets"], part["weights"], mode,
                                                  perm_b if perm_total else 0, part["perm_f"] if perm_total else 0, train, out,
                                                  part["perm_off"], perm_total)
                if train:
                    rows_in, prefix, offsets_now = pr["served"]
                    lane.last_train_epoch = e
                    saved.append(dict(rev=rev, gsrc=gsrc, gscale=gscale, rows_in=rows_in, prefix=prefix, epoch=e, lane=lane, heap=h,
                                      offsets=offsets_now))
            return out, (saved if train else None)

    def _forward_group_native(self, emb_mod, parts, mode, perm_b, perm_total, n_rows, train, readonly, threshold, step):
        """The same launch order issued by ONE native call (``csrc/bind/bind_exchange.cpp``); growth decisions stay here."""
        C = native()
        lanes = []
        for part in parts:
            lane = self._lane(part["key"], part["ids"])
            if lane.pending_grad_epoch and not self.immediate_reduce:
                self._flush_pending(emb_mod.impl, lane)
            d = lane.demand_of(lane.steps - GROW_LAG)
            if d is not None and (d[0] > GROW_AT * lane.send_cap or d[1] > GROW_AT * lane.in_cap):
                lane.grow(d[0], d[1])
            lanes.append(lane)
        link = self._link_stream().cuda_stream if (not self.host and len(parts) > 1) else 0
        out, saved_t, epochs = C.exchange_forward_group(
            [l.native for l in lanes], emb_mod.impl.store, [p["ids"] for p in parts], [p["offsets"] for p in parts],
            [p["weights"] for p in parts], [int(p["perm_f"]) for p in parts], [int(p["perm_off"]) for p in parts], mode, perm_b,
            perm_total, n_rows, train, readonly, threshold, step, self.status, self.wait_us, self.wait_stats, link, self.push_blocks)
        if not train:
            return out, None
        W = self.world
        saved = [dict(rev=t[0], gsrc=t[1], gscale=t[2], rows_in=t[3], prefix=t[4], offsets=t[4][3 * W + 1:], epoch=e, lane=lane,
                      heap=lane.heap) for t, e, lane in zip(saved_t, epochs, lanes)]
        return out, saved

    # ------------------------------------------------------------------ backward (requester side) + staging
    def backward(self, emb_mod, s, grad_out, worker_scale):
        with torch.profiler.record_function("recis_b200/exchange_backward"):
            if isinstance(s, list):
                self._backward_group(emb_mod, s, grad_out, worker_scale)
            else:
                self._backward(emb_mod, s, grad_out, worker_scale)

    def _check_epoch(self, s):
        lane = s["lane"]
        if s["epoch"] != lane.last_train_epoch or s["heap"] is not lane.heap:
            # A newer TRAINING forward of this (table, runtime group) owns the lane's gradient window and flag epochs now: this
            # older forward's gradients can no longer be exchanged through them (a read-only forward in between is harmless).
            # Every rank gets here in the same step.
            raise RuntimeError(
                "fused exchange: the same feature group of a table was looked up again before the gradients of an earlier lookup "
                "were back-propagated (two training lookups per step share one set of exchange windows); call the embedding "
                "engine once per step for these features, or run with RECIS_COMM=nccl")

    def _grad_push(self, s, grad_out, csr, blocks=0):
        C = native()
        lane, h = s["lane"], s["heap"]
        csr_u, csr_elem, start = csr
        tok = span_open("grad_push")
        C.comm_grad_reduce_push(grad_out, s["gsrc"], s["gscale"], csr_u, csr_elem, start, self.D, s["offsets"], s["prefix"],
                                h["gin"].ptrs, lane.in_cap, blocks)
        C.comm_signal(h["flags"].ptrs, CH_GRAD, self.rank, s["epoch"], self.host)
        span_close(tok)

    def _stage(self, emb_mod, s, worker_scale):
        lane = s["lane"]
        rec = dict(rows_in=s["rows_in"], prefix=s["prefix"], epoch=s["epoch"], scale=worker_scale, exchange=self, lane=lane,
                   heap=s["heap"], mean_by_id=emb_mod.option.grad_reduce_by == "id", children=lane.children)
        if self.immediate_reduce:
            rows, grads = self.owner_reduce(emb_mod.impl, rec, apply=False)
            emb_mod.impl.accept_grad(rows, grads)
        else:
            rec["kind"] = "peer"
            lane.pending_grad_epoch = s["epoch"]
            emb_mod.impl.records().append(rec)

    def _backward(self, emb_mod, s, grad_out, worker_scale):
        self._check_epoch(s)
        csr = native().build_csr(s["rev"])
        self._grad_push(s, grad_out, csr)
        self._stage(emb_mod, s, worker_scale)

    def _backward_group(self, emb_mod, saved, grad_out, worker_scale):
        """Backward of ``forward_group``: per lane, the element sort stays on the model's stream and the NVLink-bound reduce + push
        goes to the link stream, so that lane i's push runs under lane i+1's sort and, later, under lane i-1's owner update."""
        for s in saved:
            self._check_epoch(s)
        C = native()
        cuda = not self.host
        if self.native_executor:
            link = self._link_stream().cuda_stream if (cuda and len(saved) > 1) else 0
            C.exchange_backward_group([s["lane"].native for s in saved],
                                      [[s["rev"], s["gsrc"], s["gscale"], s["rows_in"], s["prefix"]] for s in saved],
                                      [int(s["epoch"]) for s in saved], grad_out, self.status, link, self.grad_push_blocks)
            for s in saved:
                self._stage(emb_mod, s, worker_scale)
            return
        link = self._link_stream() if cuda and len(saved) > 1 else None
        main = torch.cuda.current_stream(self.device) if cuda else None
        if link is not None:
            grad_out.record_stream(link)
        for s in saved:
            csr = C.build_csr(s["rev"])
            if link is not None:
                ev = torch.cuda.Event()
                ev.record(main)
                for t in (*csr, s["gsrc"], s["gscale"], s["offsets"], s["prefix"]):
                    t.record_stream(link)
                with torch.cuda.stream(link):
                    link.wait_event(ev)
                    self._grad_push(s, grad_out, csr, self.grad_push_blocks)
            else:
                self._grad_push(s, grad_out, csr)
            self._stage(emb_mod, s, worker_scale)

    def _flush_pending(self, impl, lane):
        keep = []
        for rec in impl.records():
            if rec.get("kind") == "peer" and rec["lane"] is lane:
                rows, grads = self.owner_reduce(impl, rec, apply=False)
                keep.append({"kind": "rows", "rows": rows, "grad": grads})
            else:
                keep.append(rec)
        impl.records()[:] = keep

    # ------------------------------------------------------------------ owner side: reduce (+ update)
    def owner_reduce(self, impl, rec, apply, kind=2, lr=0.0, b1=0.0, b2=0.0, eps=0.0, decay=1.0, alpha=0.0, grad_scale=1.0,
                     w=None, s1=None, s2=None):
        with torch.profiler.record_function("recis_b200/owner_reduce_update"):
            return self._owner_reduce(impl, rec, apply, kind, lr, b1, b2, eps, decay, alpha, grad_scale, w, s1, s2)

    def _owner_reduce(self, impl, rec, apply, kind, lr, b1, b2, eps, decay, alpha, grad_scale, w, s1, s2):
        C = native()
        lane = rec["lane"]
        h = rec["heap"]
        tok = span_open("grad_wait")
        self._wait(h["flags"].tensor, CH_GRAD, rec["epoch"])
        span_close(tok)
        head = self._head_for(impl.store)
        rows, grads = C.comm_owner_reduce(rec["rows_in"], head, rec["prefix"], h["gin"].tensor, self.world, self.D,
                                          rec["mean_by_id"], apply, kind, lr, b1, b2, eps, decay, alpha, rec["scale"] * grad_scale,
                                          w, s1, s2, rec["rows_in"].numel(), self.owner_unroll)
        if lane.pending_grad_epoch == rec["epoch"]:
            lane.pending_grad_epoch = 0
        return rows, grads
