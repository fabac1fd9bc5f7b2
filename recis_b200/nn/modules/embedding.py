"""DynamicEmbedding: one row-sharded dynamic table with pooled lookup.

Public surface of the reference's ``recis/nn/modules/embedding.py:161-624`` (``EmbeddingOption``,
``DynamicEmbedding``). What one forward/backward does is the same: dedup ids and bucket them by owner shard
(owner = contiguous range of the 65536 slices selected by the low 16 id bits), owners look rows up (inserting
unknown ids while training), embeddings come back, the requester pools them (sum / mean / tile), and in
backward the per-unique gradients travel to the owners where duplicates across requesters are added and the
sparse optimizer later updates each touched row once.

How it is done differs:

* world size 1: no exchange at all; the pooling kernel reads rows straight out of the table arena and the
  backward pass only *stages* the pooled gradient, so that the optimizer step is one fused
  reduce-duplicates + update kernel (no per-unique gradient tensor is ever written).
* world size > 1, ``RECIS_COMM=fused`` (CUDA): the exchange runs inside our own kernels over peer-mapped
  memory (see ``recis_b200/parallel/fused_exchange.py``): no NCCL call and no host read of split sizes.
* world size > 1, collective path (``RECIS_COMM=nccl``, and always on CPU/gloo): the four
  ``all_to_all_single`` calls of the reference (counts, ids, embeddings, gradients). This is the measured
  baseline and the fallback.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional, Union

import torch
import torch.distributed as dist

from ... import native
from ...parallel.spans import span_close, span_open
from ...ragged.tensor import RaggedTensor
from ..hashtable_hook import AdmitHook, FilterHook
from ..initializers import ConstantInitializer, Initializer
from .hashtable import HashTable, gen_slice
from .hashtable_hook_impl import admit_params

_MODE = {"sum": 0, "mean": 1, "mean_weight": 2}


@dataclass
class EmbeddingOption:
    """Configuration of one (logical) embedding table. Field names and defaults follow the reference."""

    embedding_dim: int = 16
    block_size: int = 10240
    dtype: torch.dtype = torch.float32
    device: torch.device = None
    trainable: bool = True
    pg: "dist.ProcessGroup" = None
    max_partition_num: int = 65536
    shared_name: str = "embedding"
    children: List[str] = field(default_factory=list)
    coalesced: Optional[bool] = False
    initializer: Optional[Initializer] = None
    use_weight: Optional[bool] = True
    combiner: Optional[str] = "sum"
    combiner_kwargs: Optional[dict] = None
    grad_reduce_by: Optional[str] = "worker"
    filter_hook: Optional[FilterHook] = None
    admit_hook: Optional[AdmitHook] = None
    fp16_enabled: bool = False
    # additions
    capacity: int = 0            # rows to pre-size the shard for (0: grow on demand)
    mean_by_weight: bool = False  # "mean" divides by the weight sum instead of the bag length
    exchange_capacity: int = 0   # unique ids per rank and step the peer-memory exchange windows are sized for (0: measured on
                                 # the first batch, plus half as much again; the windows grow with the demand either way);
                                 # features merged into one table add up
    exchange_strict: bool = False  # read every step's window demand before using it (one host read per lookup) and repeat
                                   # the id phase with larger windows instead of ever dropping ids

    def __post_init__(self):
        if self.device is None:
            self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(self.device)
        if not self.children:
            self.children = [self.shared_name]
        if self.initializer is None:
            self.initializer = ConstantInitializer(init_val=0)
        if self.fp16_enabled:
            assert self.dtype in (torch.int8,), "only int8 emb can set fp16_enabled"
        if self.dtype not in (torch.float32, torch.float16, torch.bfloat16, torch.int8):
            # rows are stored in this dtype (optimizer state and accumulation stay fp32); int8 tables are read-only (filled by
            # insert() or a checkpoint) and are served as float16 (fp16_enabled) or float32, as the reference does
            # (recis/nn/modules/embedding.py:610-615)
            raise NotImplementedError(f"embedding dtype {self.dtype} is not supported (float32, float16, bfloat16, int8 are)")
        assert self.combiner in ("sum", "mean", "tile"), \
            f"Hashtable combiner only support [sum/mean/tile], but got {self.combiner}"
        assert self.grad_reduce_by in ("worker", "id")
        if self.combiner == "tile":
            if self.combiner_kwargs is None:
                raise RuntimeError("combiner_kwargs must be set when combiner is tile.")
            if "tile_len" not in self.combiner_kwargs:
                raise RuntimeError("tile_len must be in combiner_kwargs when combiner is tile.")

    def coalesced_info(self) -> str:
        import json
        return json.dumps({
            "dim": self.embedding_dim, "dtype": str(self.dtype), "device": str(self.device.type),
            "initializer": str(self.initializer), "grad_reduce_by": self.grad_reduce_by,
            "filter_hook": str(self.filter_hook),
        })

    def runtime_info(self) -> str:
        import json
        return json.dumps({
            "combiner": self.combiner, "use_weight": self.use_weight, "trainable": self.trainable,
            "admit_hook": str(self.admit_hook), "fp16_enabled": self.fp16_enabled,
            "combiner_kwargs": self.combiner_kwargs if self.combiner == "tile" else None,
            "mean_by_weight": self.mean_by_weight,
        })


def _a2a(out, inp, out_splits, in_splits, pg):
    dist.all_to_all_single(out, inp, out_splits, in_splits, group=pg)
    return out


class _LookupPoolFn(torch.autograd.Function):
    """ids/offsets/weights -> pooled embeddings; backward stages gradients on the owner table(s)."""

    @staticmethod
    def forward(ctx, holder, emb_mod: "DynamicEmbedding", ids, offsets, weights, combiner, tile_len, perm, training, admit_hook,
                lane="default", prepared=None):
        C = native()
        impl = emb_mod.impl
        store = impl.store
        W, pg = emb_mod.world_size, emb_mod.pg
        readonly, threshold = admit_params(admit_hook)
        train = training and impl.trainable and emb_mod.option.trainable
        if not (training and impl.trainable):
            readonly = True
        step = emb_mod.table.step_tensor() if not readonly else None
        mode = 0 if combiner != "mean" else (2 if emb_mod.option.mean_by_weight else 1)
        perm_b, perm_f = perm if perm is not None else (0, 0)
        ctx.train = train
        ctx.emb_mod = emb_mod
        D = impl.dim

        def pool(base, rows, rev):
            if combiner == "tile":
                return C.tile_forward(base, rows, rev, offsets, weights, tile_len, train)
            return C.pool_forward(base, rows, rev, offsets, weights, mode, perm_b, perm_f, train)

        if W == 1:
            uniq, rev, _counts, offs = C.dedup_partition(ids, 1)
            n_dev = offs[1:2]
            rows = store.find(uniq, n_dev) if readonly else store.lookup_or_insert(uniq, n_dev, step, threshold, True)
            out, gsrc, gscale = pool(store.emb(), rows, rev)
            if train:
                ctx.saved = dict(rev=rev, gsrc=gsrc, gscale=gscale, rows=rows)
            ctx.path = "local"
            return out

        if emb_mod.fused is not None:
            out, saved = emb_mod.fused.forward(emb_mod, lane, ids, offsets, weights, combiner, tile_len, mode, perm_b, perm_f, train,
                                               readonly, threshold, step, prepared["fused"] if prepared is not None else None)
            ctx.saved = saved
            ctx.path = "fused"
            return out

        # ---- collective path (the reference's C1..C3)
        p = prepared if prepared is not None else emb_mod._begin_collective(ids)
        rev, send_splits, recv_splits, n_u, n_in, ids_in = p["rev"], p["send_splits"], p["recv_splits"], p["n_u"], p["n_in"], p["ids_in"]
        tok = span_open("ids")
        p["work"].wait()                          # the id all-to-all was issued asynchronously (for all groups before any wait)
        span_close(tok)
        # owner side: different requesters may ask for the same id
        o_uniq, o_rev, _c, o_offs = C.dedup_partition(ids_in, 1)
        o_n = o_offs[1:2]
        o_rows = store.find(o_uniq, o_n) if readonly else store.lookup_or_insert(o_uniq, o_n, step, threshold, True)
        rows_in = o_rows[o_rev.long()] if n_in else o_rows[:0]
        emb_out = C.gather_rows(store.emb(), rows_in)                 # rows travel in their storage type
        emb_back = torch.empty(n_u, D, dtype=emb_out.dtype, device=ids.device)
        tok = span_open("emb")
        _a2a(emb_back, emb_out, [s for s in send_splits], [r for r in recv_splits], pg)
        span_close(tok)
        out, gsrc, gscale = pool(emb_back, None, rev)
        if train:
            ctx.saved = dict(rev=rev, gsrc=gsrc, gscale=gscale, n_u=n_u, n_in=n_in, send_splits=send_splits,
                             recv_splits=recv_splits, o_rev=o_rev, o_rows=o_rows)
        ctx.path = "collective"
        return out

    @staticmethod
    def backward(ctx, grad_out):
        if not ctx.train:
            return (None,) * 12
        C = native()
        emb_mod = ctx.emb_mod
        impl = emb_mod.impl
        D, W = impl.dim, emb_mod.world_size
        s = ctx.saved
        grad_out = grad_out.contiguous().to(torch.float32).view(-1, D)
        worker_scale = 1.0 / W if emb_mod.option.grad_reduce_by == "worker" else 1.0
        if ctx.path == "local":
            impl.stage_fused(dict(grad_out=grad_out, gsrc=s["gsrc"], gscale=s["gscale"], rev=s["rev"], rows=s["rows"],
                                  scale=worker_scale))
            return (None,) * 12
        if ctx.path == "fused":
            emb_mod.fused.backward(emb_mod, s, grad_out, worker_scale)
            return (None,) * 12
        # ---- collective path (the reference's C4 + owner-side duplicate reduction)
        csr_u, csr_elem, start = C.build_csr(s["rev"])
        gu = C.grad_reduce(grad_out, s["gsrc"], s["gscale"], csr_u, csr_elem, start, D, None, False, 2, 0.0, 0.0, 0.0, 0.0,
                           1.0, 0.0, 1.0, None, None, None, max(s["n_u"], 1))
        g_in = torch.empty(s["n_in"], D, dtype=torch.float32, device=grad_out.device)
        tok = span_open("grad_push")
        _a2a(g_in, gu[:s["n_u"]].contiguous(), s["recv_splits"], s["send_splits"], emb_mod.pg)
        span_close(tok)
        o_rev = s["o_rev"].long()
        o_rows = s["o_rows"]
        g_own = torch.zeros(o_rows.numel(), D, dtype=torch.float32, device=grad_out.device)
        if s["n_in"]:
            g_own.index_add_(0, o_rev, g_in)
            if emb_mod.option.grad_reduce_by == "id":
                cnt = torch.zeros(o_rows.numel(), dtype=torch.float32, device=grad_out.device)
                cnt.index_add_(0, o_rev, torch.ones_like(o_rev, dtype=torch.float32))
                g_own = g_own / cnt.clamp_(min=1.0).unsqueeze(1)
            else:
                g_own = g_own * worker_scale
        impl.accept_grad(o_rows, g_own)
        return (None,) * 12


class _GroupLookupFn(torch.autograd.Function):
    """Lookup of one runtime group split into exchange lanes (``FusedExchange.forward_group``): one shared output, one
    backward that pushes each lane's per-unique gradients to their owners."""

    @staticmethod
    def forward(ctx, holder, emb_mod: "DynamicEmbedding", parts, mode, perm_b, perm_total, n_rows, training, admit_hook):
        impl = emb_mod.impl
        readonly, threshold = admit_params(admit_hook)
        train = training and impl.trainable and emb_mod.option.trainable
        if not (training and impl.trainable):
            readonly = True
        step = emb_mod.table.step_tensor() if not readonly else None
        out, saved = emb_mod.fused.forward_group(emb_mod, parts, mode, perm_b, perm_total, n_rows, train, readonly, threshold, step)
        ctx.train, ctx.emb_mod, ctx.saved = train, emb_mod, saved
        return out

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.train:
            emb_mod = ctx.emb_mod
            grad_out = grad_out.contiguous().to(torch.float32).view(-1, emb_mod.impl.dim)
            worker_scale = 1.0 / emb_mod.world_size if emb_mod.option.grad_reduce_by == "worker" else 1.0
            emb_mod.fused.backward(emb_mod, ctx.saved, grad_out, worker_scale)
        return (None,) * 9


@dataclass
class ExchangeIDsResults:
    """Token of a started lookup (``DynamicEmbedding.exchange_ids``)."""
    ids: torch.Tensor
    offsets: torch.Tensor
    prepared: Optional[dict] = None


@dataclass
class ExchangeEmbResults:
    ids_result: ExchangeIDsResults
    admit_hook: object = None


class DynamicEmbedding(torch.nn.Module):
    """A distributed dynamic embedding table; ``forward`` returns pooled embeddings."""

    def __init__(self, emb_opt: EmbeddingOption, pg: "dist.ProcessGroup" = None):
        super().__init__()
        self._emb_opt = emb_opt
        self.option = emb_opt
        self.pg = pg if pg is not None else emb_opt.pg
        if dist.is_available() and dist.is_initialized():
            self.world_size = dist.get_world_size(self.pg)
            self.rank = dist.get_rank(self.pg)
        else:
            self.world_size, self.rank = 1, 0
        self.fused = None
        storage = None
        growable = True
        mode = os.environ.get("RECIS_COMM", "auto")
        # CUDA: the fused exchange by default. CPU ranks of one machine: only when asked for (RECIS_COMM=fused), through the
        # shared-memory twin of the exchange; "auto" keeps the collective path there
        if self.world_size > 1 and ((emb_opt.device.type == "cuda" and mode in ("auto", "fused")) or
                                    (emb_opt.device.type == "cpu" and mode == "fused")):
            from ...parallel.fused_exchange import FusedExchange
            from ...parallel.symmetric import single_node
            if single_node(self.world_size):
                self.fused = FusedExchange.create(emb_opt, self.pg, self.world_size, self.rank)
            elif mode == "fused":
                import warnings
                warnings.warn("RECIS_COMM=fused needs all ranks on one machine (peer-mapped memory); this job spans machines, "
                              "the collective exchange is used instead", RuntimeWarning)
            if self.fused is not None:
                storage = self.fused.table_storage()
                growable = storage is None
        self.table = HashTable(
            embedding_shape=[emb_opt.embedding_dim], block_size=emb_opt.block_size, dtype=emb_opt.dtype,
            device=emb_opt.device, coalesced=emb_opt.coalesced, children=emb_opt.children,
            slice=gen_slice(self.rank, self.world_size, emb_opt.max_partition_num), initializer=emb_opt.initializer,
            name=emb_opt.shared_name, grad_reduce_by=emb_opt.grad_reduce_by, filter_hook=emb_opt.filter_hook,
            capacity=emb_opt.capacity, emb_storage=storage, growable=growable,
        )
        # duplicates across requesters are averaged by this module; the inner table must not rescale again
        self.table._worker_num = 1
        self._holder = torch.tensor([0.0], requires_grad=True)
        if self.fused is not None:
            self.fused.attach(self)
            self.impl.exchange = self.fused

    @property
    def impl(self):
        return self.table.impl

    def _begin_collective(self, ids: torch.Tensor) -> dict:
        """Id phase of the collective path: dedup + bucket by owner, exchange the counts (blocking, with the host read of the
        split sizes), then start the id all-to-all WITHOUT waiting for it (the reference's C1 and C2,
        ``recis/nn/modules/embedding.py:498-542``)."""
        C = native()
        W, pg = self.world_size, self.pg
        tok = span_open("ids")
        uniq, rev, counts, _offs = C.dedup_partition(ids, W)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=pg)
        send_splits = counts.tolist()             # host read of split sizes (the fused path has none)
        recv_splits = recv_counts.tolist()
        n_u, n_in = sum(send_splits), sum(recv_splits)
        ids_in = torch.empty(n_in, dtype=torch.int64, device=ids.device)
        ids_out = uniq[:n_u].contiguous()
        work = dist.all_to_all_single(ids_in, ids_out, recv_splits, send_splits, group=pg, async_op=True)
        span_close(tok)
        return dict(rev=rev, send_splits=send_splits, recv_splits=recv_splits, n_u=n_u, n_in=n_in, ids_in=ids_in, ids_out=ids_out,
                    work=work)

    def _normalise_ids(self, ids: torch.Tensor) -> torch.Tensor:
        return ids.detach().reshape(-1).to(self.impl.device).contiguous()

    def prepare_lookup(self, ids: torch.Tensor, lane: str = "default"):
        """Start the id phase of a sharded lookup and return a token for ``lookup_pool(..., prepared=token)``, or None when
        there is nothing to start early (one rank; the fused exchange unless its staging is switched on). A model with several
        table groups calls this for every group before the first ``lookup_pool``, so that all id exchanges are in flight
        before anything waits (``recis/nn/modules/embedding_engine.py:739-801`` does the same with asynchronous all-to-alls)."""
        if self.world_size == 1:
            return None
        ids = self._normalise_ids(ids)
        if self.fused is not None:
            if not self.fused.stage_enabled:
                return None
            train = self.training and self.impl.trainable and self._emb_opt.trainable
            return dict(ids=ids, fused=self.fused.prepare(self, lane, ids, train))
        p = self._begin_collective(ids)
        p["ids"] = ids
        return p

    def serve_lookup(self, prepared, admit_hook=None):
        """Second early phase of a prepared lookup on the fused exchange: this rank's owner-side work (wait for the ids, table
        lookup, push of the rows, EMB signal) without waiting for the other owners. A model with several table groups calls it for
        all of them between ``prepare_lookup`` and the first ``lookup_pool``. No-op for tokens of the collective path."""
        if prepared is None or "fused" not in prepared or prepared["fused"]["served"] is not None:
            return prepared
        hook = admit_hook if admit_hook is not None else self._emb_opt.admit_hook
        readonly, threshold = admit_params(hook)
        if not (self.training and self.impl.trainable):
            readonly = True
        step = self.table.step_tensor() if not readonly else None
        self.fused.serve(self, prepared["fused"], readonly, threshold, step)
        return prepared

    def lookup_pool(self, ids: torch.Tensor, offsets: torch.Tensor, weights: Optional[torch.Tensor], combiner: str,
                    tile_len: int = 0, perm=None, admit_hook=None, lane: str = "default", prepared=None) -> torch.Tensor:
        """Flat ids + int32 segment offsets (+ per-id weights) -> pooled rows ``[segments, D]`` (tile: ``[segments, T*D]``)."""
        dev = self.impl.device
        ids = prepared["ids"] if prepared is not None else self._normalise_ids(ids)
        offsets = offsets.to(device=dev, dtype=torch.int32).contiguous()
        if weights is not None:
            weights = weights.detach().reshape(-1).to(device=dev, dtype=torch.float32).contiguous()
        out = _LookupPoolFn.apply(self._holder, self, ids, offsets, weights, combiner, int(tile_len), perm, self.training,
                                  admit_hook if admit_hook is not None else self._emb_opt.admit_hook, lane, prepared)
        return self._out_cast(out)

    def _out_cast(self, out):
        """Pooling accumulates in fp32; the model sees the table's dtype (int8 tables: float16 with ``fp16_enabled``, else float32)."""
        dt = self._emb_opt.dtype
        if dt == torch.int8:
            return out.to(torch.float16) if self._emb_opt.fp16_enabled else out
        return out if dt == torch.float32 else out.to(dt)

    def lookup_pool_group(self, parts, combiner: str, perm_b: int, perm_total: int, n_rows: int, admit_hook=None) -> torch.Tensor:
        """Pooled lookup of several lanes of one runtime group into ONE output ``[n_rows, D]`` (fused exchange only). ``parts``:
        per lane a dict with ``key``, ``ids``, ``offsets``, ``weights`` and the slice of the output it fills (``perm_f`` features
        from feature ``perm_off`` of a ``[perm_b, perm_total, D]`` cube, or ``n_seg`` rows from row ``perm_off`` when
        ``perm_total`` is 0)."""
        assert self.fused is not None and combiner != "tile"
        dev = self.impl.device
        for p in parts:
            p["ids"] = self._normalise_ids(p["ids"])
            p["offsets"] = p["offsets"].to(device=dev, dtype=torch.int32).contiguous()
            if p.get("weights") is not None:
                p["weights"] = p["weights"].detach().reshape(-1).to(device=dev, dtype=torch.float32).contiguous()
        mode = 0 if combiner != "mean" else (2 if self._emb_opt.mean_by_weight else 1)
        out = _GroupLookupFn.apply(self._holder, self, parts, mode, int(perm_b), int(perm_total), int(n_rows), self.training,
                                   admit_hook if admit_hook is not None else self._emb_opt.admit_hook)
        return self._out_cast(out)

    # ---- the reference's three-stage interface (``recis/nn/modules/embedding.py:498-624``) on top of prepare_lookup / lookup_pool
    def exchange_ids(self, ids: torch.Tensor, offsets: torch.Tensor) -> "ExchangeIDsResults":
        """Stage 1: start the id phase (dedup + routing + id exchange) of a lookup of flat ``ids`` with segment ``offsets``."""
        return ExchangeIDsResults(ids=ids, offsets=offsets, prepared=self.prepare_lookup(ids))

    def lookup_exchange_emb(self, ids_exchange_result: "ExchangeIDsResults", admit_hook=None) -> "ExchangeEmbResults":
        """Stage 2 of the reference (owner-side lookup + embedding exchange). On the fused exchange with staging switched on this
        runs the owner side now (rows are pushed, nothing is waited for); otherwise it records the admission hook and the work
        happens in ``emb_reduce``."""
        self.serve_lookup(ids_exchange_result.prepared, admit_hook)
        return ExchangeEmbResults(ids_result=ids_exchange_result, admit_hook=admit_hook)

    def wait_exchange_emb(self, emb_exchange_result: "ExchangeEmbResults"):
        return emb_exchange_result

    def emb_reduce(self, emb_exchange_result: "ExchangeEmbResults", weight, combiner, combiner_kwargs=None, fp16_enable=False):
        """Stage 3: finish the lookup and pool (``sum`` / ``mean`` / ``tile``); returns ``[segments, D]`` (tile: ``[segments, T*D]``)."""
        r = emb_exchange_result.ids_result
        tile_len = (combiner_kwargs or {}).get("tile_len", 0) if combiner == "tile" else 0
        out = self.lookup_pool(r.ids, r.offsets, weight, combiner, tile_len, admit_hook=emb_exchange_result.admit_hook, prepared=r.prepared)
        return out.to(torch.float16) if fp16_enable else out

    def deal_with_tensor(self, input_tensor):
        if isinstance(input_tensor, RaggedTensor):
            ids = input_tensor.values()
            offsets = input_tensor.offsets()[-1]
            weight = input_tensor.weight()
            shape = tuple(o.numel() - 1 for o in input_tensor.offsets()[:1]) if len(input_tensor.offsets()) == 1 else (
                input_tensor.offsets()[-1].numel() - 1,)
            return ids, offsets, weight, shape
        if input_tensor.is_sparse:
            raise TypeError("DynamicEmbedding doesn't support sparse ids")
        bs, fea = input_tensor.shape[0], input_tensor.shape[-1]
        n_seg = input_tensor.numel() // fea
        offsets = torch.arange(0, (n_seg + 1) * fea, fea, dtype=torch.int32, device=input_tensor.device)
        return input_tensor.reshape(-1), offsets, None, tuple(input_tensor.shape[:-1])

    def forward(self, input_ids: Union[torch.Tensor, RaggedTensor], input_weights=None):
        ids, offsets, weight, shape = self.deal_with_tensor(input_ids)
        if input_weights is not None:
            weight = input_weights
        if not self._emb_opt.use_weight:
            weight = None
        opt = self._emb_opt
        tile_len = opt.combiner_kwargs["tile_len"] if opt.combiner == "tile" else 0
        emb = self.lookup_pool(ids, offsets, weight, opt.combiner, tile_len)
        if opt.combiner == "tile":
            emb = emb.view(-1, tile_len * opt.embedding_dim)
        else:
            emb = emb.view(shape + (opt.embedding_dim,))
        if not opt.trainable:
            emb = emb.detach()
        return emb
