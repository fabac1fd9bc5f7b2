"""EmbeddingEngine: many features, few physical tables.

Semantics of the reference's ``recis/nn/modules/embedding_engine.py:17-832``:

* features whose ``EmbeddingOption.coalesced_info()`` (dim, dtype, device, initializer, grad_reduce_by,
  filter_hook) agree are merged into ONE physical table named ``CoalescedHashtable_<sha256>``; each distinct
  ``shared_name`` becomes a child with a 12-bit prefix in the top bits of the id;
* inside a table, features with equal ``runtime_info()`` (combiner, use_weight, trainable, admit_hook, ...)
  are concatenated so that each (table, runtime group) does one lookup/exchange per step;
* results are split back per feature and shaped ``[batch, ..., dim]``; keys without an embedding option pass
  through (ragged tensors become dense).

The concatenation (id prefixing + offset rebasing for all features of a group) is a single multi-tensor
kernel driven by a small descriptor table that is copied asynchronously; nothing synchronises with the host.
With ``interleave=True`` the pooled rows of a group are written directly in ``[batch, feature, dim]`` order,
so a model that wants the stacked tensor (``EmbeddingEngine.packed``) gets it without a copy.
"""
from __future__ import annotations

import copy
import hashlib
import os
import math
from collections import OrderedDict, defaultdict

import torch
from torch import nn

from ... import native
from ...ragged.tensor import RaggedTensor
from ...utils import debug as _debug
from .embedding import DynamicEmbedding, EmbeddingOption


class _Group:
    """Features that share one physical table."""

    def __init__(self, name):
        self.name = name
        self.opt = None
        self.children = OrderedDict()  # shared_name -> child index
        self.fea_runtime = {}
        self.fea_child = {}

    def add(self, fea_name, opt: EmbeddingOption):
        if self.opt is None:
            self.opt = copy.copy(opt)
        if opt.shared_name not in self.children:
            self.children[opt.shared_name] = len(self.children)
        self.fea_runtime[fea_name] = opt.runtime_info()
        self.fea_child[fea_name] = self.children[opt.shared_name]

    def embedding_option(self, capacity, exchange_capacity=0, exchange_strict=False):
        o = self.opt
        return EmbeddingOption(
            embedding_dim=o.embedding_dim, block_size=o.block_size, dtype=o.dtype, device=o.device, shared_name=self.name,
            children=list(self.children.keys()), coalesced=True, initializer=o.initializer, grad_reduce_by=o.grad_reduce_by,
            fp16_enabled=o.fp16_enabled, filter_hook=o.filter_hook, pg=o.pg, max_partition_num=o.max_partition_num,
            capacity=capacity, mean_by_weight=o.mean_by_weight, exchange_capacity=exchange_capacity,
            exchange_strict=exchange_strict,
        )


class EmbeddingEngine(nn.Module):
    def __init__(self, emb_options: dict, interleave: bool = False, exchange_lanes: int = 0):
        super().__init__()
        # exchange_lanes > 1 (or RECIS_EXCHANGE_LANES): the features of one (table, runtime group) are split into that many
        # lanes (features of one shared_name stay together), each with its own exchange windows; the lanes run as a pipeline
        # in which one lane's NVLink-bound kernels overlap the other lanes' memory-bound ones. Only used with more than one
        # rank and the peer-memory exchange.
        self._lanes = int(exchange_lanes or os.environ.get("RECIS_EXCHANGE_LANES", "1"))
        self._ht = nn.ModuleDict()
        self._groups = {}
        self._fea_to_ht = {}
        self._emb_opts = emb_options
        self._interleave = interleave
        self.packed = {}
        self._desc_ring = {}
        shared_to_ht = {}
        capacity = defaultdict(int)
        for fea_name, opt in emb_options.items():
            ht_name = f"CoalescedHashtable_{hashlib.sha256(opt.coalesced_info().encode()).hexdigest()}"
            if shared_to_ht.setdefault(opt.shared_name, ht_name) != ht_name:
                raise RuntimeError(
                    f"Create embedding failed, emb shared name {opt.shared_name} already created with a different "
                    f"merge key; current: {opt.coalesced_info()}")
            if ht_name not in self._groups:
                self._groups[ht_name] = _Group(ht_name)
            self._groups[ht_name].add(fea_name, opt)
            self._fea_to_ht[fea_name] = ht_name
        xcap = defaultdict(int)
        strict = defaultdict(bool)
        for fea_name, opt in emb_options.items():
            capacity[self._fea_to_ht[fea_name]] += int(opt.capacity or 0)
            xcap[self._fea_to_ht[fea_name]] += int(opt.exchange_capacity or 0)
            strict[self._fea_to_ht[fea_name]] |= bool(getattr(opt, "exchange_strict", False))
        for ht_name, group in self._groups.items():
            self._ht[ht_name] = DynamicEmbedding(group.embedding_option(capacity[ht_name], xcap[ht_name], strict[ht_name]))

    # ------------------------------------------------------------------ helpers
    def tables(self):
        return {k: v for k, v in self._ht.items()}

    def table_of(self, fea_name) -> DynamicEmbedding:
        return self._ht[self._fea_to_ht[fea_name]]

    @staticmethod
    def _format(fea, opt: EmbeddingOption, device):
        """feature tensor -> (ids int64 [n], offsets int32 [S+1], weights or None, n_segments, out shape)."""
        dim = opt.embedding_dim
        if isinstance(fea, RaggedTensor):
            ids = fea.values()
            weight = fea.weight()
            offsets = fea.offsets()[-1]
            n_seg = offsets.numel() - 1
            if len(fea.offsets()) == 1:
                lead = (n_seg,)
            else:
                lead = fea.real_shape(0, -1)
                if math.prod(lead) != n_seg:
                    raise RuntimeError(f"RaggedTensor must pad before lookup, got: {fea}")
            if opt.combiner == "tile":
                shape = (lead[0], opt.combiner_kwargs["tile_len"], dim) if len(lead) == 1 else lead + (opt.combiner_kwargs["tile_len"] * dim,)
            else:
                shape = tuple(lead) + (dim,)
        elif isinstance(fea, torch.Tensor):
            if fea.is_sparse:
                raise TypeError("EmbeddingEngine doesn't support sparse ids")
            if fea.dim() == 1:
                fea = fea.unsqueeze(-1)
            width = fea.shape[-1]
            n_seg = fea.numel() // max(width, 1)
            ids = fea.reshape(-1)
            weight = None
            offsets = torch.arange(0, (n_seg + 1) * width, width, dtype=torch.int32, device=fea.device)
            if opt.combiner == "tile":
                shape = (fea.shape[0], dim * opt.combiner_kwargs["tile_len"])
            else:
                shape = tuple(fea.shape[:-1]) + (dim,)
        else:
            raise TypeError(f"EmbeddingEngine only support tensor but get {type(fea)}")
        if _debug.enabled():
            _debug.check_ragged("embedding input", ids, offsets, weight)
        if ids.dtype != torch.int64:
            ids = ids.to(torch.int64)
        if offsets.dtype != torch.int32:
            offsets = offsets.to(torch.int32)
        ids = ids.to(device).contiguous()
        offsets = offsets.to(device).contiguous()
        if not opt.use_weight:
            weight = None
        elif weight is not None:
            weight = weight.to(device=device, dtype=torch.float32).contiguous()
        return ids, offsets, weight, n_seg, shape

    def _coalesce(self, feats, device):
        """Concatenate formatted features: one kernel prefixes ids and rebases offsets for all of them."""
        return self._coalesce_many([feats], device)[0]

    def _coalesce_many(self, parts, device):
        """``_coalesce`` for several feature lists at once (the lanes of one runtime group), in one native call: the descriptor
        tables of all of them travel to the device in ONE asynchronous copy, then one kernel per list prefixes ids and rebases
        offsets."""
        merged = native().coalesce_lanes([[f["ids"] for f in feats] for feats in parts], [[f["offsets"] for f in feats] for feats in parts],
                                         [[int(f["child"]) for f in feats] for feats in parts])
        out = []
        for feats, (ids, offsets) in zip(parts, merged):
            weights = None
            if any(f["weight"] is not None for f in feats):
                ws = [f["weight"] if f["weight"] is not None else torch.ones(f["ids"].numel(), device=device) for f in feats]
                weights = torch.cat(ws) if len(ws) > 1 else ws[0]
            out.append((ids, offsets, weights))
        return out

    # ------------------------------------------------------------------ lanes
    @staticmethod
    def _lane_ranges(children, lanes):
        """Split features 0..n-1 into at most ``lanes`` contiguous ranges such that no child table (``shared_name``) has features
        in two ranges: the rows of two lanes are then disjoint, which is what lets their gradient windows be applied one after
        the other (a row in two lanes would get two optimizer updates instead of one update of the summed gradient). Returns the
        list of range boundaries ``[0, ..., n]``."""
        n = len(children)
        if lanes <= 1 or n < 2:
            return [0, n]
        last = {}
        for i, c in enumerate(children):
            last[c] = i
        allowed, reach = [], -1
        for i, c in enumerate(children):           # a cut in front of feature i+1 is allowed when no child seen so far comes back later
            reach = max(reach, last[c])
            if reach == i and i + 1 < n:
                allowed.append(i + 1)
        bounds = [0]
        for k in range(1, lanes):
            target = n * k // lanes
            cands = [a for a in allowed if a > bounds[-1]]
            if not cands:
                break
            cut = min(cands, key=lambda a: (abs(a - target), a))
            bounds.append(cut)
        bounds.append(n)
        return bounds

    def _use_lanes(self, ht, feats, opt, n_groups) -> bool:
        """The lane pipeline (one native call per forward / backward of the whole group) serves every pooled lookup of the
        peer-memory exchange, with one lane when lanes are off; ``tile`` lookups and the staged mode for several groups
        (``RECIS_STAGE_EXCHANGE``) take the per-group path."""
        ex = getattr(ht, "fused", None)
        if ex is None or opt.combiner == "tile":
            return False
        if ex.stage_enabled and n_groups > 1:
            return False
        return self._lanes > 1 or ex.native_executor

    def _lookup_in_lanes(self, ht, feats, opt, run_key, dev, perm):
        """One runtime group as a pipeline of exchange lanes (``FusedExchange.forward_group``). Returns the pooled rows of the
        whole group: ``[segments_per_feature * n_features, D]`` in the interleaved layout when ``perm`` is set, else the features'
        segments one after the other."""
        bounds = self._lane_ranges([f["child"] for f in feats], self._lanes)
        L = len(bounds) - 1
        parts, seg_off = [], 0
        merged = self._coalesce_many([feats[bounds[i]:bounds[i + 1]] for i in range(L)], dev)
        for i in range(L):
            part = feats[bounds[i]:bounds[i + 1]]
            ids, offsets, weights = merged[i]
            key = f"{run_key}#lane{i}of{L}"
            ht.fused.lane_children[key] = frozenset(f["child"] for f in part)
            n_seg = sum(f["n_seg"] for f in part)
            parts.append(dict(key=key, ids=ids, offsets=offsets, weights=weights, perm_f=len(part), n_seg=n_seg,
                              perm_off=bounds[i] if perm is not None else seg_off))
            seg_off += n_seg
        if perm is not None:
            return ht.lookup_pool_group(parts, opt.combiner, perm[0], perm[1], perm[0] * perm[1], opt.admit_hook)
        return ht.lookup_pool_group(parts, opt.combiner, 0, 0, seg_off, opt.admit_hook)

    # ------------------------------------------------------------------ forward
    def forward(self, input_features: dict):
        grouped = defaultdict(lambda: defaultdict(list))
        outs = {}
        direct = {}
        for fea_name, fea in input_features.items():
            if fea_name not in self._fea_to_ht:
                direct[fea_name] = fea
                continue
            ht_name = self._fea_to_ht[fea_name]
            group = self._groups[ht_name]
            opt = self._emb_opts[fea_name]
            dev = self._ht[ht_name].impl.device
            ids, offsets, weight, n_seg, shape = self._format(fea, opt, dev)
            grouped[ht_name][group.fea_runtime[fea_name]].append(dict(
                name=fea_name, ids=ids, offsets=offsets, weight=weight, n_seg=n_seg, shape=shape, child=group.fea_child[fea_name],
                opt=opt))
        self.packed = {}
        # pass 1: coalesce every (table, runtime group) and, when there are several, start the id phase of all of them before
        # anything waits (the reference issues all its id all-to-alls up front, embedding_engine.py:739-801)
        n_groups = sum(len(r) for r in grouped.values())
        plan = []
        for ht_name, runtimes in grouped.items():
            ht: DynamicEmbedding = self._ht[ht_name]
            dev = ht.impl.device
            for run_key, feats in runtimes.items():
                opt = feats[0]["opt"]
                tile_len = opt.combiner_kwargs["tile_len"] if opt.combiner == "tile" else 0
                segs = [f["n_seg"] for f in feats]
                perm = None
                if self._interleave and opt.combiner != "tile" and len(set(segs)) == 1 and len(feats) > 1:
                    perm = (segs[0], len(feats))
                lanes = self._use_lanes(ht, feats, opt, n_groups)
                ids = offsets = weights = prepared = None
                if not lanes:
                    ids, offsets, weights = self._coalesce(feats, dev)
                    if getattr(ht, "fused", None) is not None:
                        ht.fused.lane_children[run_key] = frozenset(f["child"] for f in feats)
                    if n_groups > 1:
                        prepared = ht.prepare_lookup(ids, lane=run_key)
                plan.append((ht_name, ht, dev, run_key, feats, opt, tile_len, segs, perm, lanes, ids, offsets, weights, prepared))
        # pass 1b (fused exchange with staging): every group's owner-side work and EMB signal before the first EMB wait
        for entry in plan:
            if entry[-1] is not None:
                entry[1].serve_lookup(entry[-1], entry[5].admit_hook)
        # pass 2: finish the lookups in the same order
        for ht_name, ht, dev, run_key, feats, opt, tile_len, segs, perm, lanes, ids, offsets, weights, prepared in plan:
            ht.option.mean_by_weight = opt.mean_by_weight
            if lanes:
                pooled = self._lookup_in_lanes(ht, feats, opt, run_key, dev, perm)
            else:
                pooled = ht.lookup_pool(ids, offsets, weights, opt.combiner, tile_len, perm, opt.admit_hook, lane=run_key,
                                        prepared=prepared)
            if not opt.trainable:
                pooled = pooled.detach()
            D = opt.embedding_dim
            if perm is not None:
                cube = pooled.view(segs[0], len(feats), D)
                self.packed[(ht_name, run_key)] = (cube, [f["name"] for f in feats])
                for j, f in enumerate(feats):
                    outs[f["name"]] = cube[:, j, :].reshape(f["shape"]) if len(f["shape"]) != 2 else cube[:, j, :]
            else:
                rows_per = segs
                pooled = pooled.view(-1, (tile_len or 1) * D)
                start = 0
                for f, s in zip(feats, rows_per):
                    outs[f["name"]] = pooled[start:start + s].reshape(f["shape"])
                    start += s
        for k, v in direct.items():
            if isinstance(v, RaggedTensor):
                outs[k] = v.to_dense()
            elif isinstance(v, torch.Tensor) and v.is_sparse:
                raise TypeError("EmbeddingEngine doesn't support sparse tensor")
            else:
                outs[k] = v
        return outs
