"""Sparse checkpoint loader with resharding (``recis/serialize/loader.py``, ``csrc/serialize/load_internal.cc:25-273``,
``read_block.cc:71-241``).

For every logical table of every physical table: each saved shard whose slice range intersects this rank's range is read;
ids are kept when ``id & 0xFFFF`` (= ``uint64(id) % 65536``) falls in this rank's range, re-prefixed with the child index of
merged tables and inserted; slot rows (embedding, optimizer state, last-seen step) follow in chunks of
``RECIS_BLOCK_READ_SIZE`` rows, written only to the rows of kept ids. A checkpoint saved by W1 ranks can therefore be
loaded by W2 ranks. Dense tensors are copied in place."""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from .. import native
from ..nn.modules.hashtable import ChildrenInfo
from . import names as N
from .checkpoint_reader import BundleIndex


class Loader:
    def __init__(self, checkpoint_path: str, hashtables: Optional[Dict[str, object]] = None,
                 tensors: Optional[Dict[str, torch.Tensor]] = None, parallel: int = 16, filter_func=lambda x: x, strict: bool = True):
        """``filter_func`` receives the default load plan ``{"hashtables": [logical table names], "tensors": [dense names]}`` (what
        the model asks for) and returns the plan to execute; names it drops are left untouched (the reference passes its
        load-info JSON through the same hook, ``recis/serialize/loader.py:60-77``)."""
        self.index = BundleIndex(checkpoint_path)
        self.hashtables, self.tensors, self.strict = hashtables or {}, tensors or {}, strict
        self.filter_func = filter_func
        self.chunk = max(int(os.environ.get("RECIS_BLOCK_READ_SIZE", 1 << 20)), 1)
        # slot blocks of a chunk are read by up to ``parallel`` threads (the native file reads release the GIL), the role of the
        # reference loader's thread pool (``csrc/serialize/load_internal.cc:195-273``)
        self.parallel = max(int(parallel), 1)

    def load(self):
        seen = set()
        impls = []
        for impl in self.hashtables.values():
            if id(impl) not in seen:
                seen.add(id(impl))
                impls.append(impl)
        plan = self.filter_func({"hashtables": sorted(c for impl in impls for c in impl.children_info().children()),
                                 "tensors": sorted(self.tensors)})
        self._wanted_children = set(plan.get("hashtables", []))
        wanted_tensors = set(plan.get("tensors", []))
        for impl in impls:
            self._load_table(impl)
        dense = set(self.index.dense_names())
        for name, t in self.tensors.items():
            if name not in wanted_tensors:
                continue
            if name not in dense:
                if self.strict:
                    raise KeyError(f"dense tensor {name} is missing from the checkpoint")
                continue
            src = self.index.read(N.dense_key(name))
            if tuple(src.shape) != tuple(t.shape):
                raise ValueError(f"shape mismatch for {name}: checkpoint {tuple(src.shape)} vs model {tuple(t.shape)}")
            with torch.no_grad():
                t.copy_(src.to(t.dtype))

    def _load_table(self, impl):
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=self.parallel) as pool:
            self._load_table_with(impl, pool)

    def _load_table_with(self, impl, pool):
        C = native()
        dev = impl.device
        sl = impl.slice
        coalesced = impl.children_info().is_coalesce()
        slot_names = [N.EMB_SLOT] + impl.store.slot_names()
        if impl.store.last_seen() is not None and impl.store.last_seen().numel():
            slot_names.append(N.FILTER_SLOT)
        for ci, child in enumerate(impl.children_info().children()):
            if child not in self._wanted_children:
                continue
            parts = self.index.table_parts(child, N.ID_SLOT)
            if not parts:
                if self.strict:
                    raise KeyError(f"table {child} is missing from the checkpoint")
                continue
            for disk, beg, end, size in parts:
                if size != sl.slice_size:
                    raise ValueError(f"{child}: slice space {size} in the checkpoint vs {sl.slice_size} in the model")
                if end <= sl.slice_begin or beg >= sl.slice_end:
                    continue                                     # no overlap with the slices this rank owns
                n = self.index.block_meta(disk)[3][0]
                for r0 in range(0, n, self.chunk):
                    r1 = min(r0 + self.chunk, n)
                    ids = self.index.read(disk, r0, r1)
                    slice_of = ids & (sl.slice_size - 1) if sl.slice_size & (sl.slice_size - 1) == 0 else ids.remainder(sl.slice_size)
                    keep = ((slice_of >= sl.slice_begin) & (slice_of < sl.slice_end)).nonzero().view(-1)
                    if keep.numel() == 0:
                        continue
                    kept = ids[keep]
                    enc = ChildrenInfo.encode(kept, ci) if coalesced else kept
                    pending = {}
                    for slot in slot_names:                          # all slot reads of the chunk are in flight together
                        sdisk = disk.replace(f".{N.ID_SLOT}/", f".{slot}/")
                        if sdisk not in self.index.block_file:
                            if self.strict and slot == N.EMB_SLOT:
                                raise KeyError(f"{sdisk} missing from the checkpoint")
                            continue
                        pending[slot] = pool.submit(self.index.read, sdisk, r0, r1)
                    rows = impl.store.lookup_or_insert(enc.to(dev).contiguous(), None, None, 1, True)
                    if bool((rows < 0).any()):
                        # the table could not take every id of the checkpoint (fixed storage that is too small, or a full index)
                        raise RuntimeError(
                            f"checkpoint does not fit: table '{impl.name}' (child '{child}') holds {impl.size()} rows of "
                            f"{impl.store.capacity()} and could not admit {int((rows < 0).sum())} of {rows.numel()} ids of this "
                            "chunk; create the table with a larger capacity")
                    for slot, fut in pending.items():
                        data = fut.result()[keep]
                        if slot == N.FILTER_SLOT:
                            impl.store.last_seen().index_copy_(0, rows.long(), data.view(-1).to(dev))
                        else:
                            slab = impl.store.emb() if slot == N.EMB_SLOT else impl.store.slot(slot)
                            C.scatter_rows(slab, rows, data.to(dev, slab.dtype).contiguous(), False)      # rows in the table's storage type
