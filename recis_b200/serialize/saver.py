"""Sparse checkpoint writer (``recis/serialize/saver.py`` + ``csrc/serialize/saver.cc:38-64``, ``save_bundle.cc``).

Every shard writes ``parallel`` safetensors files ``model-<shard*parallel+i>-of-<parallel*shard_num>.safetensors`` holding,
for each logical (child) table of its physical tables, the blocks ``<child>.id``, ``<child>.embedding`` and one block per
optimizer / filter slot (suffix ``/part_<shard>_<shard_num>``), plus - on shard 0 - the dense tensors (key ``<name>^ ``).
Shard 0 then merges the per-shard metadata into ``index``, ``tensorkey.json`` and
``torch_rank_weights_embs_table_multi_shard.json``. The merge is a gather over the process group; the reference polls the
file system for the other shards' files instead (``save_bundle.cc:131-160``).
Rows are gathered on the device and streamed through pinned staging by the native writer, so a save never materialises a
host copy of a table.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from .. import native
from ..nn.modules.hashtable import ChildrenInfo
from . import names as N


class Saver:
    def __init__(self, shard_index: int = 0, shard_num: int = 1, parallel: int = 8, path: str = ".",
                 hashtables: Optional[Dict[str, object]] = None, tensors: Optional[Dict[str, torch.Tensor]] = None,
                 filter_func=lambda x: x, pg=None):
        """Argument order as in the reference (``recis/serialize/saver.py:32-41``). ``filter_func`` receives the list of write
        blocks, tuples ``(disk key, internal block name or None, dtype string, shape, is_dense, payload)``, and returns the
        blocks to write (drop entries to leave tensors out of the bundle)."""
        assert parallel > 0 and 0 <= shard_index < shard_num
        self.shard_index, self.shard_num, self.parallel = shard_index, shard_num, parallel
        self.hashtables, self.tensors, self.path, self.pg = hashtables or {}, tensors or {}, path, pg
        self.filter_func = filter_func

    # ---- collect blocks: (disk key, internal name or None, dtype str, shape, dense?, native block tuple)
    def _table_blocks(self):
        blocks = []
        seen = set()
        for impl in self.hashtables.values():
            if id(impl) in seen:
                continue
            seen.add(id(impl))
            ids, rows = impl.store.snapshot(False, 0)
            order = torch.argsort(ids)                      # deterministic file contents
            ids, rows = ids[order], rows[order]
            children = impl.children_info().children()
            coalesced = impl.children_info().is_coalesce()
            child_idx = ChildrenInfo.decode_index(ids) if coalesced else torch.zeros_like(ids)
            slots = [(N.EMB_SLOT, impl.store.emb())] + [(s, impl.store.slot(s)) for s in impl.store.slot_names()]
            last_seen = impl.store.last_seen()
            if last_seen is not None and last_seen.numel():
                slots.append((N.FILTER_SLOT, last_seen))
            for ci, child in enumerate(children):
                sel = (child_idx == ci).nonzero().view(-1)
                c_ids = (ChildrenInfo.decode_id(ids[sel]) if coalesced else ids[sel]).cpu().contiguous()
                c_rows = rows[sel].to(torch.int32).contiguous()
                n = c_ids.numel()
                key = lambda slot: (N.disk_key(child, slot, self.shard_index, self.shard_num), N.block_name(child, slot, impl.slice))
                blocks.append((*key(N.ID_SLOT), "I64", [n], False, (0, c_ids, None)))
                for slot, slab in slots:
                    shape = [n] + list(slab.shape[1:]) if slab.dim() > 1 else [n, 1]
                    blocks.append((*key(slot), N.dtype_to_str(slab.dtype), shape, False, (1, slab, c_rows)))
        return blocks

    def _dense_blocks(self):
        blocks = []
        if self.shard_index == 0:
            for name, t in self.tensors.items():
                t = t.detach().cpu().contiguous()
                blocks.append((N.dense_key(name), None, N.dtype_to_str(t.dtype), list(t.shape), True, (0, t, None)))
        return blocks

    def save(self):
        os.makedirs(self.path, exist_ok=True)
        blocks = list(self.filter_func(self._table_blocks() + self._dense_blocks()))
        total_files = self.parallel * self.shard_num
        files = [dict(name=N.data_file_name(self.shard_index * self.parallel + i, total_files), header={}, blocks=[], offset=0)
                 for i in range(self.parallel)]
        tensorkey, block_index, rank_json = {}, {}, {}
        for k, (disk, internal, dt, shape, dense, nb) in enumerate(blocks):
            f = files[k % self.parallel]
            nbytes = N.str_to_dtype(dt).itemsize
            for s in shape:
                nbytes *= s
            f["header"][disk] = {"dtype": dt, "shape": shape, "data_offsets": [f["offset"], f["offset"] + nbytes]}
            f["offset"] += nbytes
            f["blocks"].append(nb)
            block_index[disk] = f["name"]
            if internal is not None:
                tensorkey[disk] = internal
            entry = {"name": disk, "dtype": N.rank_json_dtype(dt), "shape": shape, "dense": dense}
            if dense:
                entry.update(dimension=0, is_hashmap=False)
                rank_json[disk] = entry
            elif f".{N.EMB_SLOT}/part_" in disk:
                entry.update(dimension=shape[-1], is_hashmap=True, hashmap_key=disk.replace(f".{N.EMB_SLOT}", f".{N.ID_SLOT}"),
                             hashmap_key_dtype="int64", hashmap_value=disk)
                rank_json[disk] = entry
        jobs = [(N.join(self.path, f["name"]), json.dumps(f["header"], separators=(",", ":")), f["blocks"]) for f in files if f["blocks"]]
        # the native writer gathers rows on streams of its own (one per writer thread): everything queued so far on this
        # thread's streams - the last optimizer update, the row-index tensors built above - has to be complete before it starts
        for dev in {impl.store.emb().device for impl in self.hashtables.values() if impl.store.emb().is_cuda}:
            torch.cuda.synchronize(dev)
        native().st_write_files(jobs)
        meta = dict(files=[f["name"] for f in files if f["blocks"]], block_index=block_index, tensorkey=tensorkey, rank_json=rank_json)
        self._merge_meta(meta)

    def _merge_meta(self, meta):
        metas = [meta]
        if self.shard_num > 1:
            if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.pg) == self.shard_num:
                metas = [None] * self.shard_num if self.shard_index == 0 else None
                dist.gather_object(meta, metas, dst=0, group=self.pg)
                if self.shard_index != 0:
                    return
            else:
                # shards saved one after another by a single process (tools, tests): park the metadata next to the data and
                # merge once the last shard has arrived
                with open(N.join(self.path, f"shardmeta-{self.shard_index}.json"), "w") as fh:
                    json.dump(meta, fh)
                paths = [N.join(self.path, f"shardmeta-{i}.json") for i in range(self.shard_num)]
                if not all(os.path.exists(p) for p in paths):
                    return
                metas = [json.load(open(p)) for p in paths]
                for p in paths:
                    os.remove(p)
        file_index, block_index, tensorkey, rank_json = {}, {}, {}, {}
        for m in metas:
            for f in m["files"]:
                file_index.setdefault(f, len(file_index))
        for m in metas:
            for blk, f in m["block_index"].items():
                block_index[blk] = file_index[f]
            tensorkey.update(m["tensorkey"])
            rank_json.update(m["rank_json"])
        for name, obj in ((N.INDEX_FILE, {"file_index": file_index, "block_index": block_index}), (N.TENSORKEY_FILE, tensorkey),
                          (N.RANK_JSON_FILE, rank_json)):
            tmp = N.join(self.path, name + ".tmp")
            with open(tmp, "w") as fh:
                json.dump(obj, fh, indent=4)
            os.replace(tmp, N.join(self.path, name))
