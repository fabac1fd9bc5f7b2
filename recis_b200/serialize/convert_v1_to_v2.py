"""Convert a version-1 checkpoint directory (one ``torch.save`` file per table shard holding ``{"ids", "embeddings",
<slot>...}`` plus ``dense.pt``) into the safetensors bundle layout (role of ``recis/serialize/convert_v1_to_v2.py``)."""
from __future__ import annotations

import glob
import json
import os
import re

import torch

from .. import native
from ..nn.modules.hashtable import Slice
from . import names as N


def convert_v1_to_v2(src_dir: str, dst_dir: str, slice_size: int = 65536):
    os.makedirs(dst_dir, exist_ok=True)
    shard_files = sorted(glob.glob(os.path.join(src_dir, "*.shard_*_of_*.pt")))
    header, blocks, tensorkey, block_index, rank_json, offset = {}, [], {}, {}, {}, 0
    fname = N.data_file_name(0, 1)

    def add(disk, dt, t, dense, internal=None):
        nonlocal offset
        t = t.detach().cpu().contiguous()
        header[disk] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [offset, offset + t.numel() * t.element_size()]}
        offset += t.numel() * t.element_size()
        blocks.append((0, t, None))
        block_index[disk] = 0
        if internal:
            tensorkey[disk] = internal
        rank_json[disk] = {"name": disk, "dtype": N.rank_json_dtype(dt), "shape": list(t.shape), "dense": dense,
                           "dimension": 0 if dense else (t.shape[-1] if t.dim() > 1 else 1), "is_hashmap": False}

    for f in shard_files:
        m = re.match(r"(.+)\.shard_(\d+)_of_(\d+)\.pt$", os.path.basename(f))
        child, shard, shard_num = m.group(1), int(m.group(2)), int(m.group(3))
        q, r = divmod(slice_size, shard_num)
        beg = shard * q + min(shard, r)
        sl = Slice(beg, beg + q + (1 if shard < r else 0), slice_size)
        data = torch.load(f, map_location="cpu", weights_only=False)
        for key, t in data.items():
            slot = {"ids": N.ID_SLOT, "embeddings": N.EMB_SLOT}.get(key, key)
            add(N.disk_key(child, slot, shard, shard_num), N.dtype_to_str(t.dtype), t, False, N.block_name(child, slot, sl))
    dense_path = os.path.join(src_dir, "dense.pt")
    if os.path.exists(dense_path):
        for name, t in torch.load(dense_path, map_location="cpu", weights_only=False).items():
            add(N.dense_key(name), N.dtype_to_str(t.dtype), t, True)
    native().st_write_files([(os.path.join(dst_dir, fname), json.dumps(header, separators=(",", ":")), blocks)])
    for name, obj in ((N.INDEX_FILE, {"file_index": {fname: 0}, "block_index": block_index}), (N.TENSORKEY_FILE, tensorkey),
                      (N.RANK_JSON_FILE, rank_json)):
        with open(os.path.join(dst_dir, name), "w") as fh:
            json.dump(obj, fh, indent=4)
