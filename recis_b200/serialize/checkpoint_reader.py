"""Read any tensor of a checkpoint bundle (``recis/serialize/checkpoint_reader.py``, ``csrc/serialize/checkpoint_reader.cc:25-69``).

``read_tensor("<child>@<slot>")`` (or the dotted form) concatenates all saved shards of a table block; dense tensors are
addressed by their plain name."""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

from .. import native
from . import names as N


class BundleIndex:
    """Parsed ``index`` + ``tensorkey.json`` + safetensors headers of a checkpoint directory."""

    def __init__(self, path: str):
        self.path = path
        idx_path = N.join(path, N.INDEX_FILE)
        if not os.path.exists(idx_path):
            raise FileNotFoundError(f"{idx_path}: not a checkpoint directory (missing index)")
        with open(idx_path) as fh:
            idx = json.load(fh)
        self.files: List[str] = [None] * len(idx["file_index"])
        for name, i in idx["file_index"].items():
            self.files[i] = name
        self.block_file: Dict[str, str] = {blk: self.files[i] for blk, i in idx["block_index"].items()}
        tk = N.join(path, N.TENSORKEY_FILE)
        self.tensorkey: Dict[str, str] = json.load(open(tk)) if os.path.exists(tk) else {}
        self._headers = {}

    def header(self, file_name: str):
        if file_name not in self._headers:
            full = N.join(self.path, file_name)
            if not os.path.exists(full):
                raise FileNotFoundError(f"checkpoint shard {full} listed in the index is missing")
            text, start = native().st_read_header(full)
            self._headers[file_name] = (json.loads(text), start)
        return self._headers[file_name]

    def block_meta(self, disk_key: str):
        if disk_key not in self.block_file:
            raise KeyError(f"{disk_key} is not in the checkpoint index")
        f = self.block_file[disk_key]
        header, start = self.header(f)
        if disk_key not in header:
            raise KeyError(f"{disk_key} is indexed in {f} but missing from that file's header")
        m = header[disk_key]
        return f, start + m["data_offsets"][0], N.str_to_dtype(m["dtype"]), list(m["shape"])

    def read(self, disk_key: str, row_begin: int = 0, row_end: int = None) -> torch.Tensor:
        f, off, dtype, shape = self.block_meta(disk_key)
        rows = shape[0] if shape else 1
        row_end = rows if row_end is None else min(row_end, rows)
        inner = 1
        for s in shape[1:]:
            inner *= s
        out_shape = [max(row_end - row_begin, 0)] + shape[1:] if shape else []
        out = torch.empty(out_shape, dtype=dtype)
        if out.numel():
            native().st_read_into(N.join(self.path, f), off + row_begin * inner * dtype.itemsize, out)
        return out

    def table_parts(self, child: str, slot: str):
        """[(disk key, beg, end, size)] of every saved shard of ``<child>.<slot>``."""
        out = []
        for disk, internal in self.tensorkey.items():
            c, s, beg, end, size = N.parse_block_name(internal)
            if c == child and s == slot:
                out.append((disk, beg, end, size))
        return sorted(out, key=lambda x: x[1])

    def dense_names(self):
        return [k[:-2] for k in self.block_file if k.endswith("^ ")]

    def table_blocks(self):
        return sorted({tuple(N.parse_block_name(v)[:2]) for v in self.tensorkey.values()})


class CheckpointReader:
    def __init__(self, path: str):
        self._index = BundleIndex(path)

    def list_tensors(self) -> List[str]:
        return sorted(self._index.dense_names() + [f"{c}@{s}" for c, s in self._index.table_blocks()])

    def tensor_names(self) -> List[str]:
        return self.list_tensors()

    def _resolve(self, name: str):
        if name in self._index.dense_names():
            return "dense", N.dense_key(name)
        for sep in ("@", "."):
            if sep in name:
                child, slot = name.rsplit(sep, 1)
                parts = self._index.table_parts(child, slot)
                if parts:
                    return "table", parts
        raise KeyError(f"tensor {name} not found in checkpoint")

    def read_tensor(self, name: str) -> torch.Tensor:
        kind, ref = self._resolve(name)
        if kind == "dense":
            return self._index.read(ref)
        return torch.cat([self._index.read(disk) for disk, *_ in ref])

    def tensor_shape(self, name: str) -> List[int]:
        kind, ref = self._resolve(name)
        if kind == "dense":
            return self._index.block_meta(ref)[3]
        shapes = [self._index.block_meta(disk)[3] for disk, *_ in ref]
        return [sum(s[0] for s in shapes)] + shapes[0][1:]

    def tensor_dtype(self, name: str) -> torch.dtype:
        kind, ref = self._resolve(name)
        return self._index.block_meta(ref if kind == "dense" else ref[0][0])[2]
