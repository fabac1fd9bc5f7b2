"""Names and small formats of the sparse checkpoint bundle (layout of the reference's ``csrc/serialize``:
``name.cc:58-152``, ``save_bundle.cc:83-111``, ``dtype_serialize.cc:4-66``, ``index_info.cc:15-127``)."""
from __future__ import annotations

import os

import torch

INDEX_FILE = "index"
TENSORKEY_FILE = "tensorkey.json"
RANK_JSON_FILE = "torch_rank_weights_embs_table_multi_shard.json"
ID_SLOT = "id"
EMB_SLOT = "embedding"
FILTER_SLOT = "step_filter"

_DT = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int64: "I64",
       torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}
_DT_INV = {v: k for k, v in _DT.items()}
_DT_INV["bool"] = torch.bool          # the reference writes lowercase "bool" (dtype_serialize.cc:5); accept both spellings
_RANK_JSON_DT = {"F64": "float64", "F32": "float32", "F16": "float16", "BF16": "bfloat16", "I64": "int64", "I32": "int32",
                 "I16": "int16", "I8": "int8", "U8": "uint8", "BOOL": "bool"}


def dtype_to_str(dt: torch.dtype) -> str:
    return _DT[dt]


def str_to_dtype(s: str) -> torch.dtype:
    return _DT_INV[s]


def rank_json_dtype(s: str) -> str:
    return _RANK_JSON_DT.get(s, s)


def data_file_name(idx: int, total: int) -> str:
    return f"model-{idx:06d}-of-{total:06d}.safetensors"


def slice_str(beg: int, end: int, size: int) -> str:
    """``beg@end@size`` with begin and end zero-padded to the width of ``size``, e.g. ``08192@16384@65536``
    (``csrc/embedding/slice_info.cc:38-48`` in the reference)."""
    width = len(str(size))
    return f"{beg:0{width}d}@{end:0{width}d}@{size}"


def block_name(child: str, slot: str, sl) -> str:
    """Internal block name ``<child>@<slot>^<beg>@<end>@<size>``."""
    return f"{child}@{slot}^{slice_str(sl.slice_begin, sl.slice_end, sl.slice_size)}"


def disk_key(child: str, slot: str, shard: int, shard_num: int) -> str:
    """On-disk key of a table block: ``<child>.<slot>/part_<shard>_<shard_num>``."""
    return f"{child}.{slot}/part_{shard}_{shard_num}"


def dense_key(name: str) -> str:
    """On-disk key of a dense tensor: name, separator, and a single space as (empty) slice info."""
    return f"{name}^ "


def parse_block_name(block: str):
    """``child@slot^beg@end@size`` -> (child, slot, beg, end, size)."""
    tensor, sl = block.split("^")
    child, slot = tensor.rsplit("@", 1)
    beg, end, size = (int(x) for x in sl.split("@"))
    return child, slot, beg, end, size


def join(path, *names):
    return os.path.join(path, *names)
