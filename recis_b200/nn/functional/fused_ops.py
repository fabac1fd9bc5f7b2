"""Multi-tensor ("fused") feature transforms (``recis/nn/functional/fused_ops.py``): one launch for a list of tensors.
The ``_gpu`` suffixed names of the reference are kept; the functions run on CPU tensors as well."""
from __future__ import annotations

from typing import List

import torch

from ... import native


def _to_list(t):
    return [int(v) for v in (t.tolist() if isinstance(t, torch.Tensor) else t)]


def fused_bucketize_gpu(values: List[torch.Tensor], boundaries: List[torch.Tensor]) -> List[torch.Tensor]:
    return native().fused_bucketize(list(values), list(boundaries))


def fused_uint64_mod_gpu(values: List[torch.Tensor], mods) -> List[torch.Tensor]:
    mods = _to_list(mods) if not isinstance(mods, (list, tuple)) or (mods and isinstance(mods[0], torch.Tensor)) is False else \
        [int(m.item()) for m in mods]
    return native().fused_mod(list(values), [int(m) for m in mods])


def fused_ids_encode_gpu(ids_list: List[torch.Tensor], table_ids) -> torch.Tensor:
    """Concatenate id tensors, replacing the top 12 bits of every id with its table index."""
    from .embedding_ops import ids_encode
    return ids_encode(ids_list, table_ids)


def fused_multi_hash(inputs: List[torch.Tensor], muls: List[torch.Tensor], primes: List[torch.Tensor],
                     bucket_nums: List[torch.Tensor]) -> List[torch.Tensor]:
    """Returns the outputs of all tensors flattened tensor-major (tensor 0's hashes first), as the reference does."""
    res = native().fused_multi_hash(list(inputs), [_to_list(m) for m in muls], [_to_list(p) for p in primes],
                                    [_to_list(b) for b in bucket_nums])
    return [t for per_tensor in res for t in per_tensor]
