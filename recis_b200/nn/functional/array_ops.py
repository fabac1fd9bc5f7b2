"""Single-tensor feature transforms (``recis/nn/functional/array_ops.py``): thin wrappers over the fused kernels."""
from __future__ import annotations

import torch

from ... import native


def bucketize(input: torch.Tensor, boundaries: torch.Tensor) -> torch.Tensor:
    """Number of boundaries ``<= value`` for every value (int64)."""
    return native().fused_bucketize([input], [boundaries])[0]


def bucketize_mod(input: torch.Tensor, bucket: int) -> torch.Tensor:
    """``uint64(x) % bucket``."""
    return native().fused_mod([input], [int(bucket)])[0]


def multi_hash(input: torch.Tensor, muls, primes, bucket_num):
    """``(((x * mul) % prime + prime) % prime) % bucket`` for up to four (mul, prime, bucket) triples."""
    to_list = lambda t: [int(v) for v in (t.tolist() if isinstance(t, torch.Tensor) else t)]
    return native().fused_multi_hash([input], [to_list(muls)], [to_list(primes)], [to_list(bucket_num)])[0]
