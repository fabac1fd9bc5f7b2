"""String hashing (``recis/nn/functional/hash_ops.py``): byte tensors + int32 offsets -> int64 hashes, several tensors per
launch. FarmHash Fingerprint64 and MurmurHash64A (seed 0), bit-identical to the reference; unlike the reference's op
(CUDA only, ``csrc/ops/fused_hash.cc:15-19``) both run on CPU tensors too."""
from __future__ import annotations

from typing import List

import torch

from ... import native


def farmhash(inputs: List[torch.Tensor], splits: List[torch.Tensor]) -> List[torch.Tensor]:
    return native().fused_hash(list(inputs), list(splits), 0)


def murmurhash(inputs: List[torch.Tensor], splits: List[torch.Tensor]) -> List[torch.Tensor]:
    return native().fused_hash(list(inputs), list(splits), 1)
