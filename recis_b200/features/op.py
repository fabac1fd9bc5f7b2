"""Feature transformation ops (``recis/features/op.py:129-686``): ``SelectField(s)``, ``Hash``, ``Mod``, ``Bucketize``,
``FeatureCross``, ``SequenceTruncate``, ``IDMultiHash``. Each op also runs stand-alone; inside a ``FeatureEngine`` ops of
the same kind at the same step are executed by one multi-tensor kernel (see ``fused_op_impl.py``)."""
from __future__ import annotations

import hashlib
import math
from typing import Dict, List, Union

import torch
from torch import nn

from ..nn.functional.array_ops import bucketize, bucketize_mod
from ..nn.functional.fused_ops import fused_multi_hash
from ..nn.functional.hash_ops import farmhash, murmurhash
from ..nn.functional.ragged_ops import feature_cross_ragged, fused_ragged_cutoff_2D, fused_ragged_cutoff_3D
from ..ragged.tensor import RaggedPadInfo, RaggedTensor


def values_of(x) -> torch.Tensor:
    """The flat value tensor of a RaggedTensor, a sparse COO tensor or a dense tensor (what a value-wise op works on)."""
    if isinstance(x, RaggedTensor):
        return x.values()
    if isinstance(x, torch.Tensor):
        return x._values() if x.is_sparse else x
    raise ValueError(f"Unsupported data type: {type(x)}")


def with_values(x, new_values: torch.Tensor):
    """``x`` with its values replaced: same offsets / weights / padding record (ragged), same indices (sparse), same shape
    (dense)."""
    if isinstance(x, RaggedTensor):
        out = RaggedTensor(new_values, x.offsets(), x.weight(), dense_shape=x._dense_shape)
        out.set_pad_info(x.pad_info)
        return out
    if x.is_sparse:
        return torch.sparse_coo_tensor(indices=x._indices(), values=new_values, size=x.shape)
    return new_values.reshape(x.shape)


class _OP(nn.Module):
    """Base of the ops: ``get_hash`` identifies an op by class and configuration, so that equal chains are computed once."""

    def _get_config(self) -> Dict:
        raise NotImplementedError

    def get_hash(self) -> int:
        text = repr((type(self).__name__, sorted(self._get_config().items())))
        return int.from_bytes(hashlib.blake2b(text.encode(), digest_size=8).digest(), "big", signed=True)


class SelectField(_OP):
    def __init__(self, name: str, dtype=torch.long, dim=None, from_dict=True):
        super().__init__()
        self._name, self._dtype, self._dim, self._from_dict = name, dtype, dim, from_dict

    def forward(self, data):
        if self._from_dict:
            assert isinstance(data, dict), f"data must be a dict, fn:{self._name}"
            x = data[self._name]
        else:
            x = data
        if isinstance(x, RaggedTensor) and self._dim and self._dim > 0:
            x.set_dim_by_rank(self._dim, -1)
        return x

    def _get_config(self):
        return {"name": self._name, "dtype": str(self._dtype), "dim": self._dim, "from_dict": self._from_dict}


class SelectFields(_OP):
    def __init__(self, input_list: List[SelectField]):
        super().__init__()
        self.input_list = nn.ModuleList(input_list)

    def forward(self, data):
        return [op(data) for op in self.input_list]

    def _get_config(self):
        return {"input_hashes": [op.get_hash() for op in self.input_list]}


class Mod(_OP):
    """Unsigned 64-bit modulo."""

    def __init__(self, mod_value):
        super().__init__()
        self.mod_value = int(mod_value)

    def forward(self, x):
        return with_values(x, bucketize_mod(values_of(x), self.mod_value))

    def _get_config(self):
        return {"mod": self.mod_value}


class Bucketize(_OP):
    """value -> number of boundaries <= value."""

    def __init__(self, boundary):
        super().__init__()
        self.boundary = torch.tensor(boundary, dtype=torch.float) if isinstance(boundary, (list, tuple)) else boundary.float()

    def forward(self, x):
        return with_values(x, bucketize(values_of(x), self.boundary))

    def _get_config(self):
        return {"boundary": self.boundary.tolist()}


class FeatureCross(_OP):
    def forward(self, data: List[RaggedTensor]):
        x, y = data
        assert isinstance(x, RaggedTensor) and isinstance(y, RaggedTensor)
        val, offsets, weight = feature_cross_ragged(x.values(), x.offsets()[-1], y.values(), y.offsets()[-1], x.weight(), y.weight())
        return RaggedTensor(values=val, offsets=offsets, weight=weight, dense_shape=(x._dense_shape[0], -1))

    def _get_config(self):
        return {}


class SequenceTruncate(_OP):
    """Keep at most ``seq_len`` entries per row (2-D) or exactly ``seq_len`` inner rows per sample (3-D)."""

    def __init__(self, seq_len=64, check_length=True, truncate=True, truncate_side="left", n_dims=2, dtype=torch.long):
        super().__init__()
        assert n_dims in (2, 3)
        assert truncate_side in ("left", "right")
        self.n_dims, self.seq_len, self.check_length, self.truncate = n_dims, int(seq_len), check_length, truncate
        self.truncate_side, self.dtype = truncate_side, dtype

    def sides(self):
        return self.truncate_side == "left", False

    def forward(self, x: RaggedTensor):
        if self.check_length and not self.truncate:
            assert x.shape[1] <= self.seq_len, f"sequence length must be less than {self.seq_len}"
        if not self.truncate:
            return x
        keep = torch.tensor([self.seq_len], dtype=torch.int32)
        drop = torch.tensor([self.truncate_side == "left"])
        pad = torch.tensor([False])
        return self.rebuild(x, *self.run([x], keep, drop, pad, self.n_dims))[0]

    @staticmethod
    def run(xs, keep, drop, pad, n_dims):
        if n_dims == 2:
            v, o, d, p, ds, ps = fused_ragged_cutoff_2D([x.values() for x in xs], [x.offsets()[-1] for x in xs], keep, drop, pad)
            return v, o, d, p
        v, o = fused_ragged_cutoff_3D([x.values() for x in xs], [x.offsets() for x in xs], keep, drop, pad)
        return v, o, [None] * len(xs), [None] * len(xs)

    def rebuild(self, x, values, offsets, drops, pads):
        outs = []
        for v, o, d, p in zip(values, offsets, drops, pads):
            shape = list(x._dense_shape)
            shape[1] = self.seq_len
            weight = x.weight()
            if weight is not None and weight.numel() != v.numel():
                weight = None      # weights cannot follow truncated values; re-derive them downstream if needed
            out = RaggedTensor(values=v, offsets=o, weight=weight, dense_shape=shape)
            if d is not None:
                out.set_pad_info(RaggedPadInfo(d, p, torch.tensor([self.truncate_side == "left"]), torch.tensor([False])))
            outs.append(out)
        return outs

    def _get_config(self):
        return {"seq_len": self.seq_len, "check_length": self.check_length, "truncate": self.truncate,
                "truncate_side": self.truncate_side, "n_dims": self.n_dims, "dtype": str(self.dtype)}


def _is_prime(x):
    return x >= 2 and all(x % n for n in range(2, int(math.isqrt(x)) + 1))


def _find_prime_lower_than(x):
    for n in range(x, 1, -1):
        if _is_prime(n):
            return n
    return 11


class IDMultiHash(_OP):
    """Up to four independent bucket hashes of an id: ``(((x*mul) % p + p) % p) % bucket`` with muls 1,3,5,7 and
    ``p`` the largest prime <= (29,47,67,83) * bucket. Returns a dict ``multi_hash_<i>``."""
    multi_muls = [1, 3, 5, 7]
    multi_mods = [29, 47, 67, 83]

    def __init__(self, num_buckets: List[int]):
        super().__init__()
        assert 0 < len(num_buckets) <= 4, "num_buckets must be a list of 1..4 integers"
        self.bucket_lens = len(num_buckets)
        self.num_buckets = [int(b) for b in num_buckets]
        self.primes = [_find_prime_lower_than(self.multi_mods[i] * self.num_buckets[i]) for i in range(self.bucket_lens)]
        self.muls = self.multi_muls[: self.bucket_lens]

    def forward(self, x):
        vals = x.values() if isinstance(x, RaggedTensor) else x
        outs = fused_multi_hash([vals], [self.muls], [self.primes], [self.num_buckets])
        return self.wrap(x, outs)

    def wrap(self, x, outs):
        if isinstance(x, RaggedTensor):
            return {f"multi_hash_{i}": RaggedTensor(outs[i], x.offsets(), x.weight(), dense_shape=x._dense_shape)
                    for i in range(self.bucket_lens)}
        return {f"multi_hash_{i}": outs[i] for i in range(self.bucket_lens)}

    def _get_config(self):
        return {"num_buckets": self.num_buckets, "multi_muls": self.multi_muls, "multi_mods": self.multi_mods}


class Hash(_OP):
    """Byte strings (int8 values, innermost offsets delimit strings) -> int64 ids; the innermost ragged dim disappears."""

    def __init__(self, hash_type: str):
        super().__init__()
        assert hash_type in ("farm", "murmur")
        self.hash_type = hash_type

    def forward(self, x: RaggedTensor):
        fn = farmhash if self.hash_type == "farm" else murmurhash
        return self.wrap(x, fn([x.values()], [x.offsets()[-1].int()])[0])

    @staticmethod
    def wrap(x, hashed):
        outer = x.offsets()[:-1]
        if not outer:        # a flat list of strings: one id per string
            return hashed
        return RaggedTensor(values=hashed, offsets=outer, weight=x.weight(), dense_shape=x._dense_shape[:-1])

    def _get_config(self):
        return {"hash_type": self.hash_type}
