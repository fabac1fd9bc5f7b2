"""Fused executors: all ops of one kind at one execution step run as ONE multi-tensor kernel
(``recis/features/fused_op_impl.py:26-516``: ``FusedBoundaryOP/ModOP/HashOP/CutoffOP/MultiHashOP``)."""
from __future__ import annotations

from typing import List

import torch

from .. import native
from ..ragged.tensor import RaggedTensor
from .op import Bucketize, Hash, IDMultiHash, Mod, SequenceTruncate, values_of, with_values


class _FusedOP:
    def __init__(self, ops=None):
        self._ops = list(ops or [])

    def add_op(self, op):
        self._ops.append(op)

    def __call__(self, inputs: List):
        assert len(inputs) == len(self._ops)
        return self.process(inputs)

    def process(self, inputs: List):
        raise NotImplementedError


class FusedBoundaryOP(_FusedOP):
    def process(self, inputs):
        outs = native().fused_bucketize([values_of(x) for x in inputs], [op.boundary for op in self._ops])
        return [with_values(x, o) for x, o in zip(inputs, outs)]


class FusedModOP(_FusedOP):
    def process(self, inputs):
        outs = native().fused_mod([values_of(x) for x in inputs], [op.mod_value for op in self._ops])
        return [with_values(x, o) for x, o in zip(inputs, outs)]


class FusedHashOP(_FusedOP):
    def process(self, inputs):
        outs = [None] * len(inputs)
        for kind, name in ((0, "farm"), (1, "murmur")):
            idx = [i for i, op in enumerate(self._ops) if op.hash_type == name]
            if not idx:
                continue
            hashed = native().fused_hash([inputs[i].values() for i in idx], [inputs[i].offsets()[-1].int() for i in idx], kind)
            for i, h in zip(idx, hashed):
                outs[i] = Hash.wrap(inputs[i], h)
        return outs


class FusedCutoffOP(_FusedOP):
    def process(self, inputs):
        outs = [None] * len(inputs)
        for n_dims in (2, 3):
            idx = [i for i, op in enumerate(self._ops) if op.n_dims == n_dims and op.truncate]
            if not idx:
                continue
            keep = torch.tensor([self._ops[i].seq_len for i in idx], dtype=torch.int32)
            drop = torch.tensor([self._ops[i].truncate_side == "left" for i in idx])
            pad = torch.zeros(len(idx), dtype=torch.bool)
            v, o, d, p = SequenceTruncate.run([inputs[i] for i in idx], keep, drop, pad, n_dims)
            for k, i in enumerate(idx):
                outs[i] = self._ops[i].rebuild(inputs[i], [v[k]], [o[k]], [d[k]], [p[k]])[0]
        for i, op in enumerate(self._ops):
            if outs[i] is None:
                outs[i] = op(inputs[i])
        return outs


class FusedMultiHashOP(_FusedOP):
    def process(self, inputs):
        vals = [x.values() if isinstance(x, RaggedTensor) else x for x in inputs]
        res = native().fused_multi_hash(vals, [op.muls for op in self._ops], [op.primes for op in self._ops],
                                        [op.num_buckets for op in self._ops])
        return [op.wrap(x, r) for op, x, r in zip(self._ops, inputs, res)]


class FusedOpFactory:
    _registry = {Bucketize: FusedBoundaryOP, Mod: FusedModOP, Hash: FusedHashOP, SequenceTruncate: FusedCutoffOP,
                 IDMultiHash: FusedMultiHashOP}

    @staticmethod
    def register(op_class: type, fused_op_class: type):
        FusedOpFactory._registry[op_class] = fused_op_class

    @staticmethod
    def contains(op) -> bool:
        return type(op) in FusedOpFactory._registry

    @staticmethod
    def get_fused_op(op):
        return FusedOpFactory._registry[type(op)]
