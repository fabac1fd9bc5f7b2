"""Feature: a named chain of ops that starts with ``SelectField``/``SelectFields`` (``recis/features/feature.py:9-143``)."""
from __future__ import annotations

import hashlib
from typing import List

from torch import nn

from .op import _OP, SelectField, SelectFields


class Feature(nn.Module):
    def __init__(self, name: str):
        super().__init__()
        self._name = name
        self._compiled = False
        self._ops = nn.ModuleList()
        self._buffers_data = None

    def set_buffers_data(self, data):
        """Attach side data to the feature (``recis/features/feature.py:58-59``); the feature itself does not read it."""
        self._buffers_data = data

    @property
    def name(self):
        return self._name

    @property
    def compiled(self):
        return self._compiled

    def compiled_(self, value: bool):
        assert isinstance(value, bool)
        self._compiled = value

    @property
    def ops(self) -> List[nn.Module]:
        return self._ops

    def add_op(self, op: _OP):
        if self._compiled:
            raise ValueError(f"feature {self.name} has been compiled")
        if len(self._ops) == 0 and type(op) not in (SelectField, SelectFields):
            raise ValueError(f"feature {self.name} must start with DataInputOP")
        self._ops.append(op)
        return self

    @property
    def id(self):
        return id(self)

    @staticmethod
    def from_json(json_obj):
        """``{"name": ..., "ops": [{"type": "Mod", "mod_value": 7}, ...]}`` -> Feature (the reference declares this entry point
        without implementing it, ``recis/features/feature.py:110-111``)."""
        from . import op as ops
        f = Feature(json_obj["name"])
        for spec in json_obj.get("ops", []):
            spec = dict(spec)
            cls = getattr(ops, spec.pop("type"))
            f.add_op(cls(**spec))
        return f

    def get_hash(self) -> int:
        """Identity of the op chain: the ops' own hashes in chain order. The feature's name is not part of it, so two features
        that run the same chain on the same input are computed once by the engine and the second becomes an alias of the first
        (the reference mixes the name in, ``recis/features/feature.py:112-125``, which limits this to exact duplicates)."""
        if len(self._ops) == 0:
            return 0
        chain = ",".join(str(op.get_hash()) for op in self._ops)
        return int.from_bytes(hashlib.blake2b(chain.encode(), digest_size=8).digest(), "big", signed=True)

    def forward(self, data):
        x = data
        for op in self._ops:
            x = op(x)
        return x
