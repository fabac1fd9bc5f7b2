"""FeatureEngine: many op chains, few kernel launches.

Behaviour of the reference's engine (``recis/features/feature_engine.py:107-284``): features with an identical configuration are
computed once and aliased; the k-th ops of all features form step k; inside a step, ops of one fusable kind (Hash, Mod,
Bucketize, SequenceTruncate, IDMultiHash) are executed by ONE multi-tensor call, the others one by one.

Here the compiled form is a flat *plan*: a list of steps, each a list of ``_Launch`` records ``(kind, callable, feature
names)``. Running the plan is two nested loops over those records with a plain dict as the working set; nothing else is
allocated per call.
"""
from __future__ import annotations

from typing import Dict, List, NamedTuple, Sequence

from torch import nn

from .feature import Feature
from .fused_op_impl import FusedOpFactory

_SINGLE = "single"          # plan kind of ops that have no fused executor


class _Launch(NamedTuple):
    kind: str               # fused kind ("Hash", "Mod", ...) or _SINGLE
    fn: object              # fused executor over a list of inputs, or the op itself
    names: tuple            # features whose current value goes in and is replaced by the result


def _plan_step(column: Sequence[tuple]) -> List[_Launch]:
    """``column`` = [(feature name, op)] of one step -> launches: one per fusable kind (in order of first appearance), then the
    remaining ops one by one."""
    fused: Dict[str, list] = {}
    singles: List[_Launch] = []
    for name, op in column:
        if FusedOpFactory.contains(op):
            fused.setdefault(type(op).__name__, []).append((name, op))
        else:
            singles.append(_Launch(_SINGLE, op, (name,)))
    launches = []
    for kind, members in fused.items():
        executor = FusedOpFactory.get_fused_op(members[0][1])(ops=[])
        for _name, op in members:
            executor.add_op(op)
        launches.append(_Launch(kind, executor, tuple(n for n, _ in members)))
    return launches + singles


class FeatureEngine(nn.Module):
    def __init__(self, feature_list: List[Feature]):
        super().__init__()
        self._features = nn.ModuleDict()
        self._alias = {}                        # name of a duplicate feature -> name of the feature that is computed
        first_with = {}
        for feature in feature_list:
            key = feature.get_hash()
            if key in first_with:
                self._alias[feature.name] = first_with[key]
                continue
            if feature.name in self._features:
                raise ValueError(f"Duplicate feature name: {feature.name}")
            first_with[key] = feature.name
            self._features[feature.name] = feature
        self.plan = self._compile(list(self._features.values()))

    @staticmethod
    def _compile(features: List[Feature]) -> List[List[_Launch]]:
        for f in features:
            if f.compiled:
                raise ValueError(f"feature {f.name} has been compiled")
            f.compiled_(True)
        depth = max((len(f.ops) for f in features), default=0)
        return [_plan_step([(f.name, f.ops[k]) for f in features if len(f.ops) > k]) for k in range(depth)]

    def forward(self, data: Dict, remain_no_use_data: bool = True) -> Dict:
        """``data``: column name -> tensor / RaggedTensor. Returns feature name -> result; with ``remain_no_use_data`` the input
        columns that no feature overwrote are passed through."""
        assert isinstance(data, dict), "data must be a dict"
        cur: Dict[str, object] = {}
        for step in self.plan:
            for launch in step:
                if launch.kind == _SINGLE:
                    (name,) = launch.names
                    cur[name] = launch.fn(cur.get(name, data))      # a chain's first op (SelectField) reads the input dict
                else:
                    results = launch.fn([cur.get(name, data) for name in launch.names])
                    cur.update(zip(launch.names, results))
        if remain_no_use_data:
            for column, value in data.items():
                cur.setdefault(column, value)
        for duplicate, computed in self._alias.items():
            cur[duplicate] = cur[computed]
        return cur
