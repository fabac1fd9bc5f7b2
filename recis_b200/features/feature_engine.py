"""FeatureEngine (``recis/features/feature_engine.py:107-284``): features with identical configuration are computed once;
execution is compiled step-wise (step k = k-th op of every feature) and fusable ops of one kind inside a step run as one
multi-tensor kernel."""
from __future__ import annotations

from collections import defaultdict
from typing import Dict, List

from torch import nn

from .feature import Feature
from .fused_op_impl import FusedOpFactory
from .op import _OP


class RunContext:
    def __init__(self, input_data, remain_no_use_data: bool = True):
        self._data_buffer = {}
        self._input_data = input_data
        self._remain_no_use_data = remain_no_use_data

    def get(self, key):
        return self._data_buffer[key] if key in self._data_buffer else self._input_data

    def set(self, key, value):
        self._data_buffer[key] = value

    @property
    def results(self):
        if self._remain_no_use_data:
            for k, v in self._input_data.items():
                self._data_buffer.setdefault(k, v)
        return self._data_buffer


class FuseExecutionGroup:
    def __init__(self, op: _OP):
        self._feature_names = []
        self._fused_op = FusedOpFactory.get_fused_op(op)(ops=[])

    def add_op(self, feature_name: str, op: _OP):
        self._feature_names.append(feature_name)
        self._fused_op.add_op(op)

    def run(self, data: RunContext):
        outputs = self._fused_op([data.get(name) for name in self._feature_names])
        for name, output in zip(self._feature_names, outputs):
            data.set(name, output)
        return data


class NonFuseExecutionGroup:
    def __init__(self):
        self._ops, self._feature_names = [], []

    def add_op(self, feature_name: str, op: _OP):
        self._ops.append(op)
        self._feature_names.append(feature_name)

    def run(self, data: RunContext):
        for op, name in zip(self._ops, self._feature_names):
            data.set(name, op(data.get(name)))
        return data


class ExecutionStep:
    _non_fuseable_tag = "_non_fuseable_tag"

    def __init__(self):
        self.execution_groups = {}

    def add_op(self, feature_name: str, op: _OP):
        if FusedOpFactory.contains(op):
            key = type(op).__name__
            if key not in self.execution_groups:
                self.execution_groups[key] = FuseExecutionGroup(op)
        else:
            key = self._non_fuseable_tag
            if key not in self.execution_groups:
                self.execution_groups[key] = NonFuseExecutionGroup()
        self.execution_groups[key].add_op(feature_name, op)
        return self

    def run(self, data: RunContext):
        for group in self.execution_groups.values():
            data = group.run(data)
        return data


class FeatureEngine(nn.Module):
    def __init__(self, feature_list: List[Feature]):
        super().__init__()
        self._features = nn.ModuleDict()
        self._hash_cache_map = {}
        by_hash = defaultdict(list)
        for feature in feature_list:
            by_hash[feature.get_hash()].append(feature)
        for features in by_hash.values():
            primary = features[0]
            if primary.name in self._features:
                raise ValueError(f"Duplicate feature name: {primary.name}")
            self._features[primary.name] = primary
            for dup in features[1:]:
                self._hash_cache_map[dup.name] = primary.name
        self.execution_steps = self._compile(list(self._features.values()))

    @staticmethod
    def _compile(features: List[Feature]):
        for f in features:
            if f.compiled:
                raise ValueError(f"feature {f.name} has been compiled")
            f.compiled_(True)
        steps, k = [], 0
        while True:
            step, done = ExecutionStep(), True
            for f in features:
                if len(f.ops) > k:
                    step.add_op(f.name, f.ops[k])
                    done = False
            if done:
                break
            steps.append(step)
            k += 1
        return steps

    def forward(self, data: Dict, remain_no_use_data: bool = True) -> Dict:
        assert isinstance(data, dict), "data must be a dict"
        ctx = RunContext(data, remain_no_use_data)
        for step in self.execution_steps:
            ctx = step.run(ctx)
        results = ctx.results
        for name, primary in self._hash_cache_map.items():
            results[name] = results[primary]
        return results
