"""Row initializers for dynamic embedding tables.

Same eight classes and constructor arguments as the reference (``recis/nn/initializers.py:7-698``). The
implementation differs: the reference fills whole ``[block_size, dim]`` blocks from the ATen RNG stream, so a
row's initial value depends on the order in which rows were allocated. Here an initializer only resolves to a
small spec ``(kind, a, b, lo, hi, seed)``; the table's insert kernel draws the row of id ``k`` with a
counter-based Philox keyed on ``(seed, k, column)``. The distribution is the same, and a seeded run gives the
same values on CPU and GPU and for any number of shards.
"""
from __future__ import annotations

import json
import math
from typing import Optional

import torch

KIND_CONSTANT, KIND_UNIFORM, KIND_NORMAL, KIND_TRUNC_NORMAL = 0, 1, 2, 3


def _calc_gain(nonlinearity: str, a: float) -> float:
    return torch.nn.init.calculate_gain(nonlinearity, a)


class Initializer:
    """Base class: configure, ``set_shape``/``set_dtype``, ``build`` and then ``generate`` or ``spec``."""

    def __init__(self, generator: Optional[torch.Generator] = None) -> None:
        self._impl = None
        self._shape = None
        self._dtype = torch.float32
        self._generator = generator

    def set_shape(self, shape=None):
        self._shape = list(shape) if shape is not None else None

    def set_dtype(self, dtype: torch.dtype = torch.float32):
        self._dtype = dtype

    def _fans(self):
        shape = self._shape or [1, 1]
        if len(shape) < 2:
            return shape[0], shape[0]
        receptive = 1
        for s in shape[2:]:
            receptive *= s
        return shape[1] * receptive, shape[0] * receptive

    def seed(self) -> int:
        if self._generator is not None:
            return int(self._generator.initial_seed())
        return int(torch.initial_seed())

    def _spec(self):
        raise NotImplementedError

    def build(self):
        if self._impl is not None:
            raise RuntimeError("rebuild initializer")
        kind, a, b, lo, hi = self._spec()
        self._impl = (kind, float(a), float(b), float(lo), float(hi), self.seed() & 0x7FFFFFFFFFFFFFFF)

    def impl(self):
        return self._impl

    def spec(self):
        """``(kind, a, b, lo, hi, seed)`` consumed by the native table."""
        if self._impl is None:
            self.build()
        return self._impl

    def generate(self) -> torch.Tensor:
        """A tensor of the configured shape drawn from this initializer (host-side, for dense use and tests)."""
        if self._impl is None:
            raise RuntimeError("build method is not called.")
        kind, a, b, lo, hi, _seed = self._impl
        shape = self._shape
        g = self._generator
        if kind == KIND_CONSTANT:
            return torch.full(shape, a, dtype=self._dtype)
        if kind == KIND_UNIFORM:
            return torch.empty(shape, dtype=self._dtype).uniform_(a, b, generator=g)
        if kind == KIND_NORMAL:
            return torch.empty(shape, dtype=self._dtype).normal_(a, b, generator=g)
        t = torch.empty(shape, dtype=torch.float32)
        torch.nn.init.trunc_normal_(t, mean=a, std=b, a=lo, b=hi, generator=g)
        return t.to(self._dtype)

    def _info(self):
        raise NotImplementedError

    def __str__(self):
        info = self._info()
        info.update(
            shape=str(self._shape),
            dtype=str(self._dtype),
            generator_seed=self._generator.seed() if self._generator else None,
        )
        return json.dumps(info, sort_keys=True)


class ConstantInitializer(Initializer):
    def __init__(self, init_val: float = 0.0, dtype: torch.dtype = torch.float32) -> None:
        super().__init__()
        self._init_val = init_val

    def _spec(self):
        return KIND_CONSTANT, self._init_val, 0.0, 0.0, 0.0

    def _info(self):
        return {"type": "ConstantInitializer", "init_val": self._init_val}


class UniformInitializer(Initializer):
    def __init__(self, a: float = 0.0, b: float = 1.0, generator: Optional[torch.Generator] = None) -> None:
        super().__init__(generator)
        self._a, self._b = a, b

    def _spec(self):
        return KIND_UNIFORM, self._a, self._b, 0.0, 0.0

    def _info(self):
        return {"type": "UniformInitializer", "a": self._a, "b": self._b}


class NormalInitializer(Initializer):
    def __init__(self, mean: float = 0.0, std: float = 1.0, generator: Optional[torch.Generator] = None) -> None:
        super().__init__(generator)
        self._mean, self._std = mean, std

    def _spec(self):
        return KIND_NORMAL, self._mean, self._std, 0.0, 0.0

    def _info(self):
        return {"type": "NormalInitializer", "mean": self._mean, "std": self._std}


class XavierUniformInitializer(Initializer):
    def __init__(self, gain: float = 1.0, generator: Optional[torch.Generator] = None) -> None:
        super().__init__(generator)
        self._gain = gain

    def _spec(self):
        fan_in, fan_out = self._fans()
        bound = self._gain * math.sqrt(6.0 / (fan_in + fan_out))
        return KIND_UNIFORM, -bound, bound, 0.0, 0.0

    def _info(self):
        return {"type": "XavierUniformInitializer", "gain": self._gain}


class XavierNormalInitializer(Initializer):
    def __init__(self, gain: float = 1.0, generator: Optional[torch.Generator] = None) -> None:
        super().__init__(generator)
        self._gain = gain

    def _spec(self):
        fan_in, fan_out = self._fans()
        return KIND_NORMAL, 0.0, self._gain * math.sqrt(2.0 / (fan_in + fan_out)), 0.0, 0.0

    def _info(self):
        return {"type": "XavierNormalInitializer", "gain": self._gain}


class _Kaiming(Initializer):
    def __init__(self, a: float = 0.0, mode: str = "fan_in", nonlinearity: str = "leaky_relu",
                 generator: Optional[torch.Generator] = None) -> None:
        super().__init__(generator)
        if mode not in ("fan_in", "fan_out"):
            raise ValueError(f"{mode} not in [fan_in, fan_out]")
        self._a, self._mode, self._nonlinearity = a, mode, nonlinearity

    def _std(self):
        fan_in, fan_out = self._fans()
        fan = fan_in if self._mode == "fan_in" else fan_out
        return _calc_gain(self._nonlinearity, self._a) / math.sqrt(fan)

    def _info(self):
        return {"type": type(self).__name__, "a": self._a, "mode": self._mode, "nonlinearity": self._nonlinearity}


class KaimingUniformInitializer(_Kaiming):
    def _spec(self):
        bound = math.sqrt(3.0) * self._std()
        return KIND_UNIFORM, -bound, bound, 0.0, 0.0


class KaimingNormalInitializer(_Kaiming):
    """Normal variant. (The reference's wrapper builds the *uniform* generator here,
    ``recis/nn/initializers.py:585``; this one draws from the normal distribution its name promises.)"""

    def _spec(self):
        return KIND_NORMAL, 0.0, self._std(), 0.0, 0.0


class TruncNormalInitializer(Initializer):
    """Normal(mean, std) resampled into ``[mean + a*std, mean + b*std]`` (a, b in units of std)."""

    def __init__(self, mean: float = 0.0, std: float = 1.0, a: float = -2.0, b: float = 2.0,
                 generator: Optional[torch.Generator] = None) -> None:
        super().__init__(generator)
        self._mean, self._std, self._a, self._b = mean, std, a, b

    def _spec(self):
        return (KIND_TRUNC_NORMAL, self._mean, self._std, self._mean + self._a * self._std,
                self._mean + self._b * self._std)

    def _info(self):
        return {"type": "TruncNormalInitializer", "mean": self._mean, "std": self._std, "a": self._a, "b": self._b}
