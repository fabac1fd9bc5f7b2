"""Seeded synthetic recommendation batches (no dataset on disk).

Power-law ids use the inverse CDF of a continuous Zipf law on ``[1, N]``
(``rank = ((N^(1-a) - 1) u + 1)^(1/(1-a))``), optionally folded onto a fixed universe of distinct ids that are
scattered over the id space with a 64-bit mixer, so that "about U unique rows over a 2^k id space" holds by
construction. Bag lengths are Poisson / geometric / uniform / fixed, clipped. Everything is generated on the
host into (optionally pinned) tensors: a training step then pays the real host-to-device copy.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from ..ragged.tensor import RaggedTensor

_M1 = np.uint64(0xbf58476d1ce4e5b9)
_M2 = np.uint64(0x94d049bb133111eb)


def mix64(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.uint64, copy=True)
    with np.errstate(over="ignore"):
        x ^= x >> np.uint64(30); x *= _M1
        x ^= x >> np.uint64(27); x *= _M2
        x ^= x >> np.uint64(31)
    return x


def zipf_ranks(rng: np.random.Generator, n: int, a: float, N: float) -> np.ndarray:
    """n ranks in [1, N] with P(rank) ~ rank^-a (continuous approximation, a != 1)."""
    u = rng.random(n)
    one_minus_a = 1.0 - a
    x = ((N ** one_minus_a - 1.0) * u + 1.0) ** (1.0 / one_minus_a)
    return np.minimum(np.floor(x), N).astype(np.uint64)


def zipf_ids(rng, n, a, id_bits=40, universe=None, salt=0) -> np.ndarray:
    ranks = zipf_ranks(rng, n, a, float(2 ** id_bits))
    if universe:
        ranks = ranks % np.uint64(universe)
    with np.errstate(over="ignore"):
        salted = ranks + np.uint64((salt * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)
    ids = mix64(salted) & np.uint64((1 << id_bits) - 1)
    return ids.astype(np.int64)


def bag_lengths(rng, batch, kind="fixed", mean=1.0, lo=1, hi=100, p=0.2) -> np.ndarray:
    if kind == "fixed":
        return np.full(batch, int(mean), dtype=np.int64)
    if kind == "poisson":
        return np.clip(rng.poisson(mean, batch), lo, hi).astype(np.int64)
    if kind == "geometric":
        return np.clip(rng.geometric(p, batch), lo, hi).astype(np.int64)
    if kind == "uniform":
        return rng.integers(lo, hi + 1, batch).astype(np.int64)
    raise ValueError(kind)


@dataclass
class SparseFieldSpec:
    name: str
    zipf_a: float = 1.05
    id_bits: int = 40
    universe: Optional[int] = None
    length: str = "fixed"          # fixed | poisson | geometric | uniform
    mean_len: float = 1.0
    min_len: int = 1
    max_len: int = 100
    geo_p: float = 0.2


@dataclass
class SyntheticSpec:
    batch: int
    dense_dim: int = 13
    sparse: List[SparseFieldSpec] = field(default_factory=list)
    label_rate: float = 0.25
    seed: int = 0


def make_batch_arrays(spec: SyntheticSpec, step: int) -> Dict[str, object]:
    """One batch as numpy arrays: ``dense`` [B, dense_dim] fp32 (log1p of lognormal), ``label`` [B, 1] fp32 and, per
    sparse field, a tuple ``(ids int64 [nnz], offsets int32 [B+1])``."""
    rng = np.random.default_rng([spec.seed, step])
    B = spec.batch
    out: Dict[str, object] = {}
    if spec.dense_dim:
        out["dense"] = np.log1p(rng.lognormal(0.0, 1.0, (B, spec.dense_dim))).astype(np.float32)
    out["label"] = (rng.random((B, 1)) < spec.label_rate).astype(np.float32)
    for k, f in enumerate(spec.sparse):
        lens = bag_lengths(rng, B, f.length, f.mean_len, f.min_len, f.max_len, f.geo_p)
        offsets = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(lens, out=offsets[1:])
        ids = zipf_ids(rng, int(offsets[-1]), f.zipf_a, f.id_bits, f.universe, salt=k + 1)
        out[f.name] = (ids, offsets)
    return out


def make_batch(spec: SyntheticSpec, step: int, pin: bool = False) -> Dict[str, object]:
    """``make_batch_arrays`` as (optionally pinned) torch tensors, one RaggedTensor per sparse field."""

    def t(arr):
        x = torch.from_numpy(np.ascontiguousarray(arr))
        return x.pin_memory() if pin else x

    out: Dict[str, object] = {}
    for k, v in make_batch_arrays(spec, step).items():
        if isinstance(v, tuple):
            out[k] = RaggedTensor(t(v[0]), [t(v[1])], dense_shape=(spec.batch, -1))
        else:
            out[k] = t(v)
    return out


def to_device(batch: Dict[str, object], device, non_blocking=True) -> Dict[str, object]:
    out = {}
    for k, v in batch.items():
        if isinstance(v, (torch.Tensor, RaggedTensor)):
            out[k] = v.to(device, non_blocking=non_blocking)
        else:
            out[k] = v
    return out


def batch_nbytes(batch: Dict[str, object]) -> int:
    n = 0
    for v in batch.values():
        if isinstance(v, torch.Tensor):
            n += v.numel() * v.element_size()
        elif isinstance(v, RaggedTensor):
            n += v.values().numel() * v.values().element_size()
            n += sum(o.numel() * o.element_size() for o in v.offsets())
            if v.weight() is not None:
                n += v.weight().numel() * v.weight().element_size()
    return n
