"""Input validation that is too expensive for the hot path (it reads device memory on the host): enabled with
``RECIS_DEBUG_BOUNDS=1``. The kernels themselves are memory safe against the failures they can detect cheaply (arena full,
window overflow, unknown ids) and report those through status words; malformed ragged inputs (offsets that do not start at
zero, decrease, or point past the values) are the caller's contract and are checked here when debugging."""
from __future__ import annotations

import os

import torch


def enabled() -> bool:
    return os.environ.get("RECIS_DEBUG_BOUNDS") == "1"


def check_ragged(name: str, values: torch.Tensor, offsets: torch.Tensor, weights: torch.Tensor = None):
    """Raise ``ValueError`` if ``offsets`` is not a valid row partition of ``values`` (or ``weights`` has another length)."""
    if offsets.numel() == 0:
        raise ValueError(f"{name}: offsets must hold at least one entry")
    off = offsets.detach().to("cpu", torch.int64)
    if int(off[0]) != 0:
        raise ValueError(f"{name}: offsets must start at 0, got {int(off[0])}")
    if off.numel() > 1 and bool((off[1:] < off[:-1]).any()):
        bad = int(torch.nonzero(off[1:] < off[:-1])[0])
        raise ValueError(f"{name}: offsets decrease at position {bad + 1} ({int(off[bad])} -> {int(off[bad + 1])})")
    if int(off[-1]) != values.numel():
        raise ValueError(f"{name}: last offset {int(off[-1])} does not match the number of values {values.numel()}")
    if weights is not None and weights.numel() != values.numel():
        raise ValueError(f"{name}: {weights.numel()} weights for {values.numel()} values")
    if values.dtype.is_floating_point:
        raise ValueError(f"{name}: ids must be integers, got {values.dtype}")
