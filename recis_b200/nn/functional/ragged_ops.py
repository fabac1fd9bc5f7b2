"""Ragged <-> dense / sparse conversions and ragged index utilities (filled in by ragged kernels)."""
from __future__ import annotations

from typing import List

import torch


def _row_lengths(offsets: torch.Tensor) -> torch.Tensor:
    return offsets[1:] - offsets[:-1]


def ragged_to_dense(values: torch.Tensor, offsets: List[torch.Tensor], default_value=0.0) -> torch.Tensor:
    """Pad a ragged tensor (any number of ragged dims) to a dense tensor."""
    if isinstance(offsets, torch.Tensor):
        offsets = [offsets]
    dev = values.device
    # flatten nested offsets from the innermost outwards
    cur = values
    for off in reversed(offsets):
        off = off.to(torch.int64)
        lens = _row_lengths(off)
        n_rows = lens.numel()
        max_len = int(lens.max().item()) if n_rows else 0
        inner_shape = tuple(cur.shape[1:])
        out = torch.full((n_rows, max_len) + inner_shape, default_value, dtype=cur.dtype, device=dev)
        if cur.shape[0]:
            row = torch.repeat_interleave(torch.arange(n_rows, device=dev), lens)
            col = torch.arange(cur.shape[0], device=dev) - off[:-1][row]
            out[row, col] = cur
        cur = out
    return cur


def dense_to_ragged(dense: torch.Tensor, check_invalid: bool = False, invalid_value=0):
    """2-D dense -> (values, [offsets]); with ``check_invalid`` trailing ``invalid_value`` entries are stripped."""
    assert dense.dim() == 2
    B, L = dense.shape
    if check_invalid:
        valid = dense != invalid_value
        idx = torch.arange(1, L + 1, device=dense.device).unsqueeze(0)
        lens = (valid * idx).max(dim=1).values if L else torch.zeros(B, dtype=torch.int64, device=dense.device)
    else:
        lens = torch.full((B,), L, dtype=torch.int64, device=dense.device)
    offsets = torch.zeros(B + 1, dtype=torch.int32, device=dense.device)
    offsets[1:] = torch.cumsum(lens, 0)
    mask = torch.arange(L, device=dense.device).unsqueeze(0) < lens.unsqueeze(1)
    return dense[mask], [offsets]


def ragged_to_sparse(values: torch.Tensor, offsets: List[torch.Tensor]) -> torch.Tensor:
    """COO tensor with one index row per ragged level (row-major positions)."""
    if isinstance(offsets, torch.Tensor):
        offsets = [offsets]
    dev = values.device
    n = values.shape[0]
    idx_rows = []
    pos = torch.arange(n, device=dev)
    shape = []
    for level in range(len(offsets) - 1, -1, -1):
        off = offsets[level].to(torch.int64)
        lens = _row_lengths(off)
        row = torch.repeat_interleave(torch.arange(lens.numel(), device=dev), lens)
        col = pos - off[:-1][row]
        idx_rows.append(col)
        shape.append(int(lens.max().item()) if lens.numel() else 0)
        pos = row
    idx_rows.append(pos)
    shape.append(offsets[0].numel() - 1)
    indices = torch.stack(list(reversed(idx_rows)))
    return torch.sparse_coo_tensor(indices, values, tuple(reversed(shape)))
