"""Ragged-tensor functional ops (API of the reference's ``recis/nn/functional/ragged_ops.py``), each backed by one native
implementation that runs as sm_100a kernels on CUDA tensors and as C++ loops on CPU tensors."""
from __future__ import annotations

from typing import List, Optional

import torch

from ... import native


def ragged_to_dense(values: torch.Tensor, offsets: List[torch.Tensor], default_value=0.0) -> torch.Tensor:
    """Pad a ragged tensor (1..5 ragged dims, offsets outermost first) to a dense tensor."""
    if isinstance(offsets, torch.Tensor):
        offsets = [offsets]
    return native().ragged_to_dense(values, list(offsets), float(default_value))


def dense_to_ragged(tensor: torch.Tensor, check_invalid: bool = False, invalid_value=0):
    """2-D dense -> ``(values, [offsets])``; with ``check_invalid`` trailing ``invalid_value`` entries are stripped."""
    values, offsets = native().dense_to_ragged(tensor, bool(check_invalid), float(invalid_value))
    return values, [offsets]


def ragged_to_sparse(values: torch.Tensor, row_splits: List[torch.Tensor]) -> torch.Tensor:
    """COO tensor of a ragged tensor (runs on either device; the reference's op is CPU-only)."""
    if isinstance(row_splits, torch.Tensor):
        row_splits = [row_splits]
    indices, shape = native().ragged_to_sparse_indices(values.shape[0], list(row_splits))
    return torch.sparse_coo_tensor(indices, values, tuple(shape) + tuple(values.shape[1:]))


def gen_segment_indices(offsets: torch.Tensor, nnz: Optional[int] = None) -> torch.Tensor:
    return native().gen_segment_indices(offsets, int(nnz if nnz is not None else offsets[-1].item()))


def _sides(t, n, device):
    if t is None:
        return torch.zeros(n, dtype=torch.bool)
    if t.dtype != torch.bool:
        raise ValueError(f"side tensors must be of type torch.bool, but got {t.dtype}.")
    return t


def fused_ragged_cutoff_2D(values: List[torch.Tensor], offsets: List[torch.Tensor], keep_lengths: torch.Tensor,
                           drop_sides: torch.Tensor = None, pad_sides: torch.Tensor = None):
    """Truncate the rows of several 2-D ragged tensors at once.

    ``keep_lengths[t]`` values are kept per row of tensor ``t``; ``drop_sides[t]`` True drops from the left (start).
    Returns ``(values, offsets, drop_nums, pad_nums, drop_sides, pad_sides)``; no pad values are written (``pad_nums``
    tells a dense consumer how many it would need)."""
    if len(offsets) != len(values):
        raise ValueError(f"Length of 'offsets' list ({len(offsets)}) must match length of 'values' list ({len(values)}).")
    drop_sides = _sides(drop_sides, len(values), values[0].device)
    pad_sides = _sides(pad_sides, len(values), values[0].device)
    v, o, d, p = native().fused_ragged_cutoff_2d(list(values), list(offsets), keep_lengths, drop_sides, pad_sides)
    return v, o, d, p, drop_sides, pad_sides


def fused_ragged_cutoff_3D(values: List[torch.Tensor], offsets: List[List[torch.Tensor]], keep_lengths: torch.Tensor,
                           drop_sides: Optional[torch.Tensor] = None, pad_sides: Optional[torch.Tensor] = None):
    """Give every sample of several 3-D ragged tensors exactly ``keep_lengths[t]`` inner rows (drop rows / pad empty rows).
    ``offsets[t] = [outer, inner]``. Returns ``(values, [[outer, inner], ...])``."""
    drop_sides = _sides(drop_sides, len(values), values[0].device)
    pad_sides = _sides(pad_sides, len(values), values[0].device)
    v, outer, inner = native().fused_ragged_cutoff_3d(list(values), [o[0] for o in offsets], [o[1] for o in offsets], keep_lengths,
                                                      drop_sides, pad_sides)
    return v, [[a, b] for a, b in zip(outer, inner)]


def feature_cross_ragged(x_val, x_offsets, y_val, y_offsets, x_weight=None, y_weight=None):
    """Per row: unique(x) x unique(y) -> ``(ids = murmur(x, y), offsets, weights = wx * wy)``."""
    return native().feature_cross_ragged(x_val, x_offsets, y_val, y_offsets, x_weight, y_weight)


def ragged_topk_index_cutoff(drop_num, pad_num, drop_side, pad_side, offset, topk_index, indicator):
    """Map top-k positions inside truncated/padded rows back to indices of the original values.
    All four drop/pad side combinations are handled (the reference implements drop-left/pad-right only)."""
    dl = bool(drop_side.reshape(-1)[0].item()) if isinstance(drop_side, torch.Tensor) else bool(drop_side)
    pl = bool(pad_side.reshape(-1)[0].item()) if isinstance(pad_side, torch.Tensor) else bool(pad_side)
    return native().calc_ragged_index(drop_num, pad_num, dl, pl, offset, topk_index, indicator)


def ragged_tile(batch: List[int], seq: List[int], indices: torch.Tensor, offset: torch.Tensor, table: torch.Tensor,
                check_enable: bool = False):
    """Tile combiner on an explicit table: for every feature ``f`` and row, the first ``seq[f]`` rows of ``table`` addressed by
    ``indices`` (zero padded) -> ``[sum_f batch[f] * seq[f], dim]``. Differentiable with respect to ``table``."""
    check_para(batch, seq, indices, offset, table, check_enable)
    outs = []
    row0 = 0
    off = offset.to(torch.int32)
    for b, s in zip(batch, seq):
        o = (off[row0:row0 + b + 1] - off[row0]).contiguous()
        idx = indices[int(off[row0]):int(off[row0 + b])].to(torch.int32).contiguous()
        outs.append(_TileFn.apply(table, idx, o, int(s)).view(b * s, table.shape[1]))
        row0 += b
    return torch.cat(outs) if len(outs) > 1 else outs[0]


def check_para(batch: List[int], seq: List[int], indices: torch.Tensor, offset: torch.Tensor, table: torch.Tensor,
               check_enable: bool = True):
    """Argument validation of ``ragged_tile`` (``recis/nn/functional/ragged_ops.py:694-715``); a no-op unless ``check_enable``."""
    if not check_enable:
        return
    assert len(batch) == len(seq) and len(batch) > 0, "batch and seq must be non-empty lists of equal length"
    assert all(int(b) > 0 for b in batch) and all(int(s) > 0 for s in seq), "batch sizes and tile lengths must be positive"
    assert offset.dim() == 1 and offset.numel() == sum(int(b) for b in batch) + 1, "offset must hold sum(batch) + 1 boundaries"
    assert indices.dim() == 1 and table.dim() == 2, "indices must be 1-D and table 2-D"
    assert int(offset[-1]) <= indices.numel(), "offsets point past the end of indices"
    if indices.numel():
        assert int(indices.min()) >= 0 and int(indices.max()) < table.shape[0], "indices out of range of the table"


class _TileFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, idx, offsets, tile_len):
        out, gsrc, gscale = native().tile_forward(table.contiguous(), None, idx, offsets, None, tile_len, True)
        ctx.save_for_backward(idx, gsrc)
        ctx.shape = table.shape
        return out

    @staticmethod
    def backward(ctx, dy):
        idx, gsrc = ctx.saved_tensors
        D = ctx.shape[1]
        g = torch.zeros(ctx.shape, dtype=dy.dtype, device=dy.device)
        keep = gsrc >= 0
        g.index_add_(0, idx[keep].long(), dy.reshape(-1, D)[gsrc[keep].long()])
        return g, None, None, None
