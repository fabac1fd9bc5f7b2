"""Embedding-path functional ops (``recis/nn/functional/embedding_ops.py``): id partitioning, id encoding, offset merging
and ragged pooling with autograd. "Sparse mode" (mean = sum(w e) / sum(w)) and "ragged mode" (mean = sum(w e) / length) are
the same kernel with a different normalisation flag."""
from __future__ import annotations

from typing import List, Optional, Union

import torch

from ... import native

_COMBINER = {"sum": 0, "mean": 1}


def ids_partition(ids: torch.Tensor, max_partition_num: int, world_size: int):
    """Dedup ids and bucket the unique ids by owner rank.
    Returns ``(unique ids ordered by owner, per-owner counts (int64), reverse index (int32))``; the owner of an id is the
    rank whose contiguous slice range contains ``id & 0xFFFF``. ``max_partition_num`` is accepted and not used, as in the
    reference (``recis/nn/functional/embedding_ops.py:486-512``): routing always uses the 65536 slices of the low 16 id bits."""
    uniq, rev, counts, offs = native().dedup_partition(ids.reshape(-1).contiguous(), int(world_size))
    n = int(offs[-1].item())
    return uniq[:n], counts.to(torch.int64), rev


def ids_encode(ids_list: List[torch.Tensor], table_ids: Union[torch.Tensor, list]) -> torch.Tensor:
    """Concatenate id tensors with ``(id & (2^52 - 1)) | (table_id << 52)``."""
    tids = table_ids.tolist() if isinstance(table_ids, torch.Tensor) else list(table_ids)
    dev = ids_list[0].device
    ids = [t.reshape(-1).to(torch.int64).contiguous() for t in ids_list]
    prefix = [0]
    for t in ids:
        prefix.append(prefix[-1] + t.numel())
    F = len(ids)
    desc = torch.tensor([[t.data_ptr() for t in ids] + [0], prefix, [0] * (F + 1), [0] * (F + 1)], dtype=torch.int64)
    tidx = torch.tensor([int(v) for v in tids], dtype=torch.int64)
    if dev.type == "cuda":
        desc, tidx = desc.pin_memory().to(dev, non_blocking=True), tidx.pin_memory().to(dev, non_blocking=True)
    out, _ = native().encode_merge(desc, tidx, F, prefix[-1], 0, False)
    return out


def merge_offsets(offsets: List[torch.Tensor]) -> torch.Tensor:
    """Concatenate row offsets of several ragged tensors into one offsets vector over their concatenated values."""
    outs, base = [], 0
    for i, o in enumerate(offsets):
        o = o.to(torch.int64)
        outs.append((o[:-1] if i < len(offsets) - 1 else o) + base)
        base = base + int(o[-1].item())
    return torch.cat(outs).to(offsets[0].dtype)


class _SegmentReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, emb, weight, indices, offsets, mode):
        C = native()
        out, gsrc, gscale = C.pool_forward(emb.contiguous(), None, indices, offsets, weight, mode, 0, 0, True)
        ctx.save_for_backward(indices, gsrc, gscale)
        ctx.n_rows, ctx.dim = emb.shape[0], emb.shape[1]
        return out

    @staticmethod
    def backward(ctx, grad):
        C = native()
        indices, gsrc, gscale = ctx.saved_tensors
        uniq, inv = torch.unique(indices, return_inverse=True)
        rev = inv.to(torch.int32).contiguous()
        csr_u, csr_elem, start = C.build_csr(rev)
        gu = C.grad_reduce(grad.contiguous().float(), gsrc, gscale, csr_u, csr_elem, start, ctx.dim, None, False, 2, 0.0, 0.0, 0.0,
                           0.0, 1.0, 0.0, 1.0, None, None, None, max(uniq.numel(), 1))
        g = torch.zeros(ctx.n_rows, ctx.dim, dtype=grad.dtype, device=grad.device)
        g[uniq.long()] = gu[:uniq.numel()].to(grad.dtype)
        return g, None, None, None, None


def ragged_embedding_segment_reduce(unique_emb: torch.Tensor, weight, reverse_indices: torch.Tensor, offsets: torch.Tensor,
                                    combiner: str = "sum", combiner_kwargs: Optional[dict] = None, mean_by_weight: bool = False):
    """``out[s] = reduce_{i in segment s} w_i * unique_emb[reverse_indices[i]]`` (sum | mean), differentiable with respect to
    ``unique_emb``. ``combiner="tile"`` takes ``combiner_kwargs={"bs": [rows per feature], "tile_len": [rows kept per feature]}`` and
    returns the first ``tile_len`` embeddings of every row, zero padded, ``[sum_f bs[f] * tile_len[f], dim]``
    (argument names and the tile form follow ``recis/nn/functional/embedding_ops.py:332-420``)."""
    assert combiner in ("sum", "mean", "tile"), f"combiner {combiner} is not supported"
    if combiner == "tile":
        from .ragged_ops import ragged_tile
        kw = combiner_kwargs or {}
        return ragged_tile(list(kw["bs"]), list(kw["tile_len"]), reverse_indices, offsets, unique_emb)
    mode = _COMBINER[combiner]
    if mode == 1 and mean_by_weight:
        mode = 2
    w = weight.float().contiguous() if weight is not None else None
    return _SegmentReduce.apply(unique_emb, w, reverse_indices.to(torch.int32).contiguous(), offsets.to(torch.int32).contiguous(), mode)


def sparse_embedding_segment_reduce(unique_emb: torch.Tensor, weight, reverse_indices: torch.Tensor, segment_ids: torch.Tensor,
                                    num_segments: int, combiner: str = "sum"):
    """Same reduction addressed by per-element segment ids (must be sorted); mean divides by the weight sum."""
    counts = torch.bincount(segment_ids.long(), minlength=num_segments)
    offsets = torch.zeros(num_segments + 1, dtype=torch.int32, device=unique_emb.device)
    offsets[1:] = torch.cumsum(counts, 0)
    return ragged_embedding_segment_reduce(unique_emb, weight, reverse_indices, offsets, combiner, mean_by_weight=True)


def segment_sum_sparse(data, weight, indices, segment_ids, num_segments, backend="recis"):
    return sparse_embedding_segment_reduce(data, weight, indices, segment_ids, num_segments, "sum")


def weight_norm_sparse(data, weight, segment_ids, num_segments, backend="recis"):
    """``data / sum of the segment's weights`` per segment."""
    ws = torch.zeros(num_segments, dtype=torch.float32, device=data.device).index_add_(0, segment_ids.long(), weight.float())
    return data / ws.clamp(min=1e-30).unsqueeze(1)
