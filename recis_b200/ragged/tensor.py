"""RaggedTensor: flat values + nested row offsets (outermost first) + optional per-value weight.

API of the reference's ``recis/ragged/tensor.py:41-541``. One deliberate difference: unknown dimensions of
``dense_shape`` are resolved lazily. The reference resolves them in the constructor with ``max().item()``,
which is a device-to-host synchronisation per ragged tensor per step; here nothing touches the host until a
caller actually asks for a maximum length.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch


class RaggedPadInfo:
    """How many entries a truncate/pad step removed or added on each side of every row."""

    def __init__(self, drop_nums: torch.Tensor, pad_nums: torch.Tensor, drop_sides: torch.Tensor, pad_sides: torch.Tensor):
        self.drop_nums = drop_nums
        self.pad_nums = pad_nums
        self.drop_sides = drop_sides
        self.pad_sides = pad_sides

    def __repr__(self):
        return (f"RaggedPadInfo(drop_nums={self.drop_nums}, pad_nums={self.pad_nums}, "
                f"drop_sides={self.drop_sides}, pad_sides={self.pad_sides})")


class RaggedTensor:
    def __init__(self, values: torch.Tensor, offsets, weight: Optional[torch.Tensor] = None,
                 dense_shape: Optional[tuple] = None):
        self._values = values
        if isinstance(offsets, torch.Tensor):
            offsets = [offsets]
        self._offsets: List[torch.Tensor] = list(offsets)
        self._weight = weight
        if dense_shape is None:
            dense_shape = (-1,) * (len(self._offsets) + 1)
        self._dense_shape = tuple(int(s) for s in dense_shape)
        self._pad_info = None

    # ------------------------------------------------------------------ shape
    def set_dim_by_rank(self, dim, rank):
        shape = list(self._dense_shape)
        shape[rank] = int(dim)
        self._dense_shape = tuple(shape)

    @property
    def dim(self):
        return len(self._dense_shape)

    @property
    def max_length(self):
        return self.get_shape(-1)

    @property
    def pad_info(self):
        return self._pad_info

    def set_pad_info(self, pad_info: RaggedPadInfo):
        self._pad_info = pad_info

    def get_shape(self, dim):
        if dim < 0:
            dim += len(self._dense_shape)
        if self._dense_shape[dim] != -1:
            return self._dense_shape[dim]
        if dim == 0:
            size = self._offsets[0].numel() - 1
        elif self._offsets[dim - 1].numel() < 2:
            size = 0
        else:
            off = self._offsets[dim - 1]
            size = int((off[1:] - off[:-1]).max().item())  # host read, only when a caller needs the number
        shape = list(self._dense_shape)
        shape[dim] = size
        self._dense_shape = tuple(shape)
        return size

    def real_shape(self, start=0, end=None):
        n = len(self._dense_shape)
        if end is None:
            end = n
        if end < 0:
            end += n
        return tuple(self.get_shape(i) for i in range(start, end))

    @property
    def shape(self):
        return self.real_shape()

    def size(self):
        return self.real_shape()

    # ------------------------------------------------------------------ accessors
    def values(self):
        return self._values

    def set_values(self, values: torch.Tensor):
        self._values = values

    def offsets(self):
        return self._offsets

    def weight(self):
        return self._weight

    def set_weight(self, weight: torch.Tensor):
        self._weight = weight

    @property
    def dtype(self):
        return self._values.dtype

    @property
    def device(self):
        return self._values.device

    # ------------------------------------------------------------------ conversions
    def to_dense(self, default_value: float = 0.0):
        from ..nn.functional.ragged_ops import ragged_to_dense
        return ragged_to_dense(self._values, self._offsets, default_value)

    def to_sparse(self):
        from ..nn.functional.ragged_ops import ragged_to_sparse
        return ragged_to_sparse(self._values, self._offsets)

    @staticmethod
    def from_dense(dense: torch.Tensor, check_invalid: bool = False, invalid_value=0):
        from ..nn.functional.ragged_ops import dense_to_ragged
        values, offsets = dense_to_ragged(dense, check_invalid, invalid_value)
        return RaggedTensor(values, offsets)

    @staticmethod
    def from_numpy(values: np.ndarray, offsets: List[np.ndarray]):
        return RaggedTensor(torch.from_numpy(values), [torch.from_numpy(np.ascontiguousarray(o)) for o in offsets])

    @staticmethod
    def concat(parts: List["RaggedTensor"]) -> "RaggedTensor":
        """Row-wise concatenation: the rows of ``parts[0]``, then those of ``parts[1]`` ... All parts have the same number of
        offset levels; weights are kept when every part has them. (A new helper: batches assembled from several readers, as the
        proportional window datasets do, need it.)"""
        if len(parts) == 1:
            return parts[0]
        levels = len(parts[0]._offsets)
        assert all(len(p._offsets) == levels for p in parts), "parts differ in ragged depth"
        values = torch.cat([p._values for p in parts])
        offsets = []
        for lv in range(levels):
            pieces, shift = [parts[0]._offsets[lv]], parts[0]._offsets[lv][-1]
            for p in parts[1:]:
                pieces.append(p._offsets[lv][1:] + shift)
                shift = shift + p._offsets[lv][-1]
            offsets.append(torch.cat(pieces))
        weight = torch.cat([p._weight for p in parts]) if all(p._weight is not None for p in parts) else None
        shape = list(parts[0]._dense_shape)
        shape[0] = sum(int(p._offsets[0].numel()) - 1 for p in parts)
        for d in range(1, len(shape)):
            dims = [p._dense_shape[d] for p in parts]
            shape[d] = -1 if any(x == -1 for x in dims) else max(dims)
        return RaggedTensor(values, offsets, weight=weight, dense_shape=tuple(shape))

    def pin_memory(self):
        return RaggedTensor(self._values.pin_memory(), [o.pin_memory() for o in self._offsets],
                            self._weight.pin_memory() if self._weight is not None else None,
                            dense_shape=self._dense_shape)

    def to(self, *args, **kwargs):
        """Move to a device (offsets keep their integer dtype; a dtype argument converts values only)."""
        device = kwargs.get("device")
        dtype = kwargs.get("dtype")
        non_blocking = kwargs.get("non_blocking", False)
        for a in args:
            if isinstance(a, torch.dtype):
                dtype = a
            elif isinstance(a, (str, torch.device)):
                device = a
        values = self._values
        if device is not None:
            values = values.to(device, non_blocking=non_blocking)
        if dtype is not None:
            values = values.to(dtype)
        offsets = [o.to(device, non_blocking=non_blocking) if device is not None else o for o in self._offsets]
        weight = self._weight
        if weight is not None and device is not None:
            weight = weight.to(device, non_blocking=non_blocking)
        out = RaggedTensor(values, offsets, weight, dense_shape=self._dense_shape)
        out._pad_info = self._pad_info
        return out

    def cuda(self):
        return self.to("cuda")

    def clone(self):
        out = RaggedTensor(self._values.clone(), [o.clone() for o in self._offsets],
                           self._weight.clone() if self._weight is not None else None, dense_shape=self._dense_shape)
        out._pad_info = self._pad_info
        return out

    def __str__(self) -> str:
        return (f"RaggedTensor(values={self._values}, offsets={self._offsets}, weight={self._weight}, "
                f"dense_shape={self._dense_shape})")

    __repr__ = __str__
