"""Move nested batches (dict / list / tuple of tensors and RaggedTensors) between devices
(``recis/utils/data_utils.py``)."""
from __future__ import annotations

import torch

from ..ragged.tensor import RaggedTensor


def copy_data_to_device(data, device="cuda", non_blocking: bool = True):
    if isinstance(data, (torch.Tensor, RaggedTensor)):
        return data.to(device, non_blocking=non_blocking)
    if isinstance(data, dict):
        return {k: copy_data_to_device(v, device, non_blocking) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return type(data)(copy_data_to_device(v, device, non_blocking) for v in data)
    return data


def pin_data(data):
    if isinstance(data, (torch.Tensor, RaggedTensor)):
        return data.pin_memory()
    if isinstance(data, dict):
        return {k: pin_data(v) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return type(data)(pin_data(v) for v in data)
    return data
