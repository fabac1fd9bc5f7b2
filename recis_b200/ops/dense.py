"""Dense-tower building blocks: Linear/MLP with bf16 compute and the feature interactions."""
from __future__ import annotations

from typing import Sequence

import torch
from torch import nn
import torch.nn.functional as F


class Linear(nn.Module):
    """y = act(x W^T + b); fp32 master weights, bf16 compute on CUDA."""

    def __init__(self, in_features, out_features, act: bool = False, dtype=torch.bfloat16):
        super().__init__()
        self.in_features, self.out_features, self.act, self.dtype = in_features, out_features, act, dtype
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features))
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    def forward(self, x):
        if x.is_cuda and self.dtype != torch.float32:
            y = F.linear(x.to(self.dtype), self.weight.to(self.dtype), self.bias.to(self.dtype))
        else:
            y = F.linear(x.float(), self.weight, self.bias)
        return F.relu(y) if self.act else y


class MLP(nn.Module):
    def __init__(self, dims: Sequence[int], final_act: bool = False, dtype=torch.bfloat16):
        super().__init__()
        layers = []
        for i in range(len(dims) - 1):
            layers.append(Linear(dims[i], dims[i + 1], act=(i < len(dims) - 2) or final_act, dtype=dtype))
        self.layers = nn.ModuleList(layers)

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x


def dot_interaction(x: torch.Tensor, cube: torch.Tensor) -> torch.Tensor:
    """[B, D] dense vector + [B, F, D] embeddings -> [B, D + (F+1)F/2]: x and the strict lower triangle of Z Z^T."""
    B, Fn, D = cube.shape
    z = torch.cat([x.unsqueeze(1), cube.to(x.dtype)], dim=1)
    zz = torch.bmm(z, z.transpose(1, 2))
    li, lj = torch.tril_indices(Fn + 1, Fn + 1, offset=-1, device=x.device)
    return torch.cat([x, zz[:, li, lj]], dim=1)


def fm_interaction(cube: torch.Tensor) -> torch.Tensor:
    """Second-order FM term: 0.5 * sum_d ((sum_f v)^2 - sum_f v^2) -> [B, 1]."""
    s = cube.sum(dim=1)
    return 0.5 * (s * s - (cube * cube).sum(dim=1)).sum(dim=1, keepdim=True)
