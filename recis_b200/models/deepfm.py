"""DeepFM: first-order terms + FM second-order interaction + MLP over the concatenated field embeddings, on one merged dynamic
table (structure of the reference's ``examples/deepfm/deepfm_model.py:16-131``; the FM term is one fused kernel on CUDA)."""
from __future__ import annotations

from typing import Sequence

import torch
from torch import nn

from ..nn import EmbeddingEngine, EmbeddingOption
from ..nn.initializers import NormalInitializer
from ..ops.dense import MLP, fm_interaction


class DeepFM(nn.Module):
    def __init__(self, sparse_fields: Sequence[str], dense_dim: int = 13, emb_dim: int = 16, hidden: Sequence[int] = (400, 400, 400),
                 device=None, capacity: int = 0, init_std: float = 0.01, compute_dtype=torch.bfloat16):
        super().__init__()
        self.fields = list(sparse_fields)
        self.dense_dim, self.emb_dim = dense_dim, emb_dim
        init = NormalInitializer(0.0, init_std)
        opts = {}
        for f in self.fields:
            opts[f"{f}_emb"] = EmbeddingOption(embedding_dim=emb_dim, shared_name=f"{f}_emb", combiner="sum", use_weight=False,
                                               device=device, initializer=init, capacity=capacity // max(len(self.fields), 1))
            opts[f"{f}_bias"] = EmbeddingOption(embedding_dim=4, shared_name=f"{f}_bias", combiner="sum", use_weight=False,
                                                device=device, initializer=init, capacity=capacity // max(len(self.fields), 1))
        self.embedding_engine = EmbeddingEngine(opts, interleave=True)
        self.numeric_embs = nn.Parameter(torch.randn(dense_dim, emb_dim) * 0.001)
        self.numeric_bias = nn.Parameter(torch.randn(dense_dim) * 0.001)
        self.dnn = MLP([(dense_dim + len(self.fields)) * emb_dim] + list(hidden) + [1], final_act=False, dtype=compute_dtype)
        self.loss_fn = nn.BCEWithLogitsLoss()

    def forward(self, batch: dict):
        dense, label = batch["dense"], batch["label"]
        feats = {}
        for f in self.fields:
            feats[f"{f}_emb"] = batch[f]
            feats[f"{f}_bias"] = batch[f]
        out = self.embedding_engine(feats)
        B = dense.shape[0]
        emb = torch.stack([out[f"{f}_emb"] for f in self.fields], dim=1)                 # [B, F, D]
        bias = torch.stack([out[f"{f}_bias"][:, 0] for f in self.fields], dim=1)         # [B, F]
        num_emb = dense.unsqueeze(-1) * self.numeric_embs.unsqueeze(0)                   # [B, dense, D]
        cube = torch.cat([num_emb, emb], dim=1).contiguous()
        first = (dense * self.numeric_bias).sum(1, keepdim=True) + bias.sum(1, keepdim=True)
        second = fm_interaction(cube)
        deep = self.dnn(cube.view(B, -1))[:, :1].float()
        logit = first + second + deep
        return self.loss_fn(logit, label), logit
