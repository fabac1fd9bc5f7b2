"""DLRM-style CTR model: bottom MLP on dense features, one merged dynamic table for all sparse fields
(sum pooling), pairwise dot interaction, top MLP in bf16, BCE-with-logits loss."""
from __future__ import annotations

from typing import List, Sequence

import torch
from torch import nn

from ..nn import EmbeddingEngine, EmbeddingOption
from ..nn.initializers import NormalInitializer
from ..ops.dense import MLP, dot_interaction


class DLRM(nn.Module):
    def __init__(self, sparse_fields: Sequence[str], dense_dim: int = 13, emb_dim: int = 128,
                 bottom: Sequence[int] = (512, 256, 128), top: Sequence[int] = (1024, 1024, 512, 256, 1),
                 device=None, capacity: int = 0, init_std: float = 0.01, compute_dtype=torch.bfloat16, combiner: str = "sum"):
        super().__init__()
        assert bottom[-1] == emb_dim, "bottom MLP must end at the embedding width for the dot interaction"
        self.fields = list(sparse_fields)
        self.emb_dim = emb_dim
        opts = {
            f: EmbeddingOption(embedding_dim=emb_dim, shared_name=f, combiner=combiner, use_weight=False, device=device,
                               initializer=NormalInitializer(0.0, init_std), capacity=capacity // max(len(self.fields), 1))
            for f in self.fields
        }
        self.embedding_engine = EmbeddingEngine(opts, interleave=True)
        n_vec = len(self.fields) + 1
        self.n_pairs = n_vec * (n_vec - 1) // 2
        self.bottom = MLP([dense_dim] + list(bottom), final_act=True, dtype=compute_dtype)
        self.top = MLP([emb_dim + self.n_pairs] + list(top), final_act=False, dtype=compute_dtype)
        self.compute_dtype = compute_dtype
        self.loss_fn = nn.BCEWithLogitsLoss()

    def forward(self, batch: dict):
        dense = batch["dense"]
        label = batch["label"]
        self.embedding_engine({f: batch[f] for f in self.fields})
        (cube, names), = self.embedding_engine.packed.values()      # [B, F, D] fp32, no stacking copy
        assert names == self.fields
        x = self.bottom(dense)                                        # [B, D] compute dtype
        z = dot_interaction(x, cube)                                  # [B, D + pairs] compute dtype
        logit = self.top(z)[:, :1].float()
        return self.loss_fn(logit, label), logit
