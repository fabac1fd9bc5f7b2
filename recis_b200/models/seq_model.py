"""Long-sequence user-behaviour model (DIN / seq2seq style) on ragged batches.

Inputs per sample: a behaviour sequence of (item id, category id) pairs of any length, a target (item, category) pair and a
set of single-hot profile fields. Model: item/category embeddings from dynamic tables -> token projection -> target attention
over the sequence -> a small transformer encoder over the sequence -> MLP head, BCE-with-logits loss.

Layout decisions:
* Sequences stay PACKED (``[total_tokens, hidden]``) everywhere except inside the attention core: the per-token embedding
  lookup feeds the id values as a flat batch of one-id bags, so the exchange moves unique ids only and nothing is padded;
  all projections and the FFN run on the packed tokens through the tensor-core GEMM (``ops.dense.Linear``).
* Target attention (one query per sequence) is ``ops.attention.target_attention`` on the packed layout: one kernel per
  direction on CUDA, segment reductions with tensor ops elsewhere.
* The encoder's attention core is ``ops.attention.ragged_self_attention``: on CUDA the ragged tensor-core kernels (no padding,
  forward and backward); elsewhere it scatters the packed Q/K/V into ``[batch, max_len, heads, head_dim]`` and calls
  ``F.scaled_dot_product_attention`` with a key-padding mask (the reference's sequence example does that on fully padded
  tensors under bf16 autocast, ``examples/seq2seq/transformer.py:36-38`` and ``seq2seq_model.py:87-91``).
"""
from __future__ import annotations

from typing import Sequence

import torch
from torch import nn

from ..nn import EmbeddingEngine, EmbeddingOption
from ..nn.functional.ragged_ops import gen_segment_indices
from ..nn.initializers import NormalInitializer
from ..ops.attention import ragged_self_attention, target_attention
from ..ops.dense import MLP, LayerNorm, Linear
from ..ragged import RaggedTensor


def segment_softmax(scores: torch.Tensor, seg: torch.Tensor, n_seg: int) -> torch.Tensor:
    """Softmax of ``scores[t]`` within each segment ``seg[t]`` (packed layout, fp32)."""
    m = torch.full((n_seg,), -float("inf"), dtype=scores.dtype, device=scores.device).scatter_reduce(0, seg, scores, "amax")
    e = torch.exp(scores - m[seg])
    z = torch.zeros(n_seg, dtype=scores.dtype, device=scores.device).index_add_(0, seg, e)
    return e / z[seg].clamp_min(1e-30)


class EncoderLayer(nn.Module):
    """Pre-norm transformer layer on packed tokens; attention core on a padded view."""

    def __init__(self, hidden: int, heads: int, ffn: int, dtype):
        super().__init__()
        self.hidden, self.heads = hidden, heads
        self.norm1, self.norm2 = LayerNorm(hidden), LayerNorm(hidden)
        self.qkv = Linear(hidden, 3 * hidden, dtype=dtype)
        self.proj = Linear(hidden, hidden, dtype=dtype)
        self.ffn = MLP([hidden, ffn, hidden], final_act=False, dtype=dtype)

    def forward(self, x, seg, pos, lengths, max_len, offsets=None):
        # on CUDA the activations between the kernels stay bf16 and the two additions onto the fp32 residual stream happen in
        # the epilogues of the projection GEMMs
        h = self.norm1(x, out_bf16=x.is_cuda)
        qkv = self.qkv(h)                                                      # [T, 3 * hidden] packed
        qkv = qkv.to(torch.bfloat16) if x.is_cuda else qkv.float()
        if offsets is None:
            offsets = torch.cat([lengths.new_zeros(1), lengths.cumsum(0)])
        o = ragged_self_attention(qkv, offsets, self.heads, max_len, seg, pos)
        x = self.proj.forward_residual(o, x)
        f = self.ffn.layers[0](self.norm2(x, out_bf16=x.is_cuda))
        return self.ffn.layers[1].forward_residual(f, x)


class SequenceModel(nn.Module):
    def __init__(self, profile_fields: Sequence[str], emb_dim: int = 64, profile_dim: int = 32, hidden: int = 256, heads: int = 4,
                 layers: int = 2, ffn: int = 1024, head_mlp: Sequence[int] = (512, 256, 1), device=None, item_capacity: int = 0,
                 cate_capacity: int = 0, profile_capacity: int = 0, compute_dtype=torch.bfloat16, max_len: int = 1000):
        super().__init__()
        self.profile_fields = list(profile_fields)
        self.hidden, self.max_len = hidden, max_len
        init = NormalInitializer(0.0, 0.01)
        opts = {
            # the sequence and the target of one entity share rows through the shared_name
            "seq_item": EmbeddingOption(embedding_dim=emb_dim, shared_name="item", combiner="sum", use_weight=False, device=device,
                                        initializer=init, capacity=item_capacity),
            "tgt_item": EmbeddingOption(embedding_dim=emb_dim, shared_name="item", combiner="sum", use_weight=False, device=device,
                                        initializer=init),
            "seq_cate": EmbeddingOption(embedding_dim=emb_dim, shared_name="cate", combiner="sum", use_weight=False, device=device,
                                        initializer=init, capacity=cate_capacity),
            "tgt_cate": EmbeddingOption(embedding_dim=emb_dim, shared_name="cate", combiner="sum", use_weight=False, device=device,
                                        initializer=init),
        }
        for f in self.profile_fields:
            opts[f] = EmbeddingOption(embedding_dim=profile_dim, shared_name=f, combiner="sum", use_weight=False, device=device,
                                      initializer=init, capacity=profile_capacity // max(len(self.profile_fields), 1))
        self.embedding_engine = EmbeddingEngine(opts)
        self.token_proj = Linear(2 * emb_dim, hidden, dtype=compute_dtype)
        self.query_proj = Linear(2 * emb_dim, hidden, dtype=compute_dtype)
        self.layers = nn.ModuleList([EncoderLayer(hidden, heads, ffn, compute_dtype) for _ in range(layers)])
        self.final_norm = LayerNorm(hidden)
        self.head = MLP([3 * hidden + len(self.profile_fields) * profile_dim] + list(head_mlp), final_act=False, dtype=compute_dtype)
        self.loss_fn = nn.BCEWithLogitsLoss()

    def forward(self, batch: dict):
        seq_item: RaggedTensor = batch["seq_item"]
        seq_cate: RaggedTensor = batch["seq_cate"]
        offsets = seq_item.offsets()[-1]
        B = offsets.numel() - 1
        T = seq_item.values().numel()
        feats = {"seq_item": seq_item.values(), "seq_cate": seq_cate.values(), "tgt_item": batch["tgt_item"], "tgt_cate": batch["tgt_cate"]}
        for f in self.profile_fields:
            feats[f] = batch[f]
        emb = self.embedding_engine(feats)
        dev = emb["seq_item"].device
        offsets = offsets.to(dev)
        tok = torch.cat([emb["seq_item"], emb["seq_cate"]], dim=1)             # [T, 2 D] packed
        tgt = torch.cat([emb["tgt_item"].view(B, -1), emb["tgt_cate"].view(B, -1)], dim=1)
        x = self.token_proj(tok).float()                                        # [T, hidden]
        q = self.query_proj(tgt).float()                                        # [B, hidden]
        seg = gen_segment_indices(offsets, T).long()
        lengths = (offsets[1:] - offsets[:-1]).long()
        pos = torch.arange(T, device=dev) - offsets[:-1].long()[seg]
        max_len = min(self.max_len, int(batch.get("max_len", self.max_len)))
        # ---- target attention: one query per sequence, softmax over its tokens
        interest = target_attention(x, q, offsets, seg, self.hidden ** -0.5)
        # ---- encoder over the sequence
        h = x
        for layer in self.layers:
            h = layer(h, seg, pos, lengths, max_len, offsets)
        h = self.final_norm(h)
        pooled = torch.zeros(B, self.hidden, dtype=h.dtype, device=dev).index_add_(0, seg, h) / lengths.clamp_min(1)[:, None]
        profile = torch.cat([emb[f].view(B, -1) for f in self.profile_fields], dim=1) if self.profile_fields else h.new_zeros(B, 0)
        z = torch.cat([interest, pooled, q, profile], dim=1)
        logit = self.head(z)[:, :1].float()
        return self.loss_fn(logit, batch["label"]), logit
