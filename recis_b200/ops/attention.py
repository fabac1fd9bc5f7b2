"""Self-attention over ragged (packed) sequences.

``ragged_self_attention(qkv, offsets, heads, max_len)`` takes the packed projection output ``[total_tokens, 3 * hidden]``
(q | k | v) of a batch of sequences stored back to back and returns ``[total_tokens, hidden]``.

Two implementations:
* the tensor-core kernels (``csrc/kernels/attention_tcgen05.cu``): no padding, one CTA per (sequence, head, 128-row tile),
  forward and backward, head width 64: what CUDA training uses;
* the padded path: scatter into ``[batch, max_len, heads, head_dim]``, ``F.scaled_dot_product_attention`` with a key-padding
  mask, gather the valid positions back. Differentiable; other head widths, CPU tensors, ``RECIS_ATTENTION=padded``.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from .. import native


def _use_kernels() -> bool:
    """The tensor-core kernels serve CUDA inputs with head width 64 unless ``RECIS_ATTENTION=padded`` asks for the padded
    library path (kept as the fallback for other head widths, CPU tensors, and as a comparison arm)."""
    return os.environ.get("RECIS_ATTENTION", "tcgen05") != "padded"


def _padded(qkv, seg, pos, lengths, max_len, heads):
    T, width = qkv.shape
    hidden = width // 3
    hd = hidden // heads
    B = lengths.numel()
    padded = qkv.new_zeros(B, max_len, width)
    padded[seg, pos] = qkv
    q, k, v = padded.view(B, max_len, 3, heads, hd).permute(2, 0, 3, 1, 4)                # each [B, H, L, hd]
    key_ok = torch.arange(max_len, device=qkv.device)[None, :] < lengths[:, None]
    o = F.scaled_dot_product_attention(q, k, v, attn_mask=key_ok[:, None, None, :])       # [B, H, L, hd]
    return o.permute(0, 2, 1, 3).reshape(B, max_len, hidden)[seg, pos]


class _RaggedAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, offsets, heads, max_len, scale):
        out, lse = native().ragged_attention_fwd(qkv, offsets, heads, max_len, scale)
        ctx.save_for_backward(qkv, out, lse, offsets)
        ctx.args = (heads, max_len, scale)
        return out

    @staticmethod
    def backward(ctx, d_out):
        qkv, out, lse, offsets = ctx.saved_tensors
        heads, max_len, scale = ctx.args
        dqkv = native().ragged_attention_bwd(qkv, out, d_out.to(torch.bfloat16).contiguous(), lse, offsets, heads, max_len, scale)
        return dqkv.to(qkv.dtype), None, None, None, None


def ragged_self_attention(qkv: torch.Tensor, offsets: torch.Tensor, heads: int, max_len: int, seg: torch.Tensor = None,
                          pos: torch.Tensor = None) -> torch.Tensor:
    """``qkv``: ``[T, 3 * hidden]``; ``offsets``: ``[B + 1]`` sequence boundaries; returns ``[T, hidden]`` in ``qkv``'s dtype.
    ``seg`` / ``pos`` (sequence index and position of every token) are derived from ``offsets`` when not given."""
    hidden = qkv.shape[1] // 3
    hd = hidden // heads
    if _use_kernels() and qkv.is_cuda and hd == 64:
        out = _RaggedAttnFn.apply(qkv.to(torch.bfloat16).contiguous(), offsets.to(torch.int32).contiguous(), heads, int(max_len),
                                  float(hd) ** -0.5)
        return out.to(qkv.dtype)
    lengths = (offsets[1:] - offsets[:-1]).long()
    if seg is None:
        seg = torch.repeat_interleave(torch.arange(lengths.numel(), device=qkv.device), lengths)
    if pos is None:
        pos = torch.arange(qkv.shape[0], device=qkv.device) - offsets[:-1].long()[seg]
    return _padded(qkv, seg, pos, lengths, int(max_len), heads)


class _TargetAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, q, offsets, scale):
        interest, lse = native().target_attention_fwd(x, q, offsets, scale)
        ctx.save_for_backward(x, q, offsets, interest, lse)
        ctx.scale = scale
        return interest

    @staticmethod
    def backward(ctx, d_interest):
        x, q, offsets, interest, lse = ctx.saved_tensors
        dx, dq = native().target_attention_bwd(x, q, offsets, interest, lse, d_interest.contiguous().float(), ctx.scale)
        return dx, dq, None, None


def target_attention(x: torch.Tensor, q: torch.Tensor, offsets: torch.Tensor, seg: torch.Tensor = None, scale: float = None) -> torch.Tensor:
    """One query per sequence over packed tokens: ``interest[b] = sum_t softmax_t(scale * <x_t, q_b>) x_t`` for the tokens ``t``
    of sequence ``b``. ``x``: ``[T, hidden]``, ``q``: ``[B, hidden]``, ``offsets``: ``[B + 1]``. On CUDA (fp32, hidden a multiple
    of 4 up to 1024) the forward and the backward are one kernel each (``csrc/kernels/seq_ops.cu``); otherwise, and as the
    oracle in the tests, segment reductions with tensor ops."""
    hidden = x.shape[1]
    scale = float(hidden) ** -0.5 if scale is None else float(scale)
    if x.is_cuda and hidden % 4 == 0 and hidden <= 1024 and os.environ.get("RECIS_TARGET_ATTENTION", "kernel") != "eager":
        return _TargetAttnFn.apply(x.float().contiguous(), q.float().contiguous(), offsets.to(torch.int32).contiguous(), scale)
    B = q.shape[0]
    if seg is None:
        lengths = (offsets[1:] - offsets[:-1]).long()
        seg = torch.repeat_interleave(torch.arange(B, device=x.device), lengths)
    scores = (x * q[seg]).sum(-1) * scale
    m = torch.full((B,), -float("inf"), dtype=scores.dtype, device=x.device).scatter_reduce(0, seg, scores, "amax")
    e = torch.exp(scores - m[seg])
    z = torch.zeros(B, dtype=scores.dtype, device=x.device).index_add_(0, seg, e)
    att = e / z[seg].clamp_min(1e-30)
    return torch.zeros(B, hidden, dtype=x.dtype, device=x.device).index_add_(0, seg, x * att[:, None])
