"""Dense-tower building blocks.

On CUDA every Linear runs on the hand-written tcgen05 GEMM (``csrc/kernels/gemm_tcgen05.cu``): bf16 operands, fp32
accumulation in tensor memory, bias + ReLU fused in the epilogue; the backward pass uses the same kernel with MN-major
operands (no transposed copies) plus one fused ReLU-mask + bias-gradient kernel. The feature interactions (pairwise dot,
FM second order) are single kernels per direction. On CPU (or for dtypes the kernels do not take) plain PyTorch is used,
which is also the oracle in the tests. The reference's dense layers are ``nn.Linear`` under bf16 autocast
(``examples/seq2seq/seq2seq_model.py:90``, ``examples/deepfm/deepfm_model.py:49-52``).
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.nn.functional as F
from torch import nn

from .. import native


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def bf16_shadow(weight: torch.Tensor):
    """The bf16 copy of ``weight`` that the last forward pass made (or the dense optimizer rewrote), if it still matches the
    weight: same storage and no in-place change through torch since. Native optimizer steps rewrite weight and copy in one
    kernel and leave the version counter alone, so the copy stays valid across steps; anything else that touches the weight
    (another optimizer, ``load_state_dict``, ``copy_``) bumps the counter and the next forward pass casts again."""
    rec = getattr(weight, "_rb_bf16", None)
    if rec is not None and rec[1] == weight._version and rec[2] == weight.data_ptr() and rec[0].device == weight.device:
        return rec[0]
    return None


def keep_bf16_shadow(weight: torch.Tensor, wb: torch.Tensor):
    """Remember ``wb`` (the weight cast to bf16, zero-padded to multiples of 8 in both dimensions) as the copy of ``weight``; the
    dense optimizer's kernel rewrites it in that layout together with the weight."""
    weight._rb_bf16 = (wb, weight._version, weight.data_ptr())


class _LinearFn(torch.autograd.Function):
    """y[M, Np] = act(x[M, Kp] W^T + b) with W given as fp32 [N, K] (padded + cast to bf16 here)."""

    @staticmethod
    def forward(ctx, x, weight, bias, relu):
        C = native()
        N, K = weight.shape
        Np, Kp = _pad8(N), _pad8(K)
        assert x.shape[1] == Kp and x.dtype == torch.bfloat16
        wb = bf16_shadow(weight)
        if wb is None:
            wb = C.cast_pad_bf16(weight, Np, Kp)
            keep_bf16_shadow(weight, wb)
        bp = bias if Np == N else F.pad(bias, (0, Np - N))
        y = C.gemm_bf16(x, wb, bp, relu, False, False, False, None)
        ctx.save_for_backward(x, wb, y)
        ctx.relu, ctx.shape = relu, (N, K)
        return y

    @staticmethod
    def backward(ctx, dout):
        C = native()
        x, wb, y = ctx.saved_tensors
        N, K = ctx.shape
        dy, db = C.relu_bwd_bias(y, dout.contiguous(), ctx.relu)
        dx = None
        if ctx.needs_input_grad[0]:
            # dx[M, Kp] = dy[M, Np] . W[Np, Kp]   (B operand read MN-major: no transposed copy of W)
            dx = C.gemm_bf16(dy, wb, None, False, False, True, False, None)
        # dW[Np, Kp] = dy^T . x                  (both operands MN-major, reduction over the batch)
        dw = C.gemm_bf16(dy, x, None, False, True, True, True, None)
        return dx, dw[:N, :K], db[:N], None


class _LinearResidualFn(torch.autograd.Function):
    """out (fp32) = residual + x W^T + b with the addition in the GEMM's epilogue (no separate cast and add kernels)."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        C = native()
        N, K = weight.shape
        assert N % 8 == 0 and x.shape[1] == _pad8(K) and x.dtype == torch.bfloat16
        wb = bf16_shadow(weight)
        if wb is None:
            wb = C.cast_pad_bf16(weight, N, _pad8(K))
            keep_bf16_shadow(weight, wb)
        ctx.save_for_backward(x, wb)
        ctx.shape = (N, K)
        return C.gemm_bf16_residual(x, wb, bias, residual.contiguous())

    @staticmethod
    def backward(ctx, dout):
        C = native()
        x, wb = ctx.saved_tensors
        N, K = ctx.shape
        dob = dout.to(torch.bfloat16).contiguous()
        dy, db = C.relu_bwd_bias(dob, dob, False)
        dx = C.gemm_bf16(dy, wb, None, False, False, True, False, None) if ctx.needs_input_grad[0] else None
        dw = C.gemm_bf16(dy, x, None, False, True, True, True, None)
        return dx, dw[:N, :K], db[:N], dout


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, out_bf16):
        y, stats = native().layer_norm_fwd(x, gamma, beta, eps, out_bf16)
        ctx.save_for_backward(x, stats, gamma)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, stats, gamma = ctx.saved_tensors
        dx, dgamma, dbeta = native().layer_norm_bwd(dy.contiguous(), x, stats, gamma)
        return dx, dgamma, dbeta, None, None


class LayerNorm(nn.LayerNorm):
    """``nn.LayerNorm`` over the last dimension of ``[rows, hidden]``. On CUDA (fp32 input, hidden a multiple of 4 up to 1024)
    the forward is one kernel that can write bf16 directly (``out_bf16``: the output then feeds a GEMM without a separate
    cast) and the backward is one pass that produces the input gradient and both weight gradients
    (``csrc/kernels/norm_ops.cu``). Elsewhere it is the library's layer norm."""

    def forward(self, x, out_bf16: bool = False):
        H = x.shape[-1]
        if (x.is_cuda and x.dim() == 2 and x.dtype == torch.float32 and H % 4 == 0 and H <= 1024 and self.elementwise_affine
                and self.bias is not None):
            return _LayerNormFn.apply(x.contiguous(), self.weight, self.bias, self.eps, out_bf16)
        y = super().forward(x)
        return y.to(torch.bfloat16) if out_bf16 and x.is_cuda else y


class Linear(nn.Module):
    """``y = act(x W^T + b)``; fp32 master weights, bf16 compute on CUDA. Output width is padded to a multiple of 8
    (``out_pad``) so that it can feed the next layer's TMA loads directly; ``forward`` slices the padding off when asked."""

    def __init__(self, in_features, out_features, act: bool = False, dtype=torch.bfloat16):
        super().__init__()
        self.in_features, self.out_features, self.act, self.dtype = in_features, out_features, act, dtype
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features))
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    def forward(self, x, keep_pad: bool = False):
        if x.is_cuda and self.dtype == torch.bfloat16:
            Kp = _pad8(self.in_features)
            if x.dtype != torch.bfloat16:
                x = x.to(torch.bfloat16)
            if x.shape[1] != Kp:
                x = F.pad(x, (0, Kp - x.shape[1]))
            y = _LinearFn.apply(x.contiguous(), self.weight, self.bias, self.act)
            return y if keep_pad or y.shape[1] == self.out_features else y[:, :self.out_features]
        y = F.linear(x.float()[:, :self.in_features], self.weight, self.bias)
        return F.relu(y) if self.act else y

    def forward_residual(self, x, residual):
        """``residual + x W^T + b`` in fp32 (no activation): on CUDA the sum is formed in the GEMM's epilogue."""
        assert not self.act
        if (x.is_cuda and self.dtype == torch.bfloat16 and self.out_features % 8 == 0 and residual.dtype == torch.float32
                and x.shape[1] == _pad8(self.in_features)):
            return _LinearResidualFn.apply(x.to(torch.bfloat16).contiguous(), self.weight, self.bias, residual)
        return residual + self.forward(x).float()


class _MLPFn(torch.autograd.Function):
    """All layers of an MLP in two native calls (forward, backward) instead of several per layer: the dense tower of a
    recommendation model is many small GEMMs, and the host-side cost of issuing them one by one is comparable to their GPU time."""

    @staticmethod
    def forward(ctx, x, relu, *params):
        n = len(params) // 2
        weights, biases = list(params[:n]), list(params[n:])
        xp, ys, wbs = native().mlp_forward(x, weights, biases, list(relu), [bf16_shadow(w) for w in weights])
        for w, wb in zip(weights, wbs):
            keep_bf16_shadow(w, wb)
        ctx.relu, ctx.shapes, ctx.n = list(relu), [list(w.shape) for w in weights], n
        ctx.x_shape, ctx.x_dtype = x.shape, x.dtype
        ctx.save_for_backward(xp, *ys, *wbs)
        return ys[-1]

    @staticmethod
    def backward(ctx, dout):
        saved = ctx.saved_tensors
        n = ctx.n
        xp, ys, wbs = saved[0], list(saved[1:1 + n]), list(saved[1 + n:1 + 2 * n])
        dx, dws, dbs = native().mlp_backward(dout.to(torch.bfloat16), xp, ys, wbs, ctx.relu, ctx.shapes, ctx.needs_input_grad[0])
        if dx is not None and ctx.needs_input_grad[0]:
            dx = dx[:, :ctx.x_shape[1]].to(ctx.x_dtype)
        else:
            dx = None
        return (dx, None, *dws, *dbs)


class MLP(nn.Module):
    def __init__(self, dims: Sequence[int], final_act: bool = False, dtype=torch.bfloat16):
        super().__init__()
        self.dtype = dtype
        self.layers = nn.ModuleList(
            [Linear(dims[i], dims[i + 1], act=(i < len(dims) - 2) or final_act, dtype=dtype) for i in range(len(dims) - 1)])

    def forward(self, x):
        n = len(self.layers)
        if x.is_cuda and self.dtype == torch.bfloat16:
            relu = tuple(bool(l.act) for l in self.layers)
            y = _MLPFn.apply(x, relu, *[l.weight for l in self.layers], *[l.bias for l in self.layers])
            out = self.layers[-1].out_features
            return y if y.shape[1] == out else y[:, :out]
        for i, layer in enumerate(self.layers):
            x = layer(x, keep_pad=i < n - 1)
        return x


class _DotInteractionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cube):
        C = native()
        B, Fn, D = cube.shape
        out = C.dot_interaction_fwd(x, cube, _pad8(D + (Fn + 1) * Fn // 2))
        ctx.save_for_backward(x, cube)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, cube = ctx.saved_tensors
        dx, dcube = native().dot_interaction_bwd(x, cube, dout.contiguous())
        return dx.to(x.dtype), dcube


def dot_interaction(x: torch.Tensor, cube: torch.Tensor) -> torch.Tensor:
    """``x`` [B, D] + embeddings ``cube`` [B, F, D] -> [B, D + (F+1)F/2 (+ zero pad to a multiple of 8 on CUDA)]:
    ``x`` followed by the strict lower triangle (row-major) of ``Z Z^T`` with ``Z = [x; cube]``."""
    B, Fn, D = cube.shape
    if x.is_cuda and x.dtype == torch.bfloat16 and cube.dtype == torch.float32:
        return _DotInteractionFn.apply(x.contiguous(), cube.contiguous())
    z = torch.cat([x.unsqueeze(1), cube.to(x.dtype)], dim=1)
    zz = torch.bmm(z, z.transpose(1, 2))
    li, lj = torch.tril_indices(Fn + 1, Fn + 1, offset=-1, device=x.device)
    return torch.cat([x, zz[:, li, lj]], dim=1)


class _FMFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, cube):
        ctx.save_for_backward(cube)
        return native().fm_fwd(cube)

    @staticmethod
    def backward(ctx, gout):
        (cube,) = ctx.saved_tensors
        return native().fm_bwd(cube, gout)


def fm_interaction(cube: torch.Tensor) -> torch.Tensor:
    """Second-order FM term ``0.5 * sum_d ((sum_f v)^2 - sum_f v^2)`` -> [B, 1]."""
    if cube.is_cuda and cube.dtype == torch.float32:
        return _FMFn.apply(cube.contiguous())
    s = cube.sum(dim=1)
    return 0.5 * (s * s - (cube * cube).sum(dim=1)).sum(dim=1, keepdim=True)
