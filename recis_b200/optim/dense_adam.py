"""Dense Adam / AdamW with PyTorch semantics on the native multi-tensor kernel.

Same update rule as ``torch.optim.Adam`` / ``torch.optim.AdamW`` (bias-corrected second moment inside the square root's
denominator, epsilon added after it; Adam's ``weight_decay`` is an L2 term added to the gradient, AdamW's is decoupled), so
it can replace them one for one for the dense tower. On CUDA a step is one kernel launch per 24 tensors
(``csrc/kernels/dense_ops.cu``); on CPU it falls back to multi-tensor (foreach) calls. The reference leaves the dense
optimizer to ``torch.optim`` (``examples/deepfm/runner.py``) or to its own TF-style ``AdamWTF``
(``recis/optim/adamw_tf.py:21-426``).
"""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer


def _shadows(params):
    """Per parameter, the bf16 copy that the forward pass keeps of it (``ops.dense.bf16_shadow``) or None; the update kernel
    writes the rounded new weights into these copies, so the next forward pass needs no cast. An empty list when there is none."""
    from ..ops.dense import bf16_shadow
    out = [bf16_shadow(p) for p in params]
    return out if any(o is not None for o in out) else []


class DenseAdam(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, decoupled=False):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("invalid hyper-parameter")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decoupled=decoupled))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            buckets = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["step"] += 1
                buckets.setdefault(st["step"], []).append(p)
            for t, ps in buckets.items():
                gs = [p.grad for p in ps]
                ms = [self.state[p]["exp_avg"] for p in ps]
                vs = [self.state[p]["exp_avg_sq"] for p in ps]
                bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
                wd, lr = group["weight_decay"], group["lr"]
                decay = 1 - lr * wd if group["decoupled"] else 1.0
                l2 = 0.0 if group["decoupled"] else wd
                if all(p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and g.is_contiguous() for p, g in zip(ps, gs)):
                    from .. import native
                    native().dense_adam(ps, gs, ms, vs, _shadows(ps), b1, b2, group["eps"], decay, lr / bc1, 1.0 / math.sqrt(bc2), l2)
                    continue
                if l2:
                    gs = torch._foreach_add(gs, ps, alpha=l2)
                if decay != 1.0:
                    torch._foreach_mul_(ps, decay)
                torch._foreach_lerp_(ms, gs, 1 - b1)
                torch._foreach_mul_(vs, b2)
                torch._foreach_addcmul_(vs, gs, gs, 1 - b2)
                denom = torch._foreach_sqrt(vs)
                torch._foreach_div_(denom, math.sqrt(bc2))
                torch._foreach_add_(denom, group["eps"])
                torch._foreach_addcdiv_(ps, ms, denom, -lr / bc1)
        return loss


class DenseAdamW(DenseAdam):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, decoupled=True)
