"""Dense TensorFlow-style AdamW.

``param *= 1 - wd``; ``m, v`` moments; ``alpha = lr * sqrt(1 - b2^t) / (1 - b1^t)``;
``param -= alpha * m / (sqrt(v) + eps)`` (epsilon outside the bias correction), as the reference's
``recis/optim/adamw_tf.py:371-426`` and ``csrc/ops/adam_tf_op_kernel.cu:5-37``. ``fuse=True`` updates all
parameters of a group together: on CUDA with ONE launch of the native multi-tensor kernel per 24 tensors
(``csrc/kernels/dense_ops.cu``: weights, gradient and both moments are read once and written once), on CPU with
multi-tensor (foreach) calls.
"""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from .dense_adam import _shadows


class AdamWTF(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, use_nesterov: bool = False, *,
                 maximize: bool = False, fuse: bool = True, amsgrad: bool = False):
        if amsgrad:
            raise ValueError("amsgrad is not supported")
        if use_nesterov:
            # the reference accepts the flag and then asserts it is off (recis/optim/adamw_tf.py:344,389)
            raise ValueError("use_nesterov is not supported")
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("invalid hyper-parameter")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, maximize=maximize, fuse=fuse))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            params, grads, ms, vs = [], [], [], []
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("AdamWTF does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["step"] += 1
                params.append(p)
                grads.append(-p.grad if group["maximize"] else p.grad)
                ms.append(st["exp_avg"])
                vs.append(st["exp_avg_sq"])
            if not params:
                continue
            step = self.state[params[0]]["step"]
            alpha = group["lr"] * math.sqrt(1 - beta2 ** step) / (1 - beta1 ** step)
            same_step = all(self.state[p]["step"] == step for p in params)
            if group["fuse"] and same_step and all(p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and
                                                   g.is_contiguous() for p, g in zip(params, grads)):
                from .. import native
                native().dense_adam(params, grads, ms, vs, _shadows(params), beta1, beta2, group["eps"], 1 - group["weight_decay"], alpha, 1.0, 0.0)
            elif group["fuse"] and same_step:
                torch._foreach_mul_(params, 1 - group["weight_decay"])
                torch._foreach_lerp_(ms, grads, 1 - beta1)
                torch._foreach_mul_(vs, beta2)
                torch._foreach_addcmul_(vs, grads, grads, 1 - beta2)
                denom = torch._foreach_sqrt(vs)
                torch._foreach_add_(denom, group["eps"])
                torch._foreach_addcdiv_(params, ms, denom, -alpha)
            else:
                for p, g, m, v in zip(params, grads, ms, vs):
                    t = self.state[p]["step"]
                    a = group["lr"] * math.sqrt(1 - beta2 ** t) / (1 - beta1 ** t)
                    p.mul_(1 - group["weight_decay"])
                    m.lerp_(g, 1 - beta1)
                    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
                    p.addcdiv_(m, v.sqrt().add_(group["eps"]), value=-a)
        return loss
