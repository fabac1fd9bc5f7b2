"""Sparse (row-wise) optimizers over dynamic embedding tables.

API of the reference's ``recis/optim/sparse_optim.py:6-174`` and ``sparse_adam*.py`` (``step``, ``zero_grad``,
``state_dict``, ``load_state_dict``, ``set_grad_accum_steps``, ``add_params``; a dummy param group so that torch
LR schedulers drive ``lr``). The update math follows ``csrc/ops/block_apply_adamw_op_kernel.cu:11-22,109-120``:

    beta1^t *= beta1 ; beta2^t *= beta2 ; alpha = -lr * sqrt(1 - beta2^t) / (1 - beta1^t)
    w *= decay ; m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 ; w += alpha * m / (sqrt(v) + eps)

with ``decay`` = 1 (Adam), ``1 - lr*wd`` (AdamW) or ``1 - wd`` (AdamW-TF); only rows that received a gradient
are touched. ``SparseAdagrad`` is an addition (the reference has none):
``acc += g^2 ; w = w*decay - lr * g / (sqrt(acc) + eps)``.

Where the reference materialises a sparse COO gradient (cat -> unique -> index_add) and then launches the
update, a step here is one kernel when the table holds a single staged backward record: duplicates are reduced
from the pooled output gradient and the row is updated in the same pass.
"""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from .. import native
from ..nn.modules.hashtable import split_sparse_dense_state_dict

OPT_ADAM, OPT_ADAGRAD, OPT_SGD = 0, 1, 2


def _row_disjoint(recs) -> bool:
    """True when the staged exchange records are known to touch pairwise different rows: each one names the child tables its
    ids belong to, and no child appears twice. A row that showed up in two records must get ONE update of the summed gradient
    (the materialising path), not two updates."""
    seen = set()
    for r in recs:
        ch = r.get("children")
        if ch is None or (seen & ch):
            return False
        seen |= ch
    return True


class SparseOptimizer(Optimizer):
    slot_prefix = "sparse_opt"
    slot_names = ()
    slot_fill = 0.0

    def __init__(self, param_dict: dict, lr=0.01) -> None:
        self._tables = {}
        self._local_step = 0
        self._grad_accum_steps = 1
        self._step_count = 0
        super().__init__([{"initial_lr": lr, "lr": lr, "params": []}], defaults={})
        self.add_params(param_dict)

    # ---- parameters
    @staticmethod
    def filter_param_dict(param_dict):
        out, seen = {}, []
        for k, v in param_dict.items():
            if any(v is s for s in seen):
                continue
            out[k] = v
            seen.append(v)
        return out

    def add_params(self, params: dict):
        for name, table in self.filter_param_dict(params).items():
            impl = getattr(table, "impl", table)
            self._tables[name] = impl
            for slot in self.slot_names:
                impl.store.add_slot(f"{self.slot_prefix}_{slot}", self.slot_fill)

    def tables(self):
        return self._tables

    # ---- hyper-parameters of one step; subclasses fill in
    def _kernel_args(self, lr: float):
        raise NotImplementedError

    def _slots(self, impl):
        names = [f"{self.slot_prefix}_{s}" for s in self.slot_names]
        s1 = impl.store.slot(names[0]) if len(names) > 0 else None
        s2 = impl.store.slot(names[1]) if len(names) > 1 else None
        return s1, s2

    def _advance(self):
        self._step_count += 1

    def step(self, closure=None):
        assert self._grad_accum_steps > 0
        self._local_step += 1
        if self._local_step % self._grad_accum_steps != 0:
            return
        lr = float(self.param_groups[0]["lr"])
        self._advance()
        kind, b1, b2, eps, decay, alpha = self._kernel_args(lr)
        C = native()
        inv_accum = 1.0 / self._grad_accum_steps
        for impl in self._tables.values():
            recs = impl.records()
            if not recs:
                continue
            s1, s2 = self._slots(impl)
            w = impl.store.emb()
            if len(recs) == 1 and recs[0]["kind"] == "fused":
                r = recs[0]
                csr_u, csr_elem, start = C.build_csr(r["rev"])
                C.grad_reduce(r["grad_out"], r["gsrc"], r["gscale"], csr_u, csr_elem, start, impl.dim, r["rows"], True, kind, lr,
                              b1, b2, eps, decay, alpha, r.get("scale", 1.0) * inv_accum, w, s1, s2, 0)
            elif len(recs) == 1 and recs[0]["kind"] == "peer":
                r = recs[0]
                r["exchange"].owner_reduce(impl, r, True, kind, lr, b1, b2, eps, decay, alpha, inv_accum, w, s1, s2)
            elif all(r.get("kind") == "peer" for r in recs) and _row_disjoint(recs):
                # one record per exchange lane and the lanes share no table row (different child tables): each lane's update is
                # its own kernel, issued in the order the gradients were pushed, so the first ones run while the last lanes are
                # still exchanging
                for r in recs:
                    r["exchange"].owner_reduce(impl, r, True, kind, lr, b1, b2, eps, decay, alpha, inv_accum, w, s1, s2)
            else:
                rows, grads = impl.materialize()
                if rows is not None and rows.numel():
                    C.sparse_apply(rows, grads, None, kind, lr, b1, b2, eps, decay, alpha, inv_accum, w, s1, s2)

    def zero_grad(self, set_to_none: bool = True):
        assert self._grad_accum_steps > 0
        if self._local_step % self._grad_accum_steps == 0:
            for impl in self._tables.values():
                impl.clear_grad()

    def set_grad_accum_steps(self, steps: int):
        self._grad_accum_steps = int(steps)
        for impl in self._tables.values():
            # with accumulation the owner must consume each micro-batch's gradient window before the next one overwrites it
            ex = getattr(impl, "exchange", None)
            if ex is not None:
                ex.immediate_reduce = steps > 1

    # ---- state
    def _scalar_state(self) -> dict:
        return {f"{self.slot_prefix}_step": torch.tensor(float(self._step_count))}

    def state_dict(self) -> dict:
        ret = dict(self._tables)
        ret.update(self._scalar_state())
        return ret

    def load_state_dict(self, state_dict: dict):
        _tables, scalars = split_sparse_dense_state_dict(dict(state_dict))
        key = f"{self.slot_prefix}_step"
        if key in scalars:
            self._step_count = int(round(float(scalars[key])))


class _AdamBase(SparseOptimizer):
    slot_names = ("exp_avg", "exp_avg_sq")

    def __init__(self, param_dict, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-2, amsgrad=False):
        if amsgrad:
            raise ValueError("amsgrad is not support now")
        self._beta1, self._beta2, self._eps, self._weight_decay = beta1, beta2, eps, weight_decay
        super().__init__(param_dict, lr=lr)

    def _decay(self, lr):
        return 1.0

    def _kernel_args(self, lr):
        t = self._step_count
        b1p, b2p = self._beta1 ** t, self._beta2 ** t
        alpha = -lr * math.sqrt(1.0 - b2p) / (1.0 - b1p)
        return OPT_ADAM, self._beta1, self._beta2, self._eps, self._decay(lr), alpha

    def _scalar_state(self):
        t = self._step_count
        return {
            f"{self.slot_prefix}_step": torch.tensor(float(t)),
            f"{self.slot_prefix}_beta1": torch.tensor(self._beta1 ** t),
            f"{self.slot_prefix}_beta2": torch.tensor(self._beta2 ** t),
        }


class SparseAdam(_AdamBase):
    """Adam on touched rows; no decoupled decay (factor 1), as ``csrc/embedding/adam.cc:65-73``."""
    slot_prefix = "sparse_adam"


class SparseAdamW(_AdamBase):
    """AdamW on touched rows: ``w *= 1 - lr*wd`` before the Adam step (``csrc/embedding/adamw.cc:53-74``)."""
    slot_prefix = "sparse_adamw"

    def _decay(self, lr):
        return 1.0 - lr * self._weight_decay


class SparseAdamWTF(_AdamBase):
    """TensorFlow-style AdamW: ``w *= 1 - wd`` (``csrc/embedding/adamw_tf.cc:64``)."""
    slot_prefix = "sparse_adamw_tf"

    def _decay(self, lr):
        return 1.0 - self._weight_decay


class SparseAdagrad(SparseOptimizer):
    """Row-wise Adagrad with an element-wise accumulator slot (an addition to the reference's optimizer set)."""
    slot_prefix = "sparse_adagrad"
    slot_names = ("accum",)

    def __init__(self, param_dict, lr=1e-2, eps=1e-10, weight_decay=0.0, initial_accumulator_value=0.0):
        self._eps, self._weight_decay = eps, weight_decay
        self.slot_fill = float(initial_accumulator_value)      # per instance: two optimizers may start their accumulators differently
        super().__init__(param_dict, lr=lr)

    def _kernel_args(self, lr):
        return OPT_ADAGRAD, 0.0, 0.0, self._eps, 1.0 - lr * self._weight_decay, 0.0


class SparseSGD(SparseOptimizer):
    slot_prefix = "sparse_sgd"

    def __init__(self, param_dict, lr=1e-2, weight_decay=0.0):
        self._weight_decay = weight_decay
        super().__init__(param_dict, lr=lr)

    def _kernel_args(self, lr):
        return OPT_SGD, 0.0, 0.0, 0.0, 1.0 - lr * self._weight_decay, 0.0
