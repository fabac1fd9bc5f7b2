"""Streaming AUROC from a fixed-threshold confusion matrix (``recis/metrics/auroc.py:6-383``): ``num_thresholds`` evenly
spaced thresholds, cumulative TP/FP/TN/FN, trapezoid over the ROC points; ``dist_sync_on_step`` all-reduces the counts.
One ``bucketize`` + ``bincount`` per update instead of a [thresholds, batch] comparison matrix."""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn


class AUROC(nn.Module):
    def __init__(self, num_thresholds: int = 200, dist_sync_on_step: bool = False):
        super().__init__()
        assert num_thresholds >= 2
        self.num_thresholds = num_thresholds
        self.dist_sync_on_step = dist_sync_on_step
        eps = 1e-7
        th = torch.linspace(0.0, 1.0, num_thresholds)
        th[0], th[-1] = -eps, 1.0 + eps
        self.register_buffer("thresholds", th)
        self.register_buffer("pos_hist", torch.zeros(num_thresholds + 1, dtype=torch.int64))
        self.register_buffer("neg_hist", torch.zeros(num_thresholds + 1, dtype=torch.int64))

    def update(self, predictions: torch.Tensor, labels: torch.Tensor):
        p = predictions.detach().reshape(-1).float()
        y = labels.detach().reshape(-1) > 0.5
        dev = p.device
        if self.thresholds.device != dev:
            self.to(dev)
        # bucket b holds predictions with thresholds[b-1] < p <= thresholds[b]  ("p > t" counts everything above bucket t)
        b = torch.bucketize(p, self.thresholds, right=False)
        n = self.num_thresholds + 1
        self.pos_hist += torch.bincount(b[y], minlength=n)
        self.neg_hist += torch.bincount(b[~y], minlength=n)

    def _counts(self):
        pos, neg = self.pos_hist.clone(), self.neg_hist.clone()
        if self.dist_sync_on_step and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            both = torch.stack([pos, neg])
            dist.all_reduce(both, op=dist.ReduceOp.SUM)
            pos, neg = both[0], both[1]
        # tp[t] = positives with p > thresholds[t] = sum of buckets t+1..
        tp = pos.flip(0).cumsum(0).flip(0)[1:].double()
        fp = neg.flip(0).cumsum(0).flip(0)[1:].double()
        return tp, fp, pos.sum().double() - tp, neg.sum().double() - fp

    def sync(self, tp, fp, tn, fn):
        """Sum confusion-matrix components over all ranks (no-op without a process group); the API of the reference's
        ``AUROC.sync`` (``recis/metrics/auroc.py:281-316``)."""
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            both = torch.stack([tp, fp, tn, fn])
            dist.all_reduce(both, op=dist.ReduceOp.SUM)
            tp, fp, tn, fn = both[0], both[1], both[2], both[3]
        return tp, fp, tn, fn

    def compute(self) -> torch.Tensor:
        tp, fp, fn, tn = self._counts()
        eps = 1e-6
        tpr = (tp + eps) / (tp + fn + eps)
        fpr = fp / (fp + tn + eps)
        return ((fpr[:-1] - fpr[1:]) * (tpr[:-1] + tpr[1:]) / 2.0).sum().float()

    def forward(self, predictions, labels):
        self.update(predictions, labels)
        return self.compute()

    def reset(self):
        self.pos_hist.zero_()
        self.neg_hist.zero_()
