"""Grouped AUC (``recis/metrics/gauc.py:7-215``): mean of per-group AUCs weighted by group size; groups are maximal runs of
equal ``indicators``. The per-batch computation is native C++ on the host; running sums are all-reduced on demand."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import native


class Gauc(torch.nn.Module):
    def __init__(self, dist_sync: bool = True) -> None:
        super().__init__()
        self.dist_sync = dist_sync
        self.reset()

    def reset(self):
        self._auc_sum = 0.0
        self._count_sum = 0.0

    def forward(self, labels, predictions, indicators):
        """Returns ``(gauc of this batch, running gauc)``."""
        aucs, counts = native().gauc_calc(labels.detach(), predictions.detach(), indicators.detach())
        batch_auc = float((aucs * counts).sum())
        batch_cnt = float(counts.sum())
        self._auc_sum += batch_auc
        self._count_sum += batch_cnt
        total = torch.tensor([batch_auc, batch_cnt, self._auc_sum, self._count_sum], dtype=torch.float64)
        if self.dist_sync and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dev = labels.device if dist.get_backend() == "nccl" else torch.device("cpu")
            total = total.to(dev)
            dist.all_reduce(total, op=dist.ReduceOp.SUM)
            total = total.cpu()
        return (float(total[0] / total[1]) if total[1] > 0 else 0.0, float(total[2] / total[3]) if total[3] > 0 else 0.0)
