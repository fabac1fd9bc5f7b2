"""DeepFM on synthetic Criteo-shaped data with the Trainer (runs on CPU or one GPU, one process).

Default shape: batch 1024, 13 dense features (lognormal through log1p), 26 single-hot categorical fields with ids ~ Zipf(1.1)
over [0, 1e6) in one merged dynamic table of width 16 (init N(0, 0.01)), FM second-order term + MLP 400-400-400-1, labels
Bernoulli(0.25), sparse Adagrad lr 0.01 + Adam lr 1e-3, 100 steps, seed 0.

    python examples/deepfm/run.py [--device cpu|cuda] [--steps 100] [--output-dir /tmp/deepfm_ckpt]

Same structure as the reference's example (``examples/deepfm/runner.py``, ``deepfm_model.py``): Trainer + sparse/dense
optimizers + logger hook + periodic sparse checkpoints.
"""
import argparse
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from recis_b200.framework import Trainer, TrainingArguments
from recis_b200.framework.metrics import add_metric
from recis_b200.io import SparseFieldSpec, StateDataset, SyntheticDataset, SyntheticSpec, WrapEndDataset
from recis_b200.metrics.auroc import AUROC
from recis_b200.models import DeepFM
from recis_b200.nn import filter_out_sparse_param
from recis_b200.optim import DenseAdam, SparseAdagrad


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--batch", type=int, default=1024)
    ap.add_argument("--output-dir", default=None)
    args = ap.parse_args()
    torch.manual_seed(0)
    fields = [f"C{i + 1}" for i in range(26)]
    spec = SyntheticSpec(batch=args.batch, dense_dim=13, label_rate=0.25, seed=0,
                         sparse=[SparseFieldSpec(f, zipf_a=1.1, id_bits=20, universe=1_000_000, length="fixed", mean_len=1) for f in fields])
    model = DeepFM(fields, dense_dim=13, emb_dim=16, hidden=(400, 400, 400), device=args.device,
                   compute_dtype=torch.bfloat16 if args.device == "cuda" else torch.float32).to(args.device)
    auc = AUROC(num_thresholds=200)

    class WithMetrics(torch.nn.Module):
        def __init__(self, inner):
            super().__init__()
            self.inner = inner

        def forward(self, batch):
            loss, logit = self.inner(batch)
            auc.update(torch.sigmoid(logit.detach()).flatten().cpu(), batch["label"].flatten().cpu())
            add_metric("auc", auc.compute())
            return loss

    out_dir = args.output_dir or tempfile.mkdtemp(prefix="deepfm_")
    train_args = TrainingArguments(output_dir=out_dir, log_steps=20, train_steps=args.steps, save_steps=max(args.steps // 2, 1), max_to_keep=2)
    dataset = WrapEndDataset(StateDataset(SyntheticDataset(spec, steps=args.steps), save_interval=10))
    trainer = Trainer(model=WithMetrics(model), args=train_args, train_dataset=dataset,
                      dense_optimizers=(DenseAdam([p for p in model.parameters() if p.requires_grad], lr=1e-3), None),
                      sparse_optimizer=SparseAdagrad(filter_out_sparse_param(model), lr=0.01), data_to_cuda=args.device == "cuda")
    t0 = time.perf_counter()
    trainer.train()
    dt = time.perf_counter() - t0
    rows = sum(t.impl.size() for t in model.embedding_engine.tables().values())
    print(f"trained {args.steps} steps of batch {args.batch} in {dt:.1f} s ({args.steps * args.batch / dt:.0f} samples/s), "
          f"{rows} embedding rows, checkpoints in {out_dir}")


if __name__ == "__main__":
    main()
