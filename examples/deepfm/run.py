"""DeepFM on synthetic Criteo-shaped data with the Trainer (CPU or GPU; one process, or one process per GPU / CPU rank).

Default shape: batch 1024, 13 dense features (lognormal through log1p), 26 single-hot categorical fields with ids ~ Zipf(1.1)
over [0, 1e6) in one merged dynamic table of width 16 (init N(0, 0.01)), FM second-order term + MLP 400-400-400-1, labels
Bernoulli(0.25), sparse Adagrad lr 0.01 + Adam lr 1e-3, 100 steps, seed 0.

    python examples/deepfm/run.py [--device cpu|cuda] [--steps 100] [--output-dir /tmp/deepfm_ckpt]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29600 examples/deepfm/run.py   (one rank per GPU, or CPU ranks with --device cpu)

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
from recis_b200.utils.launch import finish_distributed, init_distributed


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--batch", type=int, default=1024)
    ap.add_argument("--output-dir", default=None)
    args = ap.parse_args()
    # one process, or one process per GPU / CPU rank under torch.distributed.run: tables are then sharded over the ranks and every
    # rank draws its own batches
    rank, world, dev = init_distributed(args.device)
    args.device = str(dev)
    torch.manual_seed(0)
    fields = [f"C{i + 1}" for i in range(26)]
    spec = SyntheticSpec(batch=args.batch, dense_dim=13, label_rate=0.25, seed=rank,
                         sparse=[SparseFieldSpec(f, zipf_a=1.1, id_bits=20, universe=1_000_000, length="fixed", mean_len=1) for f in fields])
    model = DeepFM(fields, dense_dim=13, emb_dim=16, hidden=(400, 400, 400), device=args.device,
                   compute_dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32).to(args.device)
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
    if world > 1:                                   # every rank writes its shard into the same directory: rank 0's choice
        box = [out_dir]
        torch.distributed.broadcast_object_list(box, src=0)
        out_dir = box[0]
    train_args = TrainingArguments(output_dir=out_dir, log_steps=20, train_steps=args.steps, save_steps=max(args.steps // 2, 1), max_to_keep=2)
    dataset = WrapEndDataset(StateDataset(SyntheticDataset(spec, steps=args.steps), save_interval=10))
    trainer = Trainer(model=WithMetrics(model), args=train_args, train_dataset=dataset,
                      dense_optimizers=(DenseAdam([p for p in model.parameters() if p.requires_grad], lr=1e-3), None),
                      sparse_optimizer=SparseAdagrad(filter_out_sparse_param(model), lr=0.01), data_to_cuda=dev.type == "cuda")
    t0 = time.perf_counter()
    trainer.train()
    dt = time.perf_counter() - t0
    rows = sum(t.impl.size() for t in model.embedding_engine.tables().values())
    if rank == 0:
        print(f"trained {args.steps} steps of batch {args.batch} x {world} rank(s) in {dt:.1f} s "
              f"({args.steps * args.batch * world / dt:.0f} samples/s), {rows} embedding rows on rank 0, checkpoints in {out_dir}")
    finish_distributed()


if __name__ == "__main__":
    main()
