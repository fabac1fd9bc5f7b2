"""Long-sequence behaviour model on synthetic ragged data (one process; see ``benchmarks/sequence_model.py`` for the timed,
multi-GPU version). Role of the reference's ``examples/seq2seq``: ragged sequences, embeddings, a transformer, bf16 on GPU.

    python examples/seq2seq/run.py [--device cpu|cuda] [--steps 20]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "benchmarks"))

import torch

from recis_b200.models import SequenceModel
from recis_b200.nn import filter_out_sparse_param
from recis_b200.optim import DenseAdam, SparseAdam


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--max-len", type=int, default=128)
    a = ap.parse_args()
    from sequence_model import make_batch
    from recis_b200.parallel.dense_reducer import DenseGradReducer
    from recis_b200.utils.launch import finish_distributed, init_distributed
    rank, world, dev = init_distributed(a.device)          # one process, or one per GPU / CPU rank under torch.distributed.run

    class Shape:
        batch, min_len, max_len, items, cates = a.batch, 8, a.max_len, 1_000_000, 1000
    pf = [f"profile_{i}" for i in range(4)]
    torch.manual_seed(0)
    model = SequenceModel(pf, hidden=128, heads=4, layers=2, ffn=256, head_mlp=(128, 1), device=dev, max_len=a.max_len,
                          compute_dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32).to(dev)
    sparse_opt = SparseAdam(filter_out_sparse_param(model), lr=1e-3)
    dense_params = [p for p in model.parameters() if p.requires_grad]
    dense_opt = DenseAdam(dense_params, lr=1e-3)
    reducer = DenseGradReducer(dense_params, world) if world > 1 else None      # data-parallel dense tower: averaged gradients
    for step in range(a.steps):
        batch, tokens = make_batch(Shape, dev, step * world + rank, pf)           # every rank draws its own batches
        loss, _ = model(batch)
        dense_opt.zero_grad(set_to_none=reducer is None)
        sparse_opt.zero_grad()
        loss.backward()
        if reducer is not None:
            reducer.all_reduce_async()
        sparse_opt.step()
        if reducer is not None:
            reducer.wait()
        dense_opt.step()
        if rank == 0 and (step % 5 == 0 or step == a.steps - 1):
            print(f"step {step:4d}  tokens {tokens:6d}  loss {float(loss.detach()):.4f}")
    finish_distributed()


if __name__ == "__main__":
    main()
