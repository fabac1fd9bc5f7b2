"""CTR model over ORC files: columnar reader -> feature engine -> embedding engine -> MLP, driven by the Trainer.

    python examples/deepctr/make_orc_data.py --out /tmp/deepctr_data
    python examples/deepctr/run.py --data /tmp/deepctr_data [--device cpu|cuda] [--windows 4] [--trace-dir /tmp/deepctr_trace]

``--windows N`` reads the directory as one row-numbered table and trains through it in N windows (``make_odps_window_io``; the
trainer moves from window to window and checkpoints the position); ``--trace-dir`` appends every sample's label and logit to
Parquet parts there (``hooks.TraceToOdpsHook``).

Feature pipeline (the reference's ``examples/deepctr/dataset.py`` builds the same kind of chains):
  dense2  -> Bucketize(boundaries)                      -> shares the table of ``sparse1`` (same ``shared_name``)
  sparse1 -> Mod(1e6)        sparse2 -> Mod(1e5)
  city    -> Hash("farm") -> Mod(1000)                   (string column read as bytes)
  seq     -> Mod(1e5) -> SequenceTruncate(20, right)     -> ``tile`` combiner (first 20 positions, zero padded)
"""
import argparse
import glob
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
from torch import nn

from recis_b200.features import Bucketize, Feature, FeatureEngine, Hash, Mod, SelectField, SequenceTruncate
from recis_b200.framework import Trainer, TrainingArguments
from recis_b200.hooks import TraceToOdpsHook, add_to_trace
from recis_b200.io import OrcDataset, StateDataset, WrapEndDataset, make_odps_window_io
from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
from recis_b200.nn.initializers import TruncNormalInitializer
from recis_b200.ops.dense import MLP
from recis_b200.optim import DenseAdamW, SparseAdamW
from recis_b200.utils.launch import finish_distributed, init_distributed

SEQ_LEN = 20


class DeepCTR(nn.Module):
    def __init__(self, device, trace=False):
        super().__init__()
        self.trace = trace
        boundaries = [0.25 * i for i in range(1, 40)]
        self.feature_engine = FeatureEngine([
            Feature("dense2").add_op(SelectField("dense2", dtype=torch.float32)).add_op(Bucketize(boundaries)),
            Feature("sparse1").add_op(SelectField("sparse1")).add_op(Mod(1_000_000)),
            Feature("sparse2").add_op(SelectField("sparse2")).add_op(Mod(100_000)),
            Feature("city").add_op(SelectField("city")).add_op(Hash("farm")).add_op(Mod(1000)),
            Feature("seq").add_op(SelectField("seq")).add_op(Mod(100_000)).add_op(SequenceTruncate(seq_len=SEQ_LEN, truncate=True,
                                                                                               truncate_side="right", check_length=False)),
        ])
        init = TruncNormalInitializer(0.0, 0.02)
        opt = lambda name, dim, **kw: EmbeddingOption(embedding_dim=dim, shared_name=name, initializer=init, device=device, use_weight=False, **kw)
        self.embedding_engine = EmbeddingEngine({
            "dense2": opt("sparse1", 16), "sparse1": opt("sparse1", 16), "sparse2": opt("sparse2", 16), "city": opt("city", 16),
            "seq": opt("seq", 16, combiner="tile", combiner_kwargs={"tile_len": SEQ_LEN}),
        })
        self.mlp = MLP([1 + 4 * 16 + SEQ_LEN * 16, 128, 64, 1], final_act=False,
                       dtype=torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32)
        self.loss_fn = nn.BCEWithLogitsLoss()

    def forward(self, batch):
        data = self.feature_engine(batch)
        emb = self.embedding_engine({k: data[k] for k in ("dense2", "sparse1", "sparse2", "city", "seq")})
        B = batch["label"].shape[0]
        x = torch.cat([batch["dense1"].reshape(B, 1).to(emb["city"].device)] + [emb[k].reshape(B, -1) for k in ("dense2", "sparse1", "sparse2", "city", "seq")], dim=1)
        logit = self.mlp(x)[:, :1].float()
        if self.trace:                                       # per-sample columns of this step's rows in the trace table
            add_to_trace("label", batch["label"].reshape(B))
            add_to_trace("logit", logit.detach().reshape(B))
        return self.loss_fn(logit, batch["label"].reshape(B, 1).to(logit.device))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default="/tmp/deepctr_data")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--output-dir", default=None)
    ap.add_argument("--windows", type=int, default=0)
    ap.add_argument("--trace-dir", default=None)
    args = ap.parse_args()
    rank, world, dev = init_distributed(args.device)      # one process, or one per GPU / CPU rank under torch.distributed.run
    args.device = str(dev)
    torch.manual_seed(0)
    if args.windows:
        ds = make_odps_window_io(split_num=args.windows)(batch_size=args.batch, worker_idx=rank, worker_num=world, read_threads_num=2)
        ds.add_path(args.data)                                # the directory's files as one row-numbered table
    else:
        ds = OrcDataset(batch_size=args.batch, worker_idx=rank, worker_num=world, read_threads_num=2, prefetch=2)   # files dealt to ranks
        ds.add_paths(sorted(glob.glob(os.path.join(args.data, "*.orc"))))
    for name in ("sparse1", "sparse2", "seq"):
        ds.varlen_feature(name)
    ds.varlen_feature("city", trans_int8=True)                # keep the bytes: the feature engine hashes them
    for name in ("label", "dense1", "dense2"):
        ds.fixedlen_feature(name)
    model = DeepCTR(args.device, trace=bool(args.trace_dir)).to(args.device)
    out_dir = args.output_dir or tempfile.mkdtemp(prefix="deepctr_")
    if world > 1:
        box = [out_dir]
        torch.distributed.broadcast_object_list(box, src=0)
        out_dir = box[0]
    trainer = Trainer(model=model, args=TrainingArguments(output_dir=out_dir, log_steps=8, train_epoch=1, save_steps=1000),
                      train_dataset=ds if args.windows else WrapEndDataset(StateDataset(ds, save_interval=4)),
                      dense_optimizers=(DenseAdamW([p for p in model.parameters() if p.requires_grad], lr=1e-3), None),
                      sparse_optimizer=SparseAdamW(filter_out_sparse_param(model), lr=1e-3), data_to_cuda=dev.type == "cuda")
    if args.trace_dir:
        trainer.add_hook(TraceToOdpsHook({"output_dir": args.trace_dir, "partition": f"rank={rank}"}, ["label", "logit"], ["double", "double"]))
    trainer.train()
    if rank == 0:
        print({n: t.impl.size() for n, t in model.embedding_engine.tables().items()})
    finish_distributed()


if __name__ == "__main__":
    main()
