"""Production-scale multi-table model: many sparse fields of mixed widths behind the feature engine, admission by count,
TTL eviction and a sparse checkpoint round trip.

Workload (defaults are the full shape; ``--fields/--batch`` scale it down):
  * ``--fields`` (1000) sparse fields; widths cycle through {8, 16, 32, 64, 128}; the EmbeddingEngine merges all fields of one
    width (same initializer, same hooks) into one physical table, so five tables and five exchanges serve the thousand fields;
  * multi-hot bag length ~ Geometric(0.2) capped at 50;
  * raw features go through the FeatureEngine first: 40 % of the fields are raw int64 ids reduced with ``Mod``, 40 % are
    8-byte strings hashed with ``Hash("farm")``, 20 % are floats binned with ``Bucketize`` over 200 boundaries; equal ops of
    all fields run as one fused launch per op type;
  * ids ~ Zipf(``--zipf``) over a 2^48 space; a row is created when its id has been seen ``--admit`` (2) times; rows not
    seen for ``--ttl`` steps are evicted every ``--filter-interval`` steps;
  * dense tower MLP 2048-1024-512-1 in bf16 over the concatenated pooled embeddings, BCE loss, sparse Adam + dense Adam;
  * after the timed steps: SafeTensors sparse checkpoint save, load into a freshly built model, and a check that table sizes
    and a probe batch's embeddings agree.

Launch: ``python benchmarks/multitable.py`` (1 GPU) or one process per GPU through ``python -m torch.distributed.run
--nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29541 benchmarks/multitable.py``; rank 0 prints one JSON
line. Device-timed with CUDA events, max over ranks. Runs on CPU (gloo) too, for functional checks at small sizes.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

DIMS = (8, 16, 32, 64, 128)
KINDS = ("mod", "mod", "hash", "hash", "bucket")        # 40 % / 40 % / 20 %


def field_plan(n_fields):
    return [(f"f{i}", DIMS[i % len(DIMS)], KINDS[(i // len(DIMS)) % len(KINDS)]) for i in range(n_fields)]


def build_model(plan, dev, rows_per_rank, xcap_total, admit, ttl):
    import torch
    from torch import nn
    from recis_b200.features import Bucketize, Feature, FeatureEngine, Hash, Mod, SelectField
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption
    from recis_b200.nn.hashtable_hook import AdmitHook, FilterHook
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.ops.dense import MLP

    boundaries = torch.linspace(-3.0, 3.0, 200).tolist()
    feats = []
    for name, _dim, kind in plan:
        f = Feature(name).add_op(SelectField(name, dtype=torch.float32 if kind == "bucket" else torch.long))
        if kind == "mod":
            f.add_op(Mod((1 << 47) - 115))
        elif kind == "hash":
            f.add_op(Hash("farm"))
        else:
            f.add_op(Bucketize(boundaries))
        feats.append(f)
    init = NormalInitializer(0.0, 0.01)
    share = 1.0 / max(len(plan), 1)
    opts = {
        name: EmbeddingOption(embedding_dim=dim, shared_name=name, combiner="sum", use_weight=False, device=dev, initializer=init,
                              admit_hook=AdmitHook("CountAdmit", {"threshold": admit}) if admit > 1 else None,
                              filter_hook=FilterHook("GlobalStepFilter", {"filter_step": ttl}) if ttl > 0 else None,
                              capacity=int(rows_per_rank * share), exchange_capacity=int(xcap_total * share) + 1)
        for name, dim, _k in plan
    }

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.feature_engine = FeatureEngine(feats)
            self.embedding_engine = EmbeddingEngine(opts, interleave=True)
            self.width = sum(d for _n, d, _k in plan)
            self.mlp = MLP([self.width, 2048, 1024, 512, 1], final_act=False)
            self.loss_fn = nn.BCEWithLogitsLoss()

        def embed(self, batch):
            data = self.feature_engine({n: batch[n] for n, _d, _k in plan})
            self.embedding_engine({n: data[n] for n, _d, _k in plan})
            cubes = [c.reshape(c.shape[0], -1) for c, _names in self.embedding_engine.packed.values()]
            return torch.cat(cubes, dim=1)

        def forward(self, batch):
            x = self.embed(batch)
            logit = self.mlp(x)[:, :1].float()
            return self.loss_fn(logit, batch["label"])

    return Model().to(dev)


def make_batch(plan, batch, zipf_a, dev, seed):
    """Raw features of one step, generated on the device: int64 ids, 8-byte strings, floats; all ragged [batch, *]."""
    import torch
    from recis_b200.ragged import RaggedTensor
    from embedding_microbench import zipf_ids
    gen = torch.Generator(device=dev).manual_seed(seed)
    F = len(plan)
    u = torch.rand((F, batch), generator=gen, device=dev)
    lens = (torch.log1p(-u) / -0.2231435513).floor().clamp_(0, 49).to(torch.int32) + 1     # Geometric(0.2) on {1..50}
    offs = torch.zeros((F, batch + 1), dtype=torch.int32, device=dev)
    offs[:, 1:] = lens.cumsum(1)
    totals = offs[:, -1].tolist()
    ids = zipf_ids(sum(totals), zipf_a, 1 << 48, gen, dev)
    out, pos = {}, 0
    for i, (name, _dim, kind) in enumerate(plan):
        n = totals[i]
        v = ids[pos:pos + n]
        pos += n
        if kind == "mod":
            out[name] = RaggedTensor(v, [offs[i]], dense_shape=(batch, -1))
        elif kind == "hash":
            chars = v.contiguous().view(torch.int8)                         # the id's 8 bytes are the string
            inner = torch.arange(0, 8 * n + 1, 8, dtype=torch.int32, device=dev)
            out[name] = RaggedTensor(chars, [offs[i], inner], dense_shape=(batch, -1, -1))
        else:
            x = (v & 0xFFFF).to(torch.float32) / 65536.0 * 6.0 - 3.0
            out[name] = RaggedTensor(x, [offs[i]], dense_shape=(batch, -1))
    out["label"] = (torch.rand((batch, 1), generator=gen, device=dev) < 0.03).float()
    return out, sum(totals)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--fields", type=int, default=1000)
    ap.add_argument("--batch", type=int, default=16384, help="per-rank batch (131072 / 8)")
    ap.add_argument("--zipf", type=float, default=1.05)
    ap.add_argument("--admit", type=int, default=2)
    ap.add_argument("--ttl", type=int, default=8)
    ap.add_argument("--filter-interval", type=int, default=4)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--rows", type=int, default=0, help="table rows per rank over all tables (0: from the data)")
    ap.add_argument("--ckpt-dir", default=None)
    ap.add_argument("--skip-checkpoint", action="store_true", help="time the training steps only (the round trip writes tens of GB per rank)")
    ap.add_argument("--profile", type=int, default=0, help="after the timed steps, list the N kernels with the most device time in one more step")
    ap.add_argument("--comm", default=None, choices=["fused", "nccl"])
    ap.add_argument("--stage-exchange", action="store_true",
                    help="fused exchange: issue every table group's id phase and owner side before the first wait (RECIS_STAGE_EXCHANGE=1)")
    args = ap.parse_args()
    if args.stage_exchange:
        os.environ["RECIS_STAGE_EXCHANGE"] = "1"
    if args.comm:
        os.environ["RECIS_COMM"] = args.comm

    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if on_gpu else torch.device("cpu")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev) if on_gpu else dist.init_process_group("gloo")

    from recis_b200.hooks import HashTableFilterHook
    from recis_b200.nn import filter_out_sparse_param
    from recis_b200.nn.modules.hashtable import HashtableRegister
    from recis_b200.optim import DenseAdam, SparseAdam
    from recis_b200.parallel.dense_reducer import DenseGradReducer
    from recis_b200.serialize import Loader, Saver

    plan = field_plan(args.fields)
    n_batches = args.warmup + args.steps
    batches, nnz = [], 0
    for i in range(n_batches):
        b, n = make_batch(plan, args.batch, args.zipf, dev, 7919 * rank + i)
        batches.append(b)
        nnz = max(nnz, n)
    # admission keeps most ids of a step out of the tables, and the tables grow in place when they fill up: start small
    rows = args.rows or nnz // 4 + 4096
    torch.manual_seed(99)
    model = build_model(plan, dev, rows, int(nnz * 1.05) + 4096, args.admit, args.ttl)
    sparse_opt = SparseAdam(filter_out_sparse_param(model), lr=1e-3)
    dense_params = [p for p in model.parameters() if p.requires_grad]
    dense_opt = DenseAdam(dense_params, lr=1e-3)
    reducer = DenseGradReducer(dense_params, world) if world > 1 else None
    evict = HashTableFilterHook(filter_interval=args.filter_interval, model=model) if args.ttl > 0 else None

    def step(batch):
        loss = model(batch)
        if reducer is None:
            dense_opt.zero_grad(set_to_none=False)
        loss.backward()
        if reducer is not None:
            reducer.all_reduce_async()
        sparse_opt.step()
        sparse_opt.zero_grad()
        if reducer is not None:
            reducer.wait()
        dense_opt.step()
        if evict is not None:
            evict.after_step()
        return loss

    def sync():
        if on_gpu:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            if on_gpu:
                torch.cuda.synchronize()

    for i in range(args.warmup):
        step(batches[i])
    sync()
    t0 = time.perf_counter()
    if on_gpu:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    for i in range(args.warmup, n_batches):
        loss = step(batches[i])
    if on_gpu:
        e1.record()
    sync()
    ms = e0.elapsed_time(e1) if on_gpu else (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / args.steps

    if args.profile and on_gpu:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step(batches[-1])
            torch.cuda.synchronize()
        kernels = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
        if rank == 0:
            print(json.dumps({"profile": {"kernel_ms_total": sum(e.device_time_total for e in kernels) / 1e3, "kernels": [
                {"name": e.key[:90], "ms": round(e.device_time_total / 1e3, 3), "launches": e.count} for e in kernels[:args.profile]]}}), flush=True)

    tables = model.embedding_engine.tables()
    for _tb in tables.values():
        _ex = getattr(_tb, "fused", None)
        if _ex is not None:
            _ex.check()          # a timed-out wait or an overflowing window invalidates the measurement: fail instead of reporting it
    sizes = {str(tb.impl.dim): int(tb.impl.size()) for tb in tables.values()}

    save_s = load_s = ckpt_bytes = same = None
    if not args.skip_checkpoint:
        # ---- sparse checkpoint round trip into a freshly built model
        ckpt = args.ckpt_dir or tempfile.mkdtemp(prefix="recis_b200_ckpt_")
        if world > 1:
            box = [ckpt]
            dist.broadcast_object_list(box, src=0)
            ckpt = box[0]
        os.makedirs(ckpt, exist_ok=True)
        probe = batches[-1]
        model.eval()
        with torch.no_grad():
            ref = model.embed(probe)
        sync()
        t0 = time.perf_counter()
        dense_state = {k: v for k, v in model.state_dict().items() if isinstance(v, torch.Tensor)} if rank == 0 else {}
        Saver(rank, world, 4, ckpt, filter_out_sparse_param(model), dense_state).save()
        sync()
        save_s = time.perf_counter() - t0
        ckpt_bytes = sum(os.path.getsize(os.path.join(ckpt, f)) for f in os.listdir(ckpt)) if rank == 0 else 0
        HashtableRegister().clear()
        model2 = build_model(plan, dev, rows, int(nnz * 1.05) + 4096, args.admit, args.ttl)
        t0 = time.perf_counter()
        Loader(ckpt, filter_out_sparse_param(model2), {}).load()
        sync()
        load_s = time.perf_counter() - t0
        model2.eval()
        with torch.no_grad():
            got = model2.embed(probe)
        sizes2 = {str(tb.impl.dim): int(tb.impl.size()) for tb in model2.embedding_engine.tables().values()}
        same = bool(torch.equal(ref, got)) and sizes == sizes2
        sync()
        if rank == 0 and args.ckpt_dir is None:
            shutil.rmtree(ckpt, ignore_errors=True)

    if rank == 0:
        print(json.dumps({
            "bench": "multitable", "n_gpus": world, "fields": args.fields, "per_rank_batch": args.batch, "global_batch": args.batch * world,
            "ids_per_rank_per_step": nnz, "ms_per_step": ms, "samples_per_s": args.batch * world / (ms / 1e3),
            "physical_tables": len(tables), "rows_by_width_rank0": sizes, "evicted_rows_rank0": evict.evicted if evict else 0,
            "admit_threshold": args.admit, "ttl_steps": args.ttl, "last_loss": float(loss.detach()),
            "checkpoint": {"save_s": save_s, "load_s": load_s, "bytes": ckpt_bytes, "round_trip_identical": same},
            "comm": os.environ.get("RECIS_COMM", "auto"), "staged_exchange": os.environ.get("RECIS_STAGE_EXCHANGE") == "1",
            "timing": "CUDA events around the timed steps, max over ranks" if on_gpu else "host clock (CPU run)",
        }), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
