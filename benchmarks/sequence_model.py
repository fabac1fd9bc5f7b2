"""Long-sequence user-behaviour model benchmark (ragged behaviour sequences, target attention, transformer encoder).

Workload (defaults are the full shape; scale down with the flags): behaviour sequences of length ~ Uniform[50, 1000] of item ids
~ Zipf(1.1) over 1e8 with category ids over 1e5, item and category embeddings of width 64, 20 single-hot profile fields of width
32, target attention + 2-layer encoder (hidden 256, 4 heads) in bf16, MLP 512-256-1, BCE on Bernoulli(0.05) labels; global
batch 16384 = 2048 per rank at 8 ranks. Data parallel over ranks for the dense part, row-sharded embeddings.

Launch: ``python benchmarks/sequence_model.py`` (1 GPU, or CPU for a functional run at small sizes) or one process per GPU
through ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29542
benchmarks/sequence_model.py``. Rank 0 prints one JSON line; device-timed with CUDA events, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_batch(args, dev, seed, profile_fields):
    import torch
    from recis_b200.ragged import RaggedTensor
    from embedding_microbench import zipf_ids
    gen = torch.Generator(device=dev).manual_seed(seed)
    B = args.batch
    lens = torch.randint(args.min_len, args.max_len + 1, (B,), generator=gen, device=dev).to(torch.int32)
    offs = torch.zeros(B + 1, dtype=torch.int32, device=dev)
    offs[1:] = lens.cumsum(0)
    T = int(offs[-1])
    items = zipf_ids(T + B, 1.1, 1 << 27, gen, dev) % args.items          # 2^27 > 1e8: fold the scrambled rank into the id space
    cates = items % args.cates
    out = {
        "seq_item": RaggedTensor(items[:T], [offs], dense_shape=(B, -1)), "seq_cate": RaggedTensor(cates[:T], [offs], dense_shape=(B, -1)),
        "tgt_item": items[T:], "tgt_cate": cates[T:],
        "label": (torch.rand((B, 1), generator=gen, device=dev) < 0.05).float(), "max_len": int(lens.max()),
    }
    for i, f in enumerate(profile_fields):
        out[f] = torch.randint(0, 10_000 * (i + 1), (B,), generator=gen, device=dev)
    return out, T


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2048, help="per-rank batch (16384 / 8)")
    ap.add_argument("--min-len", type=int, default=50)
    ap.add_argument("--max-len", type=int, default=1000)
    ap.add_argument("--items", type=int, default=100_000_000)
    ap.add_argument("--cates", type=int, default=100_000)
    ap.add_argument("--profile-fields", type=int, default=20)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
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

    from recis_b200.models import SequenceModel
    from recis_b200.nn import filter_out_sparse_param
    from recis_b200.optim import DenseAdam, SparseAdam
    from recis_b200.parallel.dense_reducer import DenseGradReducer

    pf = [f"profile_{i}" for i in range(args.profile_fields)]
    n_batches = args.warmup + args.steps
    batches, tokens = [], 0
    for i in range(n_batches):
        b, T = make_batch(args, dev, 4001 * rank + i, pf)
        batches.append(b)
        tokens = max(tokens, T)
    torch.manual_seed(5)
    model = SequenceModel(pf, hidden=args.hidden, device=dev, item_capacity=int(tokens * min(n_batches, 8) * 0.7) + 65536,
                          cate_capacity=2 * args.cates // world + 65536, profile_capacity=args.profile_fields * 50_000,
                          compute_dtype=torch.bfloat16 if on_gpu else torch.float32, max_len=args.max_len).to(dev)
    sparse_opt = SparseAdam(filter_out_sparse_param(model), lr=1e-3)
    dense_params = [p for p in model.parameters() if p.requires_grad]
    dense_opt = DenseAdam(dense_params, lr=1e-3)
    reducer = DenseGradReducer(dense_params, world) if world > 1 else None

    def step(batch):
        loss, _ = model(batch)
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
        return loss.detach()

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
    for _tb in model.embedding_engine.tables().values():
        _ex = getattr(_tb, "fused", None)
        if _ex is not None:
            _ex.check()          # a timed-out wait or an overflowing window invalidates the measurement: fail instead of reporting it
    top = None
    if args.profile and on_gpu:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step(batches[-1])
            torch.cuda.synchronize()
        rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
        total = sum(e.device_time_total for e in rows)
        top = {"kernel_ms_total": total / 1e3,
               "kernels": [{"name": e.key[:90], "ms": round(e.device_time_total / 1e3, 3), "launches": e.count} for e in rows[:args.profile]]}
    from recis_b200.ops import attention as _att
    core = ("ragged tcgen05 attention kernels (no padding), one-kernel target attention" if on_gpu and _att._use_kernels()
            else "F.scaled_dot_product_attention on the padded view")
    if rank == 0:
        if top is not None:
            print(json.dumps({"profile": top}), flush=True)
        print(json.dumps({
            "bench": "sequence_model", "n_gpus": world, "per_rank_batch": args.batch, "global_batch": args.batch * world,
            "tokens_per_rank_per_step": tokens, "hidden": args.hidden, "ms_per_step": ms,
            "samples_per_s": args.batch * world / (ms / 1e3), "tokens_per_s": tokens * world / (ms / 1e3), "last_loss": float(loss),
            "attention_core": core + "; projections and FFN on the tcgen05 GEMM",
            "timing": "CUDA events, max over ranks" if on_gpu else "host clock (CPU run)",
        }), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
