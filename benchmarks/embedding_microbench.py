"""Embedding engine microbenchmark: many small tables merged into one, exchange bandwidth against NCCL.

Workload: ``--tables`` (200) logical tables of width ``--dim`` (64, fp32) that the EmbeddingEngine merges into one physical
table and one exchange per step; per-rank batch ``--batch`` (8192 ... 131072); bag length ~ Poisson(``--bag``); ids ~
Zipf(``--zipf``) over a 2^32 space per table. Timed on the device (CUDA events, max over ranks), separately:

  forward   dedup + owner routing + remote lookup-or-insert + embedding exchange + sum pooling
  backward  per-unique gradient reduction + gradient exchange + row-wise sparse Adagrad on the owning shard

and reported, per mode (``--comm fused`` = peer-memory kernels, ``--comm nccl`` = the same framework on NCCL
``all_to_all_single``), together with the bytes every rank sends over NVLink in each phase (unique rows that live on
another rank x row bytes) and the resulting achieved exchange bandwidth = bytes / phase time. For scale the script also
times a bare NCCL ``all_to_all_single`` of exactly those bytes, with nothing else in the phase.

Launch (one process per GPU):
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29540 \
      benchmarks/embedding_microbench.py --batch 8192 --zipf 1.05 [--comm nccl]
One JSON line per run is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def zipf_ids(n, a, space, gen, dev):
    """Continuous inverse-CDF sample of a Zipf(a) rank in [0, space), scrambled so that hot ids spread over all shards."""
    import torch
    u = torch.rand(n, generator=gen, device=dev, dtype=torch.float64)
    if abs(a - 1.0) < 1e-9:
        x = torch.exp(u * torch.log(torch.tensor(float(space), dtype=torch.float64, device=dev)))
    else:
        e = 1.0 - a
        x = torch.pow(1.0 + u * (float(space) ** e - 1.0), 1.0 / e)
    r = (x.floor().clamp_(1, float(space)) - 1).to(torch.int64)
    return (r * 0x9E3779B1 + 0x7F4A7C15) & (space - 1)       # odd multiplier: a bijection of the 2^k space


def make_batch(args, dev, seed):
    import torch
    from recis_b200.ragged import RaggedTensor
    gen = torch.Generator(device=dev).manual_seed(seed)
    lens = torch.poisson(torch.full((args.tables, args.batch), float(args.bag), device=dev), generator=gen).to(torch.int32)
    offs = torch.zeros((args.tables, args.batch + 1), dtype=torch.int32, device=dev)
    offs[:, 1:] = lens.cumsum(1)
    totals = offs[:, -1].tolist()
    ids = zipf_ids(sum(totals), args.zipf, 1 << 32, gen, dev)
    out, pos = {}, 0
    for t in range(args.tables):
        out[f"t{t}"] = RaggedTensor(ids[pos:pos + totals[t]], [offs[t]], dense_shape=(args.batch, -1))
        pos += totals[t]
    return out, sum(totals), ids


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tables", type=int, default=200)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--batch", type=int, default=8192, help="per-rank batch")
    ap.add_argument("--bag", type=float, default=10.0)
    ap.add_argument("--zipf", type=float, default=1.05)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--comm", default=None, choices=["fused", "nccl"])
    ap.add_argument("--capacity", type=int, default=0, help="table rows per rank (0: from the data)")
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16", "fp16"], help="storage (and wire) type of the embedding rows")
    args = ap.parse_args()
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
    dev = torch.device("cuda", local) if on_gpu else torch.device("cpu")      # CPU: functional smoke run only (gloo)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev) if on_gpu else dist.init_process_group("gloo")

    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseAdagrad

    n_batches = args.warmup + args.steps
    batches, nnz_max, uniq_max = [], 0, 0
    for i in range(n_batches):
        b, nnz, ids = make_batch(args, dev, 1000 * rank + i)
        batches.append(b)
        nnz_max = max(nnz_max, nnz)
        if i < 2:
            # distinct (table, id) pairs of this rank's batch bound the exchange window
            key = torch.cat([v.values() + (t << 40) for t, v in enumerate(b.values())])
            uniq_max = max(uniq_max, int(torch.unique(key).numel()))
            del key
        del ids
    if world > 1:                                  # sizes derived from the data must be the same on every rank
        t = torch.tensor([nnz_max, uniq_max], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        nnz_max, uniq_max = int(t[0]), int(t[1])
    xcap = int(uniq_max * 1.15) + 1024
    rows = args.capacity or int(min(xcap * (n_batches + 2), 120e9 / (args.dim * 8)) )
    per_table = max(rows // args.tables, 1)
    row_dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[args.dtype]
    # the exchange windows size themselves from the first batch's measured demand and grow with it
    opts = {f"t{t}": EmbeddingOption(embedding_dim=args.dim, shared_name=f"t{t}", combiner="sum", use_weight=False, device=dev,
                                     initializer=NormalInitializer(0.0, 0.01), capacity=per_table, dtype=row_dtype)
            for t in range(args.tables)}
    engine = EmbeddingEngine(opts, interleave=True)
    opt = SparseAdagrad(filter_out_sparse_param(engine), lr=0.01)
    gout = None

    class _HostEvent:                      # stand-in with the CUDA event interface for the CPU smoke run
        def record(self):
            import time
            self.t = time.perf_counter()

        def elapsed_time(self, other):
            return (other.t - self.t) * 1e3

    ev = (lambda: torch.cuda.Event(enable_timing=True)) if on_gpu else _HostEvent
    fwd_ms, bwd_ms = [], []

    def sync():
        if on_gpu:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            if on_gpu:
                torch.cuda.synchronize()

    for i in range(n_batches):
        sync()
        e0, e1, e2 = ev(), ev(), ev()
        e0.record()
        engine(batches[i])
        (cube, _names), = engine.packed.values()
        e1.record()
        if gout is None:
            gout = (torch.randn_like(cube.float()) * 1e-3).to(cube.dtype)
        cube.backward(gout)
        opt.step()
        opt.zero_grad()
        e2.record()
        sync()
        if i >= args.warmup:
            fwd_ms.append(e0.elapsed_time(e1))
            bwd_ms.append(e1.elapsed_time(e2))

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _tb in engine.tables().values():
        _ex = getattr(_tb, "fused", None)
        if _ex is not None:
            _ex.check()          # a timed-out wait or an overflowing window invalidates the measurement: fail instead of reporting it
    fwd = max_over_ranks(sum(fwd_ms) / len(fwd_ms))
    bwd = max_over_ranks(sum(bwd_ms) / len(bwd_ms))
    # bytes this rank receives in the forward phase (= sends in the backward phase): unique rows owned elsewhere
    remote_rows = uniq_max * (world - 1) / max(world, 1)
    row_bytes = args.dim * torch.empty(0, dtype=row_dtype).element_size()      # forward: rows travel in their storage type
    xbytes = remote_rows * row_bytes
    xbytes_bwd = remote_rows * args.dim * 4                                     # backward: per-unique gradients travel as fp32
    nccl_ms = None
    if world > 1:
        n = int(remote_rows) * args.dim // world * world
        src = torch.empty(n, dtype=row_dtype, device=dev)
        dst = torch.empty_like(src)
        for _ in range(3):
            dist.all_to_all_single(dst, src)
        sync()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(10):
            dist.all_to_all_single(dst, src)
        e1.record()
        sync()
        nccl_ms = max_over_ranks(e0.elapsed_time(e1) / 10)
    if rank == 0:
        print(json.dumps({
            "bench": "embedding_microbench", "comm": os.environ.get("RECIS_COMM", "auto"), "n_gpus": world,
            "tables": args.tables, "dim": args.dim, "per_rank_batch": args.batch, "bag": args.bag, "zipf": args.zipf,
            "ids_per_rank": nnz_max, "unique_per_rank": uniq_max, "duplicate_ratio": 1.0 - uniq_max / max(nnz_max, 1),
            "forward_ms": fwd, "backward_update_ms": bwd,
            "samples_per_s": args.batch * world / ((fwd + bwd) / 1e3),
            "row_dtype": args.dtype, "forward_exchange_bytes_per_rank": xbytes, "backward_exchange_bytes_per_rank": xbytes_bwd,
            "forward_exchange_gbs": xbytes / (fwd / 1e3) / 1e9 if world > 1 else None,
            "backward_exchange_gbs": xbytes_bwd / (bwd / 1e3) / 1e9 if world > 1 else None,
            "bare_nccl_all_to_all_ms": nccl_ms,
            "bare_nccl_all_to_all_gbs": xbytes / (nccl_ms / 1e3) / 1e9 if nccl_ms else None,
            "timing": "CUDA events, max over ranks, inputs device resident, table rows + state far larger than L2",
        }), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
