"""Where one DLRM training step spends its time: device time per kernel (PyTorch profiler) and host time per native call.

Builds the same model, optimizers and synthetic batches as ``bench.py``, warms up, then
  * ``--mode kernels``: records three steps with ``torch.profiler`` and prints the kernels by device time (rank 0);
  * ``--mode timeline``: records two steps and prints, for rank 0, every kernel of the second step in start order with its
    stream, start offset and duration - shows what really overlaps when the exchange lanes run on two streams;
  * ``--mode host``: wraps every function of the native module with a wall-clock timer, runs twelve steps without any
    synchronisation and prints the host time per step and per native call (ranks 0 and 3) - a call that blocks on the GPU
    shows up here as milliseconds instead of microseconds.

Launch: ``python benchmarks/step_profile.py`` on one GPU, or one process per GPU:
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29519 \
      benchmarks/step_profile.py --mode kernels
Numbers printed under the profiler are for shares, not for reporting: report ``bench.py``'s CUDA-event timings.
"""
from __future__ import annotations

import argparse
import collections
import os
import sys
import time
import types

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="kernels", choices=["kernels", "host", "timeline"])
    ap.add_argument("--batch-per-gpu", type=int, default=8192)
    ap.add_argument("--capacity", type=int, default=0)
    ap.add_argument("--all-ranks", action="store_true", help="kernels mode: every rank prints its ten heaviest kernels")
    a = ap.parse_args()

    import torch
    import torch.distributed as dist
    import bench
    import recis_b200
    from recis_b200.io.synthetic import make_batch_arrays

    acc = collections.defaultdict(lambda: [0.0, 0])
    if a.mode == "host":
        C = recis_b200.native()

        def wrap(name, fn):
            def w(*args, **kw):
                t0 = time.perf_counter()
                r = fn(*args, **kw)
                d = acc[name]
                d[0] += time.perf_counter() - t0
                d[1] += 1
                return r
            return w
        for n in dir(C):
            f = getattr(C, n)
            if isinstance(f, types.BuiltinFunctionType):
                setattr(C, n, wrap(n, f))
        for n in ("lookup_or_insert", "find"):
            setattr(C.EmbeddingStore, n, wrap("store." + n, getattr(C.EmbeddingStore, n)))

    class Args:
        pass
    args = Args()
    args.batch_per_gpu = a.batch_per_gpu
    args.gpus = int(os.environ.get("WORLD_SIZE", "1"))
    world, rank, local = bench.dist_setup(args)
    arm = bench.OursArm()
    dev = torch.device("cuda", local)
    fields, spec = bench.spec_for(args, rank)
    capacity = a.capacity or min(int(1.15 * bench.UNIVERSE / world) + 8_000_000, 72_000_000)
    st = arm.build(fields, dev, world, rank, capacity)
    n_batches = 20
    host = [arm.wrap_host(make_batch_arrays(spec, i), spec.batch) for i in range(n_batches)]
    devb = [arm.to_device(b, dev) for b in host]
    for i in range(8):
        arm.step(st, devb[i])
    bench.sync_all(world)

    if a.mode == "kernels":
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            for i in range(8, 11):
                arm.step(st, devb[i])
            torch.cuda.synchronize()
        if rank == 0:
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=60))
        if a.all_ranks:
            # kernel durations differ between ranks (link contention, owner load): the step waits for the slowest one
            rows = sorted(((e.self_device_time_total / 3e3, e.key) for e in prof.key_averages() if e.self_device_time_total > 0),
                          reverse=True)[:10]
            for r in range(world):
                if rank == r:
                    print(f"[rank {rank}] " + "; ".join(f"{k[:40]} {t:.3f} ms" for t, k in rows), flush=True)
                if world > 1:
                    dist.barrier()
    elif a.mode == "timeline":
        import json
        import tempfile
        from torch.profiler import ProfilerActivity, profile
        marks = []
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(8, 10):
                arm.step(st, devb[i])
                ev = torch.cuda.Event(enable_timing=False)
                marks.append(ev)
            torch.cuda.synchronize()
        if rank == 0:
            with tempfile.TemporaryDirectory() as td:
                path = os.path.join(td, "trace.json")
                prof.export_chrome_trace(path)
                with open(path) as fh:
                    trace = json.load(fh)
            ks = [e for e in trace["traceEvents"] if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and "dur" in e]
            ks.sort(key=lambda e: e["ts"])
            # second step = the kernels after the midpoint gap: split at the launch of the second step's first encode/dedup kernel
            names = [e["name"] for e in ks]
            firsts = [i for i, n in enumerate(names) if "encode_merge" in n]
            per_step = len(firsts) // 2 if len(firsts) >= 2 else 0
            begin = firsts[per_step] if per_step else 0
            t0 = ks[begin]["ts"]
            streams = {}
            busy = collections.defaultdict(float)
            print(f"timeline of one step on rank 0 ({len(ks) - begin} device activities); columns: start ms, duration ms, stream, name")
            for e in ks[begin:]:
                sid = streams.setdefault(e["args"].get("stream", 0), len(streams))
                busy[sid] += e["dur"] / 1e3
                if e["dur"] >= 15:           # microseconds: list what matters, count the rest
                    print(f"{(e['ts'] - t0) / 1e3:8.3f} {e['dur'] / 1e3:7.3f}  s{sid}  {e['name'][:70]}")
            end = max(e["ts"] + e["dur"] for e in ks[begin:])
            print(f"step span {(end - t0) / 1e3:.3f} ms; busy per stream: " + ", ".join(f"s{k} {v:.3f} ms" for k, v in sorted(busy.items())))
    else:
        acc.clear()
        steps = []
        t0 = time.perf_counter()
        for i in range(8, 20):
            t1 = time.perf_counter()
            arm.step(st, devb[i])
            steps.append(time.perf_counter() - t1)
        issue = time.perf_counter() - t0
        bench.sync_all(world)
        wall = time.perf_counter() - t0
        for r in (0, 3):
            if rank == r:
                print(f"[rank {rank}] host issue {issue / 12 * 1e3:.2f} ms/step, wall {wall / 12 * 1e3:.2f} ms/step; per step: "
                      + " ".join(f"{x * 1e3:.1f}" for x in steps))
                for k, (t, n) in sorted(acc.items(), key=lambda kv: -kv[1][0])[:14]:
                    print(f"[rank {rank}] {k:28s} {t / 12 * 1e3:8.3f} ms/step  {n / 12:6.1f} calls/step")
            if world > 1:
                dist.barrier()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
