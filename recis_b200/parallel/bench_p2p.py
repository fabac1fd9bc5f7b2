"""NVLink microbenchmark: bandwidth of plain peer stores / loads issued from a kernel, against NCCL all_to_all_single.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 recis_b200/parallel/bench_p2p.py [--mb 256]

Every rank copies ``mb`` MiB to (stores) and from (loads) its right neighbour's symmetric buffer; device-timed with CUDA
events, max over ranks. The NCCL line moves the same number of bytes per rank with ``all_to_all_single``."""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--mb", type=int, default=256)
    p.add_argument("--iters", type=int, default=10)
    args = p.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import recis_b200
    from recis_b200.parallel.symmetric import SymmetricHeap
    C = recis_b200.native()
    n = args.mb << 20
    dev = torch.device("cuda", local)
    heap = SymmetricHeap({"buf": (torch.uint8, n)}, dev)
    local_buf = torch.empty(n, dtype=torch.uint8, device=dev)
    peer = heap["buf"].ptrs[(rank + 1) % world]

    def timed(fn):
        fn(); torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    res = {}
    # small grids matter: the exchange runs its NVLink-bound kernels with capped grids next to other kernels
    for blocks in (37, 74, 148, 296, 148 * 4, 148 * 16):
        res[f"store_{blocks}"] = n / timed(lambda: C.comm_copy(peer, local_buf.data_ptr(), n, blocks)) / 1e6
        res[f"load_{blocks}"] = n / timed(lambda: C.comm_copy(local_buf.data_ptr(), peer, n, blocks)) / 1e6
    res["local_copy"] = n / timed(lambda: C.comm_copy(heap["buf"].tensor.data_ptr(), local_buf.data_ptr(), n, 148 * 16)) / 1e6
    out = torch.empty(n, dtype=torch.uint8, device=dev)
    res["nccl_all_to_all"] = n * (world - 1) / world / timed(lambda: dist.all_to_all_single(out, local_buf)) / 1e6
    if rank == 0:
        print({k: f"{v:.0f} GB/s" for k, v in res.items()})
    dist.barrier(); dist.destroy_process_group()


if __name__ == "__main__":
    main()
