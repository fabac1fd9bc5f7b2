"""Helpers to run a function on several ranks (child processes) and collect what each rank returns."""
import os
import socket
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, backend, port, fn, args, outdir, env):
    try:
        os.environ.update(env)
        os.environ["WORLD_SIZE"], os.environ["RANK"], os.environ["LOCAL_RANK"] = str(world), str(rank), str(rank)
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        if backend == "nccl":
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        torch.save(out, os.path.join(outdir, f"rank{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(outdir, f"rank{rank}.err"), "w") as fh:
            fh.write(traceback.format_exc())
        raise


def run_ranks(fn, world, backend="gloo", args=(), env=None, timeout=300):
    """Run ``fn(rank, world, *args)`` on ``world`` child processes; returns the list of per-rank results."""
    outdir = tempfile.mkdtemp(prefix="rb_ranks_")
    ctx = mp.get_context("spawn")
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, backend, port, fn, args, outdir, dict(env or {}))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    errs = []
    for r, p in enumerate(procs):
        if p.is_alive():
            p.kill()
            errs.append(f"rank {r} timed out")
        err = os.path.join(outdir, f"rank{r}.err")
        if os.path.exists(err):
            errs.append(open(err).read())
    if errs:
        raise RuntimeError("\n".join(errs))
    return [torch.load(os.path.join(outdir, f"rank{r}.pt"), weights_only=False) for r in range(world)]
