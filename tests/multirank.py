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
        if env.get("RB_NO_FINAL_BARRIER") == "1":
            os._exit(0)                          # a peer may be gone on purpose: do not wait for it in a barrier
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(outdir, f"rank{rank}.err"), "w") as fh:
            fh.write(traceback.format_exc())
        raise


def run_ranks(fn, world, backend="gloo", args=(), env=None, timeout=300, allow_missing=False):
    """Run ``fn(rank, world, *args)`` on ``world`` child processes; returns the list of per-rank results (``None`` for a rank that
    left no result when ``allow_missing`` is set)."""
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
    outs = []
    for r in range(world):
        f = os.path.join(outdir, f"rank{r}.pt")
        if allow_missing and not os.path.exists(f):
            outs.append(None)
        else:
            outs.append(torch.load(f, weights_only=False))
    return outs
