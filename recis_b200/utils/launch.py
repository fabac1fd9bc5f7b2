"""Process-group set-up for programs started by ``torch.distributed.run`` (one process per GPU, or CPU ranks).

``init_distributed()`` reads ``RANK`` / ``WORLD_SIZE`` / ``LOCAL_RANK`` / ``MASTER_*`` from the environment, picks NCCL when
CUDA is used and gloo otherwise, binds the process to its GPU and returns ``(rank, world, device)``; with a single process it
does nothing and returns ``(0, 1, device)``. The reference's examples call ``dist.init_process_group()`` themselves
(``examples/deepfm/runner.py:103``); this is the same step with the device binding added.
"""
from __future__ import annotations

import os
from datetime import timedelta
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def init_distributed(device: Optional[str] = None, timeout_s: float = 1800.0) -> Tuple[int, int, torch.device]:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    kind = device or ("cuda" if torch.cuda.is_available() else "cpu")
    kind = torch.device(kind).type
    if kind == "cuda":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    if world > 1 and not (dist.is_available() and dist.is_initialized()):
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kw = dict(timeout=timedelta(seconds=timeout_s), rank=rank, world_size=world)
        if kind == "cuda":
            dist.init_process_group("nccl", device_id=dev, **kw)
        else:
            dist.init_process_group("gloo", **kw)
    return rank, world, dev


def finish_distributed() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
