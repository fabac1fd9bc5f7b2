"""Peer-mapped ("symmetric") device memory for one-process-per-GPU jobs on an NVLink/NVSwitch node.

Every rank allocates the same layout with ``cudaMalloc`` (outside torch's caching allocator), exports a cudaIpc handle,
and opens the handles of all other ranks; kernels then take one raw pointer per rank. ``torch.distributed`` is used only
to exchange the 64-byte handles. Regions are carved out of one allocation, so the pointer of region ``x`` on rank ``r``
is ``base[r] + offset(x)`` on every rank.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from .. import native

_DT_SIZE = {torch.int64: 8, torch.int32: 4, torch.float32: 4, torch.uint8: 1, torch.int8: 1, torch.bfloat16: 2, torch.float16: 2}


def single_node(world: int) -> bool:
    """Peer-mapped (or shared) memory needs all ranks on one machine. Launchers export ``LOCAL_WORLD_SIZE``; when it is smaller
    than the world size the job spans machines and the exchange must use collectives. Without the variable (ranks spawned by
    hand on one machine) the job is taken to be local."""
    import os
    return int(os.environ.get("LOCAL_WORLD_SIZE", world)) >= world


class SymmetricRegion:
    def __init__(self, tensor: torch.Tensor, ptrs: List[int]):
        self.tensor = tensor      # this rank's view
        self.ptrs = ptrs          # device pointer of the same region on every rank (own pointer at own rank)


class SymmetricHeap:
    """One symmetric allocation with named, 256-byte aligned regions of identical layout on all ranks."""

    def __init__(self, regions: Dict[str, Tuple[torch.dtype, int]], device: torch.device, pg=None):
        self.device = torch.device(device)
        self.pg = pg
        self.world = dist.get_world_size(pg)
        self.rank = dist.get_rank(pg)
        C = native()
        assert self.world <= C.MAX_PEERS, f"fused exchange supports up to {C.MAX_PEERS} ranks"
        layout, off = {}, 0
        for name, (dtype, numel) in regions.items():
            nbytes = (int(numel) * _DT_SIZE[dtype] + 255) // 256 * 256
            layout[name] = (off, dtype, int(numel))
            off += nbytes
        self.nbytes = off
        self._opened = []
        bases = []
        if self.device.type == "cuda":
            self.base, handle = C.sym_alloc(self.nbytes, self.device.index)
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=pg)
            for r in range(self.world):
                if r == self.rank:
                    bases.append(self.base.data_ptr())
                else:
                    p = C.sym_open(handles[r], self.device.index)
                    self._opened.append(p)
                    bases.append(p)
        else:
            # host twin (CPU ranks of one machine): a POSIX shared-memory object per rank, mapped by every rank
            import os
            import uuid
            shm_name = f"/recis_b200_{os.getpid()}_{uuid.uuid4().hex[:12]}"
            self.base = C.shm_alloc(shm_name, self.nbytes)
            names = [None] * self.world
            dist.all_gather_object(names, shm_name, group=pg)
            for r in range(self.world):
                if r == self.rank:
                    bases.append(self.base.data_ptr())
                else:
                    p, mapped = C.shm_open_peer(names[r])
                    self._opened.append((p, mapped))
                    bases.append(p)
        self.regions: Dict[str, SymmetricRegion] = {}
        for name, (o, dtype, numel) in layout.items():
            view = self.base[o:o + numel * _DT_SIZE[dtype]].view(dtype)
            self.regions[name] = SymmetricRegion(view, [b + o for b in bases])
        dist.barrier(group=pg)   # nobody touches a peer's memory before everyone has mapped it
        if self.device.type != "cuda":
            C.shm_unlink_name(shm_name)      # everybody holds a mapping now: the name can go

    def __getitem__(self, name) -> SymmetricRegion:
        return self.regions[name]

    def close(self):
        C = native()
        for p in self._opened:
            if isinstance(p, tuple):
                C.shm_close(*p)
            else:
                C.sym_close(p)
        self._opened = []
