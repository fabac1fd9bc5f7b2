"""Benchmark arm that runs the UNMODIFIED reference (installed under ``baseline/_ref``) through its own public API:
``recis.nn.EmbeddingEngine`` / ``EmbeddingOption``, ``recis.optim.SparseAdam``, ``recis.ragged.tensor.RaggedTensor``,
with a plain PyTorch dense tower (nn.Linear under bf16 autocast, DDP for more than one GPU), as the reference's
own examples do (``examples/deepfm/deepfm_model.py``, ``examples/deepfm/runner.py``). Nothing from ``recis_b200``
(models, kernels, engine) is on this path; only the seeded numpy batch generator is shared so both arms see the same data.
"""
from __future__ import annotations

import os
import sys

_REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def unavailable_reason():
    if not os.path.exists(os.path.join(_REF, "recis", "lib", "recis.so")):
        return "reference is not installed under baseline/_ref (offline build did not produce recis/lib/recis.so)"
    try:
        import torch
        if not torch.cuda.is_available():
            return "reference pooling kernels are CUDA-only and no CUDA device is visible"
    except Exception as e:  # pragma: no cover
        return f"torch import failed: {e}"
    return None


def _import_ref():
    if _REF not in sys.path:
        sys.path.insert(0, _REF)
    import recis  # noqa: F401
    return recis


class ReferenceArm:
    name = "reference"

    def build(self, fields, dev, world, rank, capacity):
        import torch
        from torch import nn
        _import_ref()
        from recis.nn import EmbeddingEngine, EmbeddingOption
        from recis.nn.initializers import TruncNormalInitializer
        from recis.nn.modules.hashtable import filter_out_sparse_param
        from recis.optim import SparseAdam

        import torch.distributed as dist
        if not dist.is_initialized():
            # the reference's DynamicEmbedding reads the default process group even on one GPU
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
        torch.manual_seed(1234)
        D = 128

        class Sparse(nn.Module):
            def __init__(self):
                super().__init__()
                self.engine = EmbeddingEngine({
                    f: EmbeddingOption(embedding_dim=D, shared_name=f, combiner="sum", use_weight=False, device=dev,
                                       initializer=TruncNormalInitializer(std=0.01)) for f in fields})

            def forward(self, feats):
                return self.engine(feats)

        class Dense(nn.Module):
            def __init__(self):
                super().__init__()
                def mlp(dims, final_act):
                    layers = []
                    for i in range(len(dims) - 1):
                        layers.append(nn.Linear(dims[i], dims[i + 1]))
                        if i < len(dims) - 2 or final_act:
                            layers.append(nn.ReLU())
                    return nn.Sequential(*layers)
                n = len(fields) + 1
                self.bottom = mlp([13, 512, 256, D], True)
                self.top = mlp([D + n * (n - 1) // 2, 1024, 1024, 512, 256, 1], False)
                li, lj = torch.tril_indices(n, n, offset=-1)
                self.register_buffer("li", li); self.register_buffer("lj", lj)

            def forward(self, dense, embs):
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    x = self.bottom(dense)
                    z = torch.cat([x.unsqueeze(1), torch.stack(embs, dim=1).to(x.dtype)], dim=1)
                    zz = torch.bmm(z, z.transpose(1, 2))
                    feat = torch.cat([x, zz[:, self.li, self.lj]], dim=1)
                    return self.top(feat).float()

        sparse = Sparse().to(dev)
        dense = Dense().to(dev)
        sparse_opt = SparseAdam(filter_out_sparse_param(sparse), lr=1e-3)
        dense_opt = torch.optim.Adam(dense.parameters(), lr=1e-3, fused=True)
        if world > 1:
            dense = nn.parallel.DistributedDataParallel(dense, device_ids=[dev.index])
        return dict(sparse=sparse, dense=dense, sparse_opt=sparse_opt, dense_opt=dense_opt, fields=list(fields),
                    loss=torch.nn.BCEWithLogitsLoss())

    def wrap_host(self, arrays, batch):
        import numpy as np
        import torch
        out = {}
        for k, v in arrays.items():
            if isinstance(v, tuple):
                out[k] = (torch.from_numpy(v[0]).pin_memory(), torch.from_numpy(v[1]).pin_memory(), batch)
            else:
                out[k] = torch.from_numpy(np.ascontiguousarray(v)).pin_memory()
        return out

    def nbytes(self, b):
        n = 0
        for v in b.values():
            ts = v[:2] if isinstance(v, tuple) else (v,)
            n += sum(t.numel() * t.element_size() for t in ts)
        return n

    def to_device(self, b, dev):
        from recis.ragged.tensor import RaggedTensor
        out = {}
        for k, v in b.items():
            if isinstance(v, tuple):
                out[k] = RaggedTensor(v[0].to(dev, non_blocking=True), [v[1].to(dev, non_blocking=True)], dense_shape=(v[2], -1))
            else:
                out[k] = v.to(dev, non_blocking=True)
        return out

    def feeder(self, host_batches, dev):
        # stock path: the reference's Trainer copies each batch right before its step (recis/framework/trainer.py,
        # copy_data_to_device on the current stream); it has no device prefetcher outside its column-io packer
        for b in host_batches:
            yield self.to_device(b, dev)

    LOSS_READ = "every step: float(loss) at the end of the step"

    def step(self, st, batch):
        embs = st["sparse"]({f: batch[f] for f in st["fields"]})
        logit = st["dense"](batch["dense"], [embs[f] for f in st["fields"]])
        loss = st["loss"](logit, batch["label"])
        st["dense_opt"].zero_grad(); st["sparse_opt"].zero_grad()
        loss.backward()
        st["dense_opt"].step(); st["sparse_opt"].step()
        return loss.detach()

    def launches(self):
        return 0

    def table_rows(self, st, world):
        """Rows in the reference's tables over all ranks, through its public ``HashTable.ids()`` (read between regions, outside all
        timing); None when that call is not available."""
        import torch
        import torch.distributed as dist
        try:
            n = 0
            for emb in st["sparse"].engine._ht.values():
                n += int(emb._hashtable.ids().numel())
        except Exception:
            return None
        if world > 1:
            t = torch.tensor([n], dtype=torch.int64, device="cuda")
            dist.all_reduce(t)
            n = int(t.item())
        return n

    def exposed_comm_ms(self, st, host_batches, dev, world, steps):
        """Device time per step of the reference's all-to-all kernels (NCCL send/receive kernels in a torch-profiler window over
        ``steps`` extra steps after the timed regions), max over ranks: its collectives run on the model's stream, so all of that
        time is exposed."""
        import torch
        import torch.distributed as dist
        if world == 1:
            return {"total": 0.0, "note": "single GPU: the all-to-alls are local copies"}
        from torch.profiler import ProfilerActivity, profile
        batches = [self.to_device(b, dev) for b in host_batches[-steps:]]
        torch.cuda.synchronize(); dist.barrier()
        total_us, err = -1.0, None
        try:
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for b in batches:
                    self.step(st, b)
                torch.cuda.synchronize()
            total_us = 0.0
            for ev in prof.key_averages():
                name = ev.key.lower()
                if "nccl" in name and ("sendrecv" in name or "alltoall" in name):
                    total_us += float(getattr(ev, "device_time_total", 0.0) or getattr(ev, "cuda_time_total", 0.0))
        except Exception as e:
            err = repr(e)
            for b in batches[:0]:
                pass
        t = torch.tensor([total_us / 1e3 / max(len(batches), 1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out = {"total": round(float(t.item()), 4),
               "how": "device time of the NCCL send/receive kernels of all_to_all_single per step (torch profiler, %d extra steps, max "
                      "over ranks)" % len(batches)}
        if err:
            out["error"] = err
        return out

    def comm_mode(self):
        return "torch.distributed all_to_all_single (NCCL)"
