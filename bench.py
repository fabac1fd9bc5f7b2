"""Headline benchmark: training throughput (samples/s) of the DLRM-style CTR configuration.

Configuration (per GPU; weak scaling, 8 GPUs give the global batch of 65536):
  batch 8192, 13 dense fp32 lognormal features, 26 multi-hot fields with Poisson(20) bag lengths clipped to [1, 100],
  ids ~ Zipf(1.05) over a 2^40 id space folded onto 1e8 distinct ids, all fields merged into one dim-128 fp32 dynamic
  table (sum pooling), bottom MLP 512-256-128, dot interaction, top MLP 1024-1024-512-256-1 in bf16, labels
  Bernoulli(0.03), sparse Adam on the embeddings, Adam on the dense tower. Synthetic data, random-init weights.

  python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run, one rank per GPU)
  python bench.py --impl reference ...                      (the unmodified reference installed under baseline/_ref)

Prints one JSON line on rank 0. ``value`` is timed on the device (CUDA events, max over ranks) with the step's inputs
already resident on the GPU; ``e2e.value`` repeats the measurement with, in every step, the host-to-device copy of that
step's inputs from pinned memory and a device-to-host read of the loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PER_GPU_BATCH = 8192
N_FIELDS = 26
EMB_DIM = 128
UNIVERSE = 100_000_000          # distinct ids over all fields ("about 1e8 unique rows total")
ID_BITS = 40


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=30)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--batch-per-gpu", type=int, default=PER_GPU_BATCH)
    p.add_argument("--capacity", type=int, default=0, help="rows per GPU to pre-size the table for")
    p.add_argument("--comm", default=None, help="override RECIS_COMM (fused | nccl)")
    p.add_argument("--regions", type=int, default=3, help="timed regions of --steps steps each, per measurement (median is reported)")
    return p.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) every ~10 ms while the timed region runs."""

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.samples = []
        self.reasons = set()
        self._stop = False
        self._thread = None
        self.max_mhz = None

    def _loop(self):
        import pynvml as nv
        bits = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, b in bits.items():
                    if r & b:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.gpu_index
            if visible:
                try:
                    idx = int(visible.split(",")[self.gpu_index])
                except ValueError:
                    idx = self.gpu_index
            self.h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None

    def stop(self) -> dict:
        if self._thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self._stop = True
        self._thread.join(timeout=2)
        sm = sorted(self.samples)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(sm)}


def dist_setup(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def sync_all(world):
    import torch
    import torch.distributed as dist
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()


def max_over_ranks(x: float, world) -> float:
    import torch
    import torch.distributed as dist
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class no_cycle_collection:
    """The interpreter's cycle collector stays out of a timed region (both arms): with hundreds of pre-built batches alive a
    full collection takes tens of milliseconds and lands in whichever region happens to trigger it. Reference counting frees
    everything a step allocates; cycles are collected between regions."""

    def __enter__(self):
        import gc
        gc.collect()
        gc.disable()

    def __exit__(self, *exc):
        import gc
        gc.enable()


def timed(step_fn, first, count, world):
    """Run ``count`` steps starting at batch index ``first``; returns elapsed ms (device time, max over ranks)."""
    import torch
    with no_cycle_collection():
        sync_all(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(count):
            step_fn(first + i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    sync_all(world)
    return max_over_ranks(ms, world)


def spec_for(args, rank):
    from recis_b200.io.synthetic import SparseFieldSpec, SyntheticSpec
    fields = [f"c{i}" for i in range(N_FIELDS)]
    sparse = [SparseFieldSpec(f, zipf_a=1.05, id_bits=ID_BITS, universe=UNIVERSE // N_FIELDS, length="poisson", mean_len=20, min_len=1,
                              max_len=100) for f in fields]
    return fields, SyntheticSpec(batch=args.batch_per_gpu, dense_dim=13, sparse=sparse, label_rate=0.03, seed=1000 + rank)


def run(args, arm):
    import torch
    world, rank, local = dist_setup(args)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    dev = torch.device("cuda", local)
    fields, spec = spec_for(args, rank)
    R, K, W = max(args.regions, 1), args.steps, args.warmup
    e2e_warm = min(3, W)
    # Every step of the run, timed or not, consumes a batch that no earlier step has seen: W warm-up steps, a short warm-up of the
    # end-to-end path, then R regions of K steps for each of the two measurements, interleaved (A1 E1 A2 E2 ...) so that the
    # device-resident number and the end-to-end number see the same mix of known and new ids.
    n_batches = W + e2e_warm + 2 * R * K
    # rows per GPU: what the run can touch (with a few GPUs the run ends long before the 1e8-row universe is covered) plus head-room
    # for the rows the allocator sets aside for calls still in flight
    # (one GPU: the whole 1e8-id universe plus the rows set aside for the calls in flight, 167 GB of rows and optimizer state; the
    # table never has to grow inside a timed region however long the run is)
    capacity = args.capacity or min(int(1.15 * UNIVERSE / world) + 8_000_000, 108_000_000)
    state = arm.build(fields, dev, world, rank, capacity)

    from recis_b200.io.synthetic import make_batch_arrays
    host = [arm.wrap_host(make_batch_arrays(spec, i), spec.batch) for i in range(n_batches)]
    h2d_bytes = arm.nbytes(host[0])
    losses = []

    def region_resident(first, count):
        """Device-resident inputs: the kernel-path number."""
        dev_batches = [arm.to_device(b, dev) for b in host[first:first + count]]
        sync_all(world)
        return timed(lambda i: arm.step(state, dev_batches[i]), 0, count, world)

    def region_e2e(first, count):
        """End to end: every step's inputs are copied host -> device from pinned memory inside the timed region (the arm's feeder
        may run those copies on a side stream ahead of use, as a data loader does) and the step's loss is read back."""
        with no_cycle_collection():
            sync_all(world)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            feeder = arm.feeder(host[first:first + count], dev)       # created inside the region: all `count` copies are timed
            for batch in feeder:
                loss = arm.step_e2e(state, batch) if hasattr(arm, "step_e2e") else arm.step(state, batch)
                if hasattr(feeder, "prefetch"):
                    feeder.prefetch()            # next batches' copies are issued while the GPU works on this step
                # device -> host read of the step's result, every step
                losses.append(arm.read_loss(state, loss) if hasattr(arm, "read_loss") else float(loss))
            e1.record()
            torch.cuda.synchronize()
            ms_ = e0.elapsed_time(e1)
        sync_all(world)
        return max_over_ranks(ms_, world)

    rows_seen = [arm.table_rows(state, world)]

    def new_rows(count):
        rows_seen.append(arm.table_rows(state, world))
        a, b = rows_seen[-2], rows_seen[-1]
        return None if a is None or b is None else (b - a) / count

    pos = 0
    region_resident(pos, W); pos += W
    new_rows(W)
    region_e2e(pos, e2e_warm); pos += e2e_warm
    new_rows(max(e2e_warm, 1))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_a, ms_e, new_a, new_e, launches = [], [], [], [], []
    for _ in range(R):
        l0 = arm.launches()
        ms_a.append(region_resident(pos, K)); pos += K
        launches.append(arm.launches() - l0)
        new_a.append(new_rows(K))
        ms_e.append(region_e2e(pos, K)); pos += K
        new_e.append(new_rows(K))
    clocks = sampler.stop() if rank == 0 else None

    def median_of(xs):
        order = sorted(range(len(xs)), key=lambda i: xs[i])
        return order[len(xs) // 2]

    ia, ie = median_of(ms_a), median_of(ms_e)
    ms, ms_e2e = ms_a[ia], ms_e[ie]

    # ---- exposed communication: a few extra steps after the timed regions
    exposed = arm.exposed_comm_ms(state, host, dev, world, min(5, K)) if hasattr(arm, "exposed_comm_ms") else None
    status_bits = arm.exchange_status(state) if hasattr(arm, "exchange_status") else None

    global_batch = spec.batch * world
    value = global_batch * K / (ms / 1e3)
    value_e2e = global_batch * K / (ms_e2e / 1e3)
    if rank == 0:
        per_step = lambda xs: [round(x / K, 4) for x in xs]
        line = {
            "metric": "train samples/s (DLRM-style CTR, device-timed, max over ranks)",
            "value": value, "unit": "samples/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded), random-init weights; every step sees a fresh batch",
            "impl": arm.name,
            "config": {
                "model": "dlrm_ctr: 13 dense + 26 multi-hot fields (Poisson(20) in [1,100]) -> one merged dim-128 dynamic table, "
                         "sum pooling, bottom MLP 512-256-128, dot interaction, top MLP 1024-1024-512-256-1, sparse Adam + Adam",
                "global_batch": global_batch, "per_gpu_batch": spec.batch, "seq_len": None,
                "ids": "Zipf(1.05) over a 2^40 id space, 1e8 distinct ids in total over the 26 fields", "parallelism": f"dp{world} dense + row-sharded embeddings",
                "l2": "no explicit flush: each step touches > 1 GB of embedding rows and optimizer state, far beyond the 126 MB L2",
                "precision": "bf16 dense tower (fp32 accumulation, fp32 master weights); fp32 embedding table, optimizer state and exchange",
                "regions": f"{R} timed regions of {K} steps per measurement, device-resident and end-to-end regions interleaved; "
                           "the median region is reported; the interpreter's cycle collector runs between regions, not inside them",
            },
            "comm": arm.comm_mode(),
            "clocks": clocks,
            "regions": {"ms_per_step": per_step(ms_a), "spread": round((max(ms_a) - min(ms_a)) / ms, 4),
                        "new_rows_per_step": new_a, "reported": ia},
            "e2e": {"value": value_e2e, "unit": "samples/s", "ms_per_step": ms_e2e / K, "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": 4, "last_loss": losses[-1] if losses else None,
                    "loss_read": arm.LOSS_READ,
                    "regions": {"ms_per_step": per_step(ms_e), "spread": round((max(ms_e) - min(ms_e)) / ms_e2e, 4),
                                "new_rows_per_step": new_e, "reported": ie}},
            "gpu_launches": launches[ia],
        }
        if exposed is not None:
            line["exposed_all_to_all_ms"] = exposed
        if status_bits is not None:
            # largest status word over the ranks; 0 = every bounded wait was answered and no exchange window overflowed during the
            # whole run (bit 4: a wait ran out, bit 8: a window overflowed; either would invalidate the numbers above)
            line["exchange_status"] = status_bits
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


# ====================================================================== our arm
class OursArm:
    name = "ours"

    def build(self, fields, dev, world, rank, capacity):
        import torch
        from recis_b200.models.dlrm import DLRM
        from recis_b200.nn import filter_out_sparse_param
        from recis_b200.optim import SparseAdam
        from recis_b200.parallel.dense_reducer import DenseGradReducer
        torch.manual_seed(1234)
        model = DLRM(fields, dense_dim=13, emb_dim=EMB_DIM, device=dev, capacity=capacity).to(dev)
        sparse_opt = SparseAdam(filter_out_sparse_param(model), lr=1e-3)
        dense_params = [p for p in model.parameters() if p.requires_grad]
        from recis_b200.optim import DenseAdam
        dense_opt = DenseAdam(dense_params, lr=1e-3)
        reducer = DenseGradReducer(dense_params, world) if world > 1 else None
        from recis_b200.utils import AsyncScalarReader
        return dict(model=model, sparse_opt=sparse_opt, dense_opt=dense_opt, reducer=reducer, loss_reader=AsyncScalarReader(dev))

    def wrap_host(self, arrays, batch):
        """The batch as the framework's packed host batch: every tensor of it inside one pinned buffer (``recis_b200.io.PackedBatch``)."""
        import numpy as np
        import torch
        from recis_b200.io import PackedBatch
        from recis_b200.ragged import RaggedTensor
        out = {}
        for k, v in arrays.items():
            if isinstance(v, tuple):
                out[k] = RaggedTensor(torch.from_numpy(v[0]), [torch.from_numpy(v[1])], dense_shape=(batch, -1))
            else:
                out[k] = torch.from_numpy(np.ascontiguousarray(v))
        return PackedBatch(out, pin=True)

    def nbytes(self, b):
        return b.payload_bytes          # bytes of the batch's tensors (the buffer adds up to 255 bytes of padding per tensor)

    def to_device(self, b, dev):
        return b.to(dev, non_blocking=True)

    def feeder(self, host_batches, dev):
        from recis_b200.io import DevicePrefetcher
        return DevicePrefetcher(host_batches, dev, depth=2)

    LOSS_READ = ("every step: the loss is copied to pinned host memory on a side stream as soon as the forward pass has produced "
                 "it, and the host reads that step's value at the end of the step")

    def step_e2e(self, st, batch):
        """The same step; the loss starts its way to the host as soon as the forward pass has produced it."""
        return self.step(st, batch, post_loss=True)

    def read_loss(self, st, ticket):
        return st["loss_reader"].get(ticket)

    def step(self, st, batch, post_loss=False):
        loss, _ = st["model"](batch)
        if post_loss:
            ticket = st["loss_reader"].post(loss)
        st["dense_opt"].zero_grad(set_to_none=False) if st["reducer"] is not None else st["dense_opt"].zero_grad()
        st["sparse_opt"].zero_grad()
        loss.backward()
        if st["reducer"] is not None:
            st["reducer"].all_reduce_async()      # side stream: overlaps with the embedding update below
        st["sparse_opt"].step()
        if st["reducer"] is not None:
            st["reducer"].wait()
        st["dense_opt"].step()
        return ticket if post_loss else loss.detach()

    def launches(self):
        import recis_b200
        return int(recis_b200.native().launch_count())

    def table_rows(self, st, world):
        """Rows in the table over all ranks (device counters; read between regions, outside all timing)."""
        import torch
        import torch.distributed as dist
        n = sum(int(t.impl.size()) for t in st["model"].embedding_engine.tables().values())
        if world > 1:
            t = torch.tensor([n], dtype=torch.int64, device="cuda")
            dist.all_reduce(t)
            n = int(t.item())
        return n

    SPAN_LABELS = ("ids", "emb", "grad_push", "grad_wait", "dense_allreduce_wait", "total")

    def exposed_comm_ms(self, st, host_batches, dev, world, steps):
        """Milliseconds per step that the model's stream spends in the exchange phases (transfer kernels + waiting for peers)
        and blocked on the dense all-reduce: CUDA events on the launching stream, max over ranks, measured on ``steps`` extra
        steps after the timed regions. Every rank always runs the same steps and the same reduction, whatever happens to
        the accounting itself."""
        import torch
        import torch.distributed as dist
        if world == 1:
            return {"total": 0.0, "note": "single GPU: no exchange"}
        from recis_b200.parallel.spans import recorder
        batches = [self.to_device(b, dev) for b in host_batches[-steps:]]
        sync_all(world)
        err = None
        exchanges = [t.fused for t in st["model"].embedding_engine.tables().values() if getattr(t, "fused", None) is not None]
        try:
            recorder.start()
            for ex in exchanges:            # flag waits of these extra steps go through the accounting kernel
                ex.wait_stats = torch.zeros(8 * world + 8, dtype=torch.int64, device=dev)
                # the phases are bracketed where Python issues them: these steps use the Python executor of the same protocol
                ex._native_before = ex.native_executor
                ex.native_executor = False
        except Exception as e:          # accounting must never take the benchmark down
            err = repr(e)
        for b in batches:
            self.step(st, b)
        for ex in exchanges:
            if hasattr(ex, "_native_before"):
                ex.native_executor = ex._native_before
        vals = [-1.0] * len(self.SPAN_LABELS)
        try:
            res = recorder.stop(steps=len(batches))
            vals = [float(res.get(k, 0.0)) for k in self.SPAN_LABELS]
        except Exception as e:
            err = repr(e)
            torch.cuda.synchronize()
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sync_all(world)
        out = dict(zip(self.SPAN_LABELS, [round(v, 4) for v in t.tolist()]))
        out["how"] = ("spans: CUDA events around the exchange phases (transfer kernels included) on the model's stream; "
                      "flag_wait_ms_per_step: time the flag-wait kernels really spent waiting for the last peer (device timer), "
                      "summed over the waits of a step; both max over ranks, %d extra steps" % len(batches))
        try:
            waited = 0.0
            for ex in exchanges:
                sums = ex.wait_stats.cpu()
                ex.wait_stats = None
                waited += sum(float(sums[ch * world:(ch + 1) * world].max()) for ch in range(3)) / 1e6 / max(len(batches), 1)
            tw = torch.tensor([waited], dtype=torch.float64, device=dev)
            dist.all_reduce(tw, op=dist.ReduceOp.MAX)
            out["flag_wait_ms_per_step"] = round(float(tw.item()), 4)
        except Exception as e:
            err = repr(e)
        if err:
            out["error"] = err
        return out

    def exchange_status(self, st):
        """OR of the status words of the fused exchanges and the dense all-reduce (one small device read each, after all timing)."""
        bits = 0
        try:
            for table in st["model"].embedding_engine.tables().values():
                ex = getattr(table, "fused", None)
                if ex is not None:
                    bits |= int(ex.status.item())
            if st["reducer"] is not None and getattr(st["reducer"], "p2p", False):
                bits |= int(st["reducer"].status.item())
        except Exception:                # the status read must never take the benchmark line down
            bits = -1
        import torch
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():      # every rank calls this: the largest value over the ranks is reported
            t = torch.tensor([bits if bits >= 0 else 1 << 20], dtype=torch.int64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            bits = int(t.item())
        return bits

    def comm_mode(self):
        return os.environ.get("RECIS_COMM", "auto")


def main():
    args = parse()
    if args.comm:
        os.environ["RECIS_COMM"] = args.comm
    if args.impl == "reference":
        from baseline.reference_arm import ReferenceArm, unavailable_reason
        why = unavailable_reason()
        if why:
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
            return
        run(args, ReferenceArm())
    else:
        run(args, OursArm())


if __name__ == "__main__":
    main()
