"""Where the end-to-end step of ``bench.py`` differs from the device-resident one (one GPU).

    python benchmarks/e2e_vs_resident.py

Builds the arm and the batches of ``bench.py``, then runs twelve device-resident steps and twelve end-to-end steps (inputs copied
from pinned host memory by the prefetcher, loss read every step) under ``torch.profiler`` and prints, for each: kernel time per
step summed over streams, busy and idle time of the GPU, the idle gaps above 40 microseconds with the kernels around them, and
the kernels whose time differs most between the two; finally the host-side phases of an end-to-end step without the profiler.
Numbers printed under the profiler are for comparison between the two loops only.
"""
import collections
import os
import sys
import time
import types

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from torch.profiler import ProfilerActivity, profile

import bench
from recis_b200.io.synthetic import make_batch_arrays

STEPS = 12            # profiled steps per loop
GAP_US = 40           # idle intervals of the whole GPU above this are listed


def summarize(tag, prof, steps):
    """Prints the totals and the largest gaps of one profiled loop; returns (kernel time per step, launches per step) by name."""
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    time_by, count_by = collections.defaultdict(float), collections.Counter()
    for e in evs:
        time_by[e.name[:70]] += e.device_time_total if hasattr(e, "device_time_total") else e.cuda_time_total
        count_by[e.name[:70]] += 1
    total = sum(time_by.values())
    # busy time: union of the kernels' intervals over all streams; span: first start to last end
    iv = sorted((e.time_range.start, e.time_range.end) for e in evs)
    busy, (cur_s, cur_e) = 0, iv[0]
    for s, e in iv[1:]:
        if s > cur_e:
            busy += cur_e - cur_s
            cur_s, cur_e = s, e
        else:
            cur_e = max(cur_e, e)
    busy += cur_e - cur_s
    span = iv[-1][1] - iv[0][0]
    gaps, gap_time = collections.Counter(), collections.defaultdict(float)
    ordered = sorted(evs, key=lambda e: e.time_range.start)
    end_so_far, last_name = ordered[0].time_range.end, ordered[0].name
    for e in ordered[1:]:
        if e.time_range.start - end_so_far > GAP_US:
            key = (last_name[:48], e.name[:48])
            gaps[key] += 1
            gap_time[key] += e.time_range.start - end_so_far
        if e.time_range.end > end_so_far:
            end_so_far, last_name = e.time_range.end, e.name
    for k, v in sorted(gap_time.items(), key=lambda kv: -kv[1])[:8]:
        print(f"   gap total {v / steps:7.1f} us/step  x{gaps[k] / steps:.2f}/step  after [{k[0]}]  before [{k[1]}]")
    print(f"[{tag}] kernels sum {total / steps:.1f} us/step, union busy {busy / steps:.1f} us/step, span {span / steps:.1f} us/step, "
          f"idle {(span - busy) / steps:.1f} us/step")
    return {k: v / steps for k, v in time_by.items()}, {k: c / steps for k, c in count_by.items()}


def main():
    args = types.SimpleNamespace(batch_per_gpu=8192, gpus=1)
    bench.dist_setup(args)
    arm = bench.OursArm()
    dev = torch.device("cuda", 0)
    fields, spec = bench.spec_for(args, 0)
    st = arm.build(fields, dev, 1, 0, 100_000_000)           # large enough that the table does not grow during the run
    host = [arm.wrap_host(make_batch_arrays(spec, i), spec.batch) for i in range(64)]

    def resident(lo, hi):
        dev_batches = [arm.to_device(b, dev) for b in host[lo:hi]]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for b in dev_batches:
            arm.step(st, b)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (hi - lo)

    def e2e(lo, hi):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        feeder = arm.feeder(host[lo:hi], dev)
        for batch in feeder:
            ticket = arm.step_e2e(st, batch)
            feeder.prefetch()
            arm.read_loss(st, ticket)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (hi - lo)

    print("warm resident", resident(0, 16))
    print("warm e2e", e2e(16, 24))
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as p1:
        ms_res = resident(24, 24 + STEPS)
    t_res, n_res = summarize("resident", p1, STEPS)
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as p2:
        ms_e2e = e2e(24 + STEPS, 24 + 2 * STEPS)
    t_e2e, n_e2e = summarize("e2e", p2, STEPS)
    print("under profiler: resident", ms_res, "e2e", ms_e2e)
    for k in sorted(set(t_res) | set(t_e2e), key=lambda k: -abs(t_e2e.get(k, 0) - t_res.get(k, 0)))[:18]:
        print(f"{t_e2e.get(k, 0) - t_res.get(k, 0):+8.1f} us  res {t_res.get(k, 0):8.1f} ({n_res.get(k, 0):.1f})  "
              f"e2e {t_e2e.get(k, 0):8.1f} ({n_e2e.get(k, 0):.1f})  {k}")
    print("plain again: resident", resident(48, 56), "e2e", e2e(56, 64))

    # host phases of the end-to-end loop, without the profiler
    phases = collections.defaultdict(float)
    more = [arm.wrap_host(make_batch_arrays(spec, 100 + i), spec.batch) for i in range(20)]
    torch.cuda.synchronize()
    t_all = time.perf_counter()
    feeder = arm.feeder(more, dev)
    it = iter(feeder)
    while True:
        t0 = time.perf_counter()
        try:
            batch = next(it)
        except StopIteration:
            break
        t1 = time.perf_counter()
        ticket = arm.step_e2e(st, batch)
        t2 = time.perf_counter()
        feeder.prefetch()
        t3 = time.perf_counter()
        arm.read_loss(st, ticket)
        t4 = time.perf_counter()
        phases["next"] += t1 - t0
        phases["step issue"] += t2 - t1
        phases["prefetch"] += t3 - t2
        phases["loss wait"] += t4 - t3
    torch.cuda.synchronize()
    print("e2e wall ms/step", (time.perf_counter() - t_all) / 20 * 1e3, {k: round(v / 20 * 1e3, 3) for k, v in phases.items()})


if __name__ == "__main__":
    main()
