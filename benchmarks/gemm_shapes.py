"""The dense tower's GEMMs, ours against the library's, shape by shape.

For every layer of the DLRM towers of the headline benchmark (batch 8192 per GPU; bottom 13-512-256-128, top
480-1024-1024-512-256-1 with the widths padded to multiples of 8 as the model pads them) this times the three GEMMs of a
training step on the tcgen05 kernel and on ``torch.matmul`` (cuBLAS behind ``nn.Linear``, which is what the reference's
dense layers run: ``examples/deepfm/deepfm_model.py:49-52``):

  forward   y[M, N]  = x[M, K] W[N, K]^T + b, ReLU, bf16 out        (library: ``F.linear`` + ``relu``; also timed without them)
  dgrad     dx[M, K] = dy[M, N] W[N, K]                              (W read MN-major by our kernel, no transposed copy)
  wgrad     dW[N, K] = dy[M, N]^T x[M, K], fp32 out, split-K         (both operands MN-major)

CUDA events around each launch, a 160 MB fill between launches so that no operand starts in L2, ``--iters`` launches per
case, median reported; SM clock sampled over the run. One JSON line per case and a markdown table at the end.

    python benchmarks/gemm_shapes.py [--batch 8192] [--iters 20]
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()

    import torch
    import torch.nn.functional as F
    import recis_b200
    C = recis_b200.native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts)

    pad8 = lambda n: (n + 7) // 8 * 8
    towers = [[13, 512, 256, 128], [480, 1024, 1024, 512, 256, 1]]
    layers = [(pad8(t[i]), pad8(t[i + 1])) for t in towers for i in range(len(t) - 1)]
    M = args.batch
    clock = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.active", "--format=csv,noheader,nounits",
                              "-lms", "200"], stdout=subprocess.PIPE, text=True)
    rows = []
    for K, N in layers:
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        b = torch.zeros(N, device=dev)
        bb = b.to(torch.bfloat16)
        dy = torch.randn(M, N, device=dev).to(torch.bfloat16)
        cases = {
            "forward": (lambda: C.gemm_bf16(x, w, b, True, False, False, False, None), lambda: F.relu(F.linear(x, w, bb)),
                        lambda: torch.matmul(x, w.t())),
            "dgrad": (lambda: C.gemm_bf16(dy, w, None, False, False, True, False, None), lambda: torch.matmul(dy, w), None),
            "wgrad": (lambda: C.gemm_bf16(dy, x, None, False, True, True, True, None), lambda: torch.matmul(dy.t(), x).float(),
                      lambda: torch.matmul(dy.t(), x)),
        }
        for kind, (ours, lib, lib_bare) in cases.items():
            r = {"layer": f"{K}->{N}", "gemm": kind, "M": M, "N": N, "K": K, "ours_us": round(timed(ours), 2),
                 "library_us": round(timed(lib), 2)}
            if lib_bare is not None:
                r["library_matmul_only_us"] = round(timed(lib_bare), 2)
            r["ours_over_library"] = round(r["library_us"] / r["ours_us"], 3)          # > 1: ours is faster
            r["TFLOPs_ours"] = round(2.0 * M * N * K / r["ours_us"] / 1e6, 1)
            rows.append(r)
            print(json.dumps(r), flush=True)
    clock.terminate()
    samples = [l.split(", ") for l in clock.stdout.read().strip().splitlines() if l.strip()]
    sm = sorted(int(s[0]) for s in samples if s and s[0].isdigit())
    print(json.dumps({"clocks": {"sm_mhz_median": sm[len(sm) // 2] if sm else None, "sm_max_mhz": int(samples[0][1]) if samples else None,
                                 "reasons": sorted({s[2] for s in samples if len(s) > 2})}}))
    print("\n| layer (K->N) | GEMM | ours us | library us | library matmul only us | library / ours | ours TFLOP/s |\n|---|---|---:|---:|---:|---:|---:|")
    for r in rows:
        print(f"| {r['layer']} | {r['gemm']} | {r['ours_us']} | {r['library_us']} | {r.get('library_matmul_only_us', '')} | "
              f"{r['ours_over_library']} | {r['TFLOPs_ours']} |")


if __name__ == "__main__":
    main()
