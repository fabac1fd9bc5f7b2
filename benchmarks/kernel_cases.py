"""Per-kernel cases: every hot kernel on one mid-size input, timed with CUDA events and set against the measured peaks.

Each case runs the kernel ``--warmup`` times, then ``--iters`` times between two events (inputs are larger than the 126 MB L2 or
an L2-sized buffer is rewritten between iterations), and reports the achieved algorithmic GB/s or TFLOP/s as a fraction of the
copy bandwidth / bf16 GEMM rate in ``MEASURED_PEAKS.json`` (HBM 6550.7 GB/s, bf16 1657.8 TFLOP/s when the file is absent).
The same script with ``--once`` runs every kernel exactly once after one warm-up, which is the shape an ``ncu`` capture wants:

    python benchmarks/kernel_cases.py --once
    ncu --set full --clock-control none -k regex:<kernel> -c 2 -o <out> python benchmarks/kernel_cases.py --once [--only <case>]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    hbm, tf = 6550.7, 1657.8
    try:
        d = json.load(open(p))
        hbm = float(d.get("hbm_gbs", hbm))
        tf = float(d.get("bf16_tflops", tf))
    except Exception:
        pass
    return hbm, tf


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--once", action="store_true")
    ap.add_argument("--only", default=None, help="comma-separated case names or name prefixes")
    args = ap.parse_args()
    if args.once:
        args.iters, args.warmup = 1, 0
    small = 2 if args.once else 1        # a profiler capture keeps device memory small: it is saved and restored around every pass

    import torch
    import recis_b200
    from recis_b200.nn.functional import fused_ops, hash_ops
    C = recis_b200.native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    hbm, tf = peaks()
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)
    results = []

    def run(name, fn, bytes_=0.0, flops=0.0, flush_l2=False):
        if args.only and not any(name == o or name.startswith(o) for o in args.only.split(",")):
            return
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(args.iters):
            if flush_l2:
                flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        ms = total / args.iters
        r = {"case": name, "ms": round(ms, 4)}
        if bytes_:
            r["GBps"] = round(bytes_ / ms / 1e6, 1)
            r["frac_of_measured_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops:
            r["TFLOPs"] = round(flops / ms / 1e9, 1)
            r["frac_of_measured_bf16"] = round(flops / ms / 1e9 / tf, 3)
        results.append(r)
        print(json.dumps(r), flush=True)

    # ---- table: lookup-or-insert of 2 M ids into a 16 M-row, width-128 store (half of them new)
    store = C.EmbeddingStore(128, 16_000_000 // (4 * small - 3), "cuda:0", 2, 0.0, 0.01, -2.0, 2.0, 1, False, False, None)
    n_ids = 2_000_000 // small
    ids_a = torch.randint(0, 1 << 40, (n_ids,), device=dev)
    store.lookup_or_insert(ids_a, None, None, 0)
    fresh = [torch.cat([ids_a[:n_ids // 2], torch.randint(0, 1 << 40, (n_ids // 2,), device=dev) + k])
             for k in range(args.warmup + args.iters + 1)]
    state = {"k": 0}

    def lookup():
        state["k"] += 1
        return store.lookup_or_insert(fresh[state["k"] % len(fresh)], None, None, 0)
    run("table_lookup_or_insert_2M", lookup, bytes_=n_ids // 2 * 512 + n_ids * 28)

    # ---- dedup + owner bucketing of 4 M ids (Zipf-like duplicates), 8 owners
    raw = (torch.rand(4_000_000, device=dev, dtype=torch.float64) ** 6 * (1 << 34)).to(torch.int64)
    run("dedup_partition_4M", lambda: C.dedup_partition(raw, 8), bytes_=4_000_000 * (8 + 4 + 4) + 2_000_000 * 8, flush_l2=True)

    # ---- pooling: 2 M unique rows (1 GB), 4.2 M (bag, id) pairs, 213 K bags, width 128
    n_u, n_seg = 2_000_000 // small, 212_992 // small
    uemb = torch.randn(n_u, 128, device=dev)
    lens = torch.poisson(torch.full((n_seg,), 20.0, device=dev)).clamp_(1, 100).to(torch.int32)
    offs = torch.zeros(n_seg + 1, dtype=torch.int32, device=dev)
    offs[1:] = lens.cumsum(0)
    nnz = int(offs[-1])
    rev = torch.randint(0, n_u, (nnz,), dtype=torch.int32, device=dev)
    run("pool_forward_sum_d128", lambda: C.pool_forward(uemb, None, rev, offs, None, 0, 0, 0, True),
        bytes_=nnz * 512 + n_seg * 512 + nnz * 12)

    # ---- backward: CSR build + segmented reduce fused with sparse Adam on the same shape
    w = torch.randn(n_u, 128, device=dev) * 0.01
    m1, m2 = torch.zeros_like(w), torch.zeros_like(w)
    gout = torch.randn(n_seg, 128, device=dev) * 1e-3
    _o, gsrc, gscale = C.pool_forward(uemb, None, rev, offs, None, 0, 0, 0, True)
    rows_id = torch.arange(n_u, dtype=torch.int32, device=dev)
    csr = C.build_csr(rev)
    run("build_csr_4M", lambda: C.build_csr(rev), bytes_=nnz * 4 * 6)
    touched = int(torch.unique(rev).numel())
    run("grad_reduce_adam_d128", lambda: C.grad_reduce(gout, gsrc, gscale, csr[0], csr[1], csr[2], 128, rows_id, True, 0, 1e-3, 0.9, 0.999,
                                                       1e-8, 1.0, -1e-3, 1.0, w, m1, m2, 0),
        bytes_=touched * 512 * 6 + nnz * 512)
    # ---- the same pooling and update on bf16 rows (half the row bytes; state and accumulation stay fp32)
    uemb_h = uemb.to(torch.bfloat16)
    run("pool_forward_sum_d128_bf16rows", lambda: C.pool_forward(uemb_h, None, rev, offs, None, 0, 0, 0, True),
        bytes_=nnz * 256 + n_seg * 512 + nnz * 12)
    w_h = w.to(torch.bfloat16)
    run("grad_reduce_adam_d128_bf16rows", lambda: C.grad_reduce(gout, gsrc, gscale, csr[0], csr[1], csr[2], 128, rows_id, True, 0, 1e-3, 0.9,
                                                                0.999, 1e-8, 1.0, -1e-3, 1.0, w_h, m1, m2, 0),
        bytes_=touched * (256 * 2 + 512 * 4) + nnz * 512)
    del uemb, w, m1, m2, uemb_h, w_h

    # ---- sequence truncation of 256 ragged features at once (three launches, one host read): 8192 rows each, keep 20 of ~50
    from recis_b200.nn.functional import ragged_ops
    n_feat, rows_c = 256 // small, 8192
    lens_c = torch.randint(0, 100, (n_feat, rows_c), device=dev)
    offs_c = torch.zeros(n_feat, rows_c + 1, dtype=torch.int32, device=dev)
    offs_c[:, 1:] = lens_c.cumsum(1)
    vals_c = [torch.randint(0, 1 << 40, (int(offs_c[f, -1]),), device=dev) for f in range(n_feat)]
    offl_c = [offs_c[f].contiguous() for f in range(n_feat)]
    keep_c = torch.full((n_feat,), 20, dtype=torch.int32)
    kept = int(lens_c.clamp(max=20).sum())
    run("fused_cutoff_2d_%dx8192_keep20" % n_feat, lambda: ragged_ops.fused_ragged_cutoff_2D(vals_c, offl_c, keep_c),
        bytes_=kept * 16 + n_feat * rows_c * 44, flush_l2=True)
    del vals_c, offl_c, offs_c, lens_c

    # ---- feature ops: 32 features x 1 M values each, one fused launch per op type
    vals = [torch.randint(0, 1 << 48, (1_000_000,), device=dev) for _ in range(32)]
    run("fused_uint64_mod_32x1M", lambda: fused_ops.fused_uint64_mod_gpu(vals, [1000003] * 32), bytes_=32 * 1_000_000 * 16, flush_l2=True)
    fl = [torch.randn(1_000_000, device=dev) for _ in range(32)]
    bounds = [torch.linspace(-3, 3, 200, device=dev) for _ in range(32)]
    run("fused_bucketize_32x1M_200b", lambda: fused_ops.fused_bucketize_gpu(fl, bounds), bytes_=32 * 1_000_000 * 12, flush_l2=True)
    chars = [v.view(torch.int8) for v in vals]
    splits = [torch.arange(0, 8_000_001, 8, dtype=torch.int32, device=dev) for _ in range(32)]
    run("fused_farmhash_32x1M_8B", lambda: hash_ops.farmhash(chars, splits), bytes_=32 * 1_000_000 * 20, flush_l2=True)
    del vals, fl, chars, splits

    # ---- interactions
    B = 8192
    cube = torch.randn(B, 26, 128, device=dev)
    x = torch.randn(B, 128, device=dev).to(torch.bfloat16)
    cols = (128 + 27 * 26 // 2 + 7) // 8 * 8
    run("dot_interaction_fwd_b8192_f27_d128", lambda: C.dot_interaction_fwd(x, cube, cols), bytes_=B * 26 * 512 + B * cols * 2,
        flush_l2=True)
    dz = torch.randn(B, cols, device=dev).to(torch.bfloat16)
    run("dot_interaction_bwd_b8192_f27_d128", lambda: C.dot_interaction_bwd(x, cube, dz), bytes_=2 * B * 26 * 512 + B * cols * 2 + B * 768,
        flush_l2=True)
    cube_fm = torch.randn(65536, 39, 16, device=dev)
    run("fm_fwd_b65536_f39_d16", lambda: C.fm_fwd(cube_fm), bytes_=65536 * 39 * 64, flush_l2=True)
    gfm = torch.randn(65536, 1, device=dev)
    run("fm_bwd_b65536_f39_d16", lambda: C.fm_bwd(cube_fm, gfm), bytes_=2 * 65536 * 39 * 64, flush_l2=True)

    # ---- tcgen05 GEMMs of the dense tower (bf16 in, fp32 accumulate)
    def gemm_case(name, M, N, K):
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        b = torch.randn(N, K, device=dev).to(torch.bfloat16)
        bias = torch.zeros(N, device=dev)
        run(name, lambda: C.gemm_bf16(a, b, bias, True, False, False, False, None), bytes_=(M * K + N * K + M * N) * 2, flops=2.0 * M * N * K)
    gemm_case("gemm_tcgen05_8192x1024x512", 8192, 1024, 512)
    gemm_case("gemm_tcgen05_8192x1024x1024", 8192, 1024, 1024)
    gemm_case("gemm_tcgen05_16384x2048x4096", 16384, 2048, 4096)
    gemm_case("gemm_tcgen05_8192x8192x8192", 8192, 8192, 8192)

    # ---- the library GEMM on the same shapes (what the reference's nn.Linear runs): the bar for the kernel above
    def lib_case(name, M, N, K):
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        b = torch.randn(N, K, device=dev).to(torch.bfloat16)
        run(name, lambda: torch.matmul(a, b.t()), bytes_=(M * K + N * K + M * N) * 2, flops=2.0 * M * N * K)
    lib_case("library_matmul_8192x1024x512", 8192, 1024, 512)
    lib_case("library_matmul_8192x1024x1024", 8192, 1024, 1024)
    lib_case("library_matmul_8192x8192x8192", 8192, 8192, 8192)

    # ---- ragged self-attention, head width 64: 512 sequences of 50..1000 tokens, 4 heads (config 4's encoder shape), forward and
    # backward, and the padded library path on the same data
    import torch.nn.functional as F
    g = torch.Generator(device="cpu").manual_seed(0)
    n_seq = 512 // (4 * small - 3)
    lens_a = torch.randint(50, 1001, (n_seq,), generator=g)
    offs_a = torch.zeros(n_seq + 1, dtype=torch.int32)
    offs_a[1:] = lens_a.cumsum(0)
    T_a, H_a, Lmax = int(offs_a[-1]), 4, int(lens_a.max())
    qkv = (torch.randn(T_a, 3 * H_a * 64, device=dev) * 0.5).to(torch.bfloat16)
    offs_ad = offs_a.to(dev)
    att_flops = 4.0 * 64 * H_a * float((lens_a.double() ** 2).sum())
    run("ragged_attention_fwd_512seq_h4", lambda: C.ragged_attention_fwd(qkv, offs_ad, H_a, Lmax, 0.125), flops=att_flops,
        bytes_=T_a * H_a * 64 * 2 * 4)
    out_a, lse_a = C.ragged_attention_fwd(qkv, offs_ad, H_a, Lmax, 0.125)
    d_out = torch.randn_like(out_a)
    run("ragged_attention_bwd_512seq_h4", lambda: C.ragged_attention_bwd(qkv, out_a, d_out, lse_a, offs_ad, H_a, Lmax, 0.125),
        flops=2.5 * att_flops, bytes_=T_a * H_a * 64 * (2 * 5 + 4 * 3))
    seg = torch.repeat_interleave(torch.arange(n_seq), lens_a.long()).to(dev)
    pos = (torch.arange(T_a) - offs_a[:-1].long()[seg.cpu()]).to(dev)
    key_ok = (torch.arange(Lmax, device=dev)[None, :] < lens_a.to(dev)[:, None])[:, None, None, :]

    def padded_sdpa():
        padded = qkv.new_zeros(n_seq, Lmax, 3 * H_a * 64)
        padded[seg, pos] = qkv
        q, k, v = padded.view(n_seq, Lmax, 3, H_a, 64).permute(2, 0, 3, 1, 4)
        return F.scaled_dot_product_attention(q, k, v, attn_mask=key_ok).permute(0, 2, 1, 3).reshape(n_seq, Lmax, H_a * 64)[seg, pos]
    run("padded_library_sdpa_fwd_512seq_h4", padded_sdpa, flops=att_flops)
    del qkv, out_a, lse_a, d_out

    # ---- dense Adam over 24 tensors of 1 M floats
    ws = [torch.randn(1_000_000, device=dev) for _ in range(24)]
    gs = [torch.randn_like(t) for t in ws]
    ms_ = [torch.zeros_like(t) for t in ws]
    vs = [torch.zeros_like(t) for t in ws]
    run("dense_adam_24x1M", lambda: C.dense_adam(ws, gs, ms_, vs, [], 0.9, 0.999, 1e-8, 1.0, 1e-3, 1.0, 0.0), bytes_=24 * 1_000_000 * 28,
        flush_l2=True)
    if not args.once:
        print(json.dumps({"summary": results, "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf}}), flush=True)


if __name__ == "__main__":
    main()
