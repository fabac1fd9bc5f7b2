"""GPU tests of the paths that are switched off by default (persistent GEMM, ragged attention kernel, exchange lanes, wait
accounting). They run only with RECIS_TEST_OPTIN=1: these kernels have not been validated on hardware yet, so the default GPU
suite does not launch them."""
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(os.environ.get("RECIS_TEST_OPTIN") != "1", reason="opt-in kernels: set RECIS_TEST_OPTIN=1")]


def _child(code: str, env: dict):
    """Run ``code`` in a fresh interpreter (the switches are read once per process)."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=root, env=dict(os.environ, **env))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    return out.stdout


def test_persistent_gemm_matches_fp32_reference():
    code = """
import torch, recis_b200
C = recis_b200.native()
torch.manual_seed(0)
for (M, N, K, relu) in [(8192, 1024, 512, True), (300, 136, 72, False), (128, 128, 64, True), (1000, 520, 1024, False)]:
    a = torch.randn(M, K, device='cuda').to(torch.bfloat16); b = torch.randn(N, K, device='cuda').to(torch.bfloat16)
    bias = torch.randn(N, device='cuda')
    y = C.gemm_bf16(a, b, bias, relu, False, False, False, None).float()
    ref = a.float() @ b.float().t() + bias
    ref = torch.relu(ref) if relu else ref
    err = (y - ref).norm() / ref.norm()
    assert err < 1e-2, (M, N, K, float(err))
    # MN-major operands (the backward GEMMs); their row pitch is M / N, which TMA wants as a multiple of 8 elements
    if M % 8 == 0 and N % 8 == 0:
        at = a.t().contiguous(); bt = b.t().contiguous()
        y2 = C.gemm_bf16(at, bt, None, False, True, True, True, None)
        assert ((y2 - a.float() @ b.float().t()).norm() / (a.float() @ b.float().t()).norm()) < 1e-2
assert C.dense_status('cuda:0') == 0
print('ok')
"""
    assert "ok" in _child(code, {"RECIS_GEMM_PERSISTENT": "1"})


def test_ragged_attention_kernel_matches_padded_path():
    code = """
import torch
from recis_b200.ops.attention import ragged_self_attention
import recis_b200
torch.manual_seed(0)
for lens, H in [([5, 128, 129, 300, 1], 4), ([1000, 50], 2), ([64] * 7, 1)]:
    lens_t = torch.tensor(lens)
    offs = torch.zeros(len(lens) + 1, dtype=torch.int32); offs[1:] = lens_t.cumsum(0)
    T = int(offs[-1])
    qkv = (torch.randn(T, 3 * H * 64, device='cuda') * 0.5).to(torch.bfloat16)
    with torch.no_grad():
        got = ragged_self_attention(qkv, offs.cuda(), H, max(lens)).float()
    import os
    os.environ['RECIS_ATTENTION'] = 'off'
    with torch.no_grad():
        ref = ragged_self_attention(qkv.float(), offs.cuda(), H, max(lens))
    os.environ['RECIS_ATTENTION'] = 'tcgen05'
    err = (got - ref).abs().max()
    assert err < 3e-2, (lens, float(err))
assert recis_b200.native().dense_status('cuda:0') == 0
print('ok')
"""
    assert "ok" in _child(code, {"RECIS_ATTENTION": "tcgen05"})


@pytest.mark.parametrize("env", [{"RECIS_EXCHANGE_LANES": "2"}, {"RECIS_WAIT_STATS": "1"}, {"RECIS_STAGE_EXCHANGE": "1"}])
def test_fused_exchange_variants_match_single_process(env):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import test_multirank as tm
    from multirank import run_ranks
    results = run_ranks(tm._rank_fn, 2, "nccl", args=("cuda",), env=dict(env, RECIS_COMM="fused", NCCL_NVLS_ENABLE="0"))
    tm._compare(results, tm._oracle(2), 2)


def test_ragged_attention_backward_matches_padded_path():
    code = """
import os, torch
from recis_b200.ops.attention import ragged_self_attention
torch.manual_seed(1)
lens = [5, 128, 200, 1]; H = 2
lens_t = torch.tensor(lens)
offs = torch.zeros(len(lens) + 1, dtype=torch.int32); offs[1:] = lens_t.cumsum(0)
T = int(offs[-1])
base = (torch.randn(T, 3 * H * 64, device='cuda') * 0.5).to(torch.bfloat16)
go = (torch.randn(T, H * 64, device='cuda') * 0.1).to(torch.bfloat16)
a = base.clone().requires_grad_(True)
ragged_self_attention(a, offs.cuda(), H, max(lens)).backward(go)
os.environ['RECIS_ATTENTION'] = 'off'
b = base.float().requires_grad_(True)
ragged_self_attention(b, offs.cuda(), H, max(lens)).backward(go.float())
err = (a.grad.float() - b.grad).abs().max() / b.grad.abs().max()
assert err < 5e-2, float(err)
print('ok')
"""
    assert "ok" in _child(code, {"RECIS_ATTENTION": "tcgen05"})


@pytest.mark.parametrize("world,dim", [(2, 16), (4, 128), (8, 64)])
def test_exchange_kernels_loopback_on_one_gpu(world, dim):
    """The peer-memory exchange kernels with ``world`` logical ranks on ONE GPU: every 'peer pointer' is a local buffer and the
    phases run one after the other on one stream (no kernel ever waits for another), so the id pull, the row push, the gradient
    push and the owner-side reduce / update are checked against a dense oracle without a second GPU."""
    import recis_b200
    C = recis_b200.native()
    dev = torch.device("cuda:0")
    torch.manual_seed(world * 100 + dim)
    W, D, S = world, dim, 700
    cap = 8192                                             # window capacity in unique ids per rank
    in_cap = min(W, 2) * cap
    status = torch.zeros(1, dtype=torch.int64, device=dev)
    ids, offs, revs = [], [], []
    ids_win = [torch.zeros(cap, dtype=torch.int64, device=dev) for _ in range(W)]
    off_win = [torch.zeros(W + 1, dtype=torch.int32, device=dev) for _ in range(W)]
    uemb = [torch.zeros(cap, D, device=dev) for _ in range(W)]
    gin = [torch.zeros(in_cap, D, device=dev) for _ in range(W)]
    ptrs = lambda ts: [t.data_ptr() for t in ts]
    # ---- requesters: dedup + bucket by owner into their windows
    for r in range(W):
        lens = torch.randint(0, 9, (S,))
        o = torch.zeros(S + 1, dtype=torch.int32); o[1:] = lens.cumsum(0)
        x = torch.randint(0, 3000, (int(o[-1]),), dtype=torch.int64) * 7919 + (torch.randint(0, 2, (int(o[-1]),)) << 40)
        x[: x.numel() // 5] = 12345                        # an id every rank asks for many times
        ids.append(x.to(dev)); offs.append(o.to(dev))
        _u, rev, _c, _o = C.dedup_partition(ids[r], W, ids_win[r], off_win[r], status)
        revs.append(rev)
    # ---- owners: pull ids, resolve rows, push rows to the requesters
    ids_in, prefix, rows_in, tables, owned = [], [], [], [], []
    for o in range(W):
        buf = torch.zeros(in_cap, dtype=torch.int64, device=dev)
        meta = torch.zeros(3 * W + 1, dtype=torch.int32, device=dev)
        n_in = torch.zeros(1, dtype=torch.int32, device=dev)
        C.comm_pull_ids(ptrs(ids_win), ptrs(off_win), o, buf, meta, n_in, status)
        n = int(n_in.item())
        assert n == int(meta[W].item()) == sum(int(off_win[r][o + 1] - off_win[r][o]) for r in range(W))
        uniq, inv = torch.unique(buf[:n], return_inverse=True)
        rows = torch.full((in_cap,), -1, dtype=torch.int32, device=dev)
        rows[:n] = inv.to(torch.int32)
        table = torch.randn(max(uniq.numel(), 1), D, device=dev)
        ids_in.append(buf); prefix.append(meta); rows_in.append(rows); tables.append(table); owned.append(uniq)
    all_owned = torch.cat(owned)
    assert all_owned.unique().numel() == all_owned.numel()                     # every id has exactly one owner
    for o in range(W):
        C.comm_push_emb(tables[o], rows_in[o], prefix[o], ptrs(uemb), o, in_cap)
    # ---- requesters: pool; oracle = rows looked up by id in the owners' tables
    order = torch.argsort(all_owned)
    keys = all_owned[order]
    flat_rows = torch.cat([tables[o][: owned[o].numel()] for o in range(W)])[order]
    saved = []
    for r in range(W):
        out, gsrc, gscale = C.pool_forward(uemb[r], None, revs[r], offs[r], None, 0, 0, 0, True)
        e = flat_rows[torch.searchsorted(keys, ids[r])]
        seg = torch.repeat_interleave(torch.arange(S, device=dev), (offs[r][1:] - offs[r][:-1]).long())
        ref = torch.zeros(S, D, device=dev).index_add_(0, seg, e)
        assert torch.allclose(out, ref, atol=1e-4, rtol=1e-4), (r, float((out - ref).abs().max()))
        saved.append((gsrc, gscale, seg))
    # ---- backward: requesters push per-unique gradients into the owners' windows
    G = torch.zeros(keys.numel(), D, dtype=torch.float64, device=dev)
    for r in range(W):
        go = torch.randn(S, D, device=dev)
        gsrc, gscale, seg = saved[r]
        csr_u, csr_elem, start = C.build_csr(revs[r])
        C.comm_grad_reduce_push(go, gsrc, gscale, csr_u, csr_elem, start, D, off_win[r], prefix[r], ptrs(gin), in_cap)
        G.index_add_(0, torch.searchsorted(keys, ids[r]), go[seg].double())
    # ---- owners: reduce across requesters (no update), then the fused update on a copy
    for o in range(W):
        head = torch.full((tables[o].size(0),), -1, dtype=torch.int32, device=dev)
        rows, grads = C.comm_owner_reduce(rows_in[o], head, prefix[o], gin[o], W, D, False, False, 2, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0,
                                          None, None, None, in_cap, 2)
        assert int(head.max().item()) == -1                                    # chains are unlinked again
        live = rows >= 0
        assert torch.equal(rows[live].long().sort().values, torch.arange(owned[o].numel(), device=dev))   # each row exactly once
        ref = G[torch.searchsorted(keys, owned[o][rows[live].long()])]
        tol = 1e-5 * float(ref.abs().max()) + 1e-4
        assert torch.allclose(grads[live].double(), ref, atol=tol, rtol=1e-4), (o, float((grads[live].double() - ref).abs().max()))
        w = tables[o].clone()
        C.comm_owner_reduce(rows_in[o], head, prefix[o], gin[o], W, D, False, True, 2, 0.5, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0,
                            w, None, None, in_cap, 2)
        want = tables[o][: owned[o].numel()].double() - 0.5 * G[torch.searchsorted(keys, owned[o])]
        assert torch.allclose(w[: owned[o].numel()].double(), want, atol=10 * tol, rtol=1e-4)
    # ---- two-shot all-reduce of a flat buffer (phase kernel of every logical rank, one after the other)
    n = 4 * W * 1000
    bufs = [torch.randn(n, device=dev) for _ in range(W)]
    mean = torch.stack(bufs).double().mean(0)
    for r in range(W):
        C.comm_allreduce_slice(ptrs(bufs), r, n, 1.0 / W)
    for b in bufs:
        assert torch.allclose(b.double(), mean, atol=1e-5)
    assert int(status.item()) == 0
