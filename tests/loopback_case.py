"""One exchange step with ``world`` logical ranks inside ONE process: every 'peer pointer' is a local buffer and the phases run one
after the other (nothing ever waits for anything), so the id pull, the row push, the gradient push, the owner-side reduce /
update and the two-shot all-reduce are checked against a dense oracle. On ``cuda`` this runs the device kernels, on ``cpu`` their
host twins; the harness is the same."""
import torch


def run_loopback(dev, world, dim):
    import recis_b200
    C = recis_b200.native()
    torch.manual_seed(world * 100 + dim)
    W, D, S = world, dim, 700
    cap = 8192                                             # window capacity in unique ids per rank
    in_cap = min(W, 2) * cap
    status = torch.zeros(1, dtype=torch.int64, device=dev)
    ids, offs, revs = [], [], []
    ids_win = [torch.zeros(cap, dtype=torch.int64, device=dev) for _ in range(W)]
    off_win = [torch.zeros(W + 1, dtype=torch.int32, device=dev) for _ in range(W)]
    cnt_win = [torch.zeros(W, dtype=torch.int32, device=dev) for _ in range(W)]
    demand = torch.zeros(2, dtype=torch.int32, device=dev)
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
        _u, rev, _c, _o = C.dedup_partition(ids[r], W, ids_win[r], off_win[r], status, cnt_win[r])
        revs.append(rev)
    # ---- owners: pull ids, resolve rows, push rows to the requesters
    ids_in, prefix, rows_in, tables, owned = [], [], [], [], []
    for o in range(W):
        buf = torch.zeros(in_cap, dtype=torch.int64, device=dev)
        meta = torch.zeros(4 * W + 2, dtype=torch.int32, device=dev)
        n_in = torch.zeros(1, dtype=torch.int32, device=dev)
        C.comm_pull_ids(ptrs(ids_win), ptrs(off_win), ptrs(cnt_win), o, buf, meta, n_in, demand, status)
        n = int(n_in.item())
        assert n == int(meta[W].item()) == sum(int(off_win[r][o + 1] - off_win[r][o]) for r in range(W))
        uniq, inv = torch.unique(buf[:n], return_inverse=True)
        rows = torch.full((in_cap,), -1, dtype=torch.int32, device=dev)
        rows[:n] = inv.to(torch.int32)
        table = torch.randn(max(uniq.numel(), 1), D, device=dev)
        ids_in.append(buf); prefix.append(meta); rows_in.append(rows); tables.append(table); owned.append(uniq)
    all_owned = torch.cat(owned)
    assert all_owned.unique().numel() == all_owned.numel()                     # every id has exactly one owner
    # the demand every owner computed from all requesters' counts: largest unique count of a requester, largest inflow of an owner
    assert int(demand[0]) == max(int(off_win[r][W]) for r in range(W))
    assert int(demand[1]) == max(sum(int(off_win[r][o + 1] - off_win[r][o]) for r in range(W)) for o in range(W))
    for o in range(W):
        C.comm_push_emb(tables[o], rows_in[o], prefix[o], ptrs(uemb), o, in_cap, 37 if o % 2 else 0)   # capped and uncapped grids
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
        C.comm_grad_reduce_push(go, gsrc, gscale, csr_u, csr_elem, start, D, off_win[r], prefix[r], ptrs(gin), in_cap, 53 if r % 2 else 0)
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
        C.comm_allreduce_slice(ptrs(bufs), r, n, 1.0 / W, dev.type != "cuda")
    for b in bufs:
        assert torch.allclose(b.double(), mean, atol=1e-5)
    assert int(status.item()) == 0


def run_loopback_overflow(dev, world, dim):
    """Every id belongs to logical rank 0 and its receive window is far too small: the owner-side kernels must see clamped
    boundaries only (guard rows behind every buffer stay untouched), the overflow bit must be set, and what did fit must be right."""
    import recis_b200
    C = recis_b200.native()
    torch.manual_seed(7)
    W, D, S = world, dim, 200
    cap, in_cap, guard = 1024, 96, 64
    status = torch.zeros(1, dtype=torch.int64, device=dev)
    ptrs = lambda ts: [t.data_ptr() for t in ts]
    ids_win = [torch.zeros(cap, dtype=torch.int64, device=dev) for _ in range(W)]
    off_win = [torch.zeros(W + 1, dtype=torch.int32, device=dev) for _ in range(W)]
    cnt_win = [torch.zeros(W, dtype=torch.int32, device=dev) for _ in range(W)]
    uemb = [torch.full((cap + guard, D), 7.0, device=dev) for _ in range(W)]
    gin = [torch.full((in_cap + guard, D), 7.0, device=dev) for _ in range(W)]
    ids, offs, revs = [], [], []
    for r in range(W):
        o = torch.arange(0, 2 * S + 1, 2, dtype=torch.int32)
        x = (torch.randperm(1000)[: 2 * S] + 1000 * r).to(torch.int64) * 65536          # low 16 bits zero: owner 0, all distinct
        ids.append(x.to(dev)); offs.append(o.to(dev))
        _u, rev, _c, _o = C.dedup_partition(ids[r], W, ids_win[r], off_win[r], status, cnt_win[r])
        revs.append(rev)
    demand = torch.zeros(2, dtype=torch.int32, device=dev)
    metas, rows_all, tables = [], [], []
    for o in range(W):
        buf = torch.full((in_cap + guard,), -5, dtype=torch.int64, device=dev)
        meta = torch.zeros(4 * W + 2, dtype=torch.int32, device=dev)
        n_in = torch.zeros(1, dtype=torch.int32, device=dev)
        C.comm_pull_ids(ptrs(ids_win), ptrs(off_win), ptrs(cnt_win), o, buf[:in_cap], meta, n_in, demand, status)
        n = int(n_in.item())
        assert n == (in_cap if o == 0 else 0) and int(meta[:W + 1].max()) <= in_cap        # clamped boundaries only
        assert bool((buf[in_cap:] == -5).all())
        rows = torch.full((in_cap,), -1, dtype=torch.int32, device=dev)
        rows[:n] = torch.arange(n, dtype=torch.int32, device=dev)
        metas.append(meta); rows_all.append(rows); tables.append(torch.randn(max(n, 1), D, device=dev))
    assert int(status.item()) & 8                                                        # overflow reported
    assert int(demand[1]) == 2 * S * W and int(demand[0]) == 2 * S                       # the true demand, unclamped
    for o in range(W):
        C.comm_push_emb(tables[o], rows_all[o], metas[o], ptrs([u[:cap] for u in uemb]), o, in_cap, 0)
    for r in range(W):
        assert bool((uemb[r][cap:] == 7.0).all())
        go = torch.randn(S, D, device=dev)
        out, gsrc, gscale = C.pool_forward(uemb[r][:cap].contiguous(), None, revs[r], offs[r], None, 0, 0, 0, True)
        csr_u, csr_elem, start = C.build_csr(revs[r])
        C.comm_grad_reduce_push(go, gsrc, gscale, csr_u, csr_elem, start, D, off_win[r], metas[r], ptrs([g[:in_cap] for g in gin]), in_cap, 0)
    for o in range(W):
        assert bool((gin[o][in_cap:] == 7.0).all())                                      # no gradient row landed behind a window
        head = torch.full((tables[o].size(0) + guard,), -1, dtype=torch.int32, device=dev)
        rows, grads = C.comm_owner_reduce(rows_all[o], head, metas[o], gin[o][:in_cap].contiguous(), W, D, False, False, 2, 0.0, 0.0, 0.0,
                                          0.0, 1.0, 0.0, 1.0, None, None, None, in_cap, 2)
        assert int(head.max().item()) == -1
        assert int((rows >= 0).sum()) == (in_cap if o == 0 else 0)
