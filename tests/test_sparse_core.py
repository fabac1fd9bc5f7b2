"""CPU tests of the native sparse core against plain PyTorch restatements of each operation."""
import math

import pytest
import torch

import recis_b200
from recis_b200.nn import EmbeddingEngine, EmbeddingOption, HashTable, filter_out_sparse_param, gen_slice
from recis_b200.nn.hashtable_hook import AdmitHook, FilterHook
from recis_b200.nn.initializers import ConstantInitializer, NormalInitializer, TruncNormalInitializer, UniformInitializer
from recis_b200.optim import SparseAdagrad, SparseAdam, SparseAdamW, SparseAdamWTF
from recis_b200.ragged import RaggedTensor

C = recis_b200.native()


def make_store(dim=8, cap=64, device="cpu", kind=2, a=0.0, b=0.01):
    return C.EmbeddingStore(dim, cap, device, kind, a, b, 0.0, 0.0, 1234, True, True, None)


def test_gen_slice_covers_space():
    for w in (1, 2, 3, 7, 8, 64):
        ranges = [gen_slice(r, w) for r in range(w)]
        assert ranges[0].slice_begin == 0 and ranges[-1].slice_end == 65536
        for a, b in zip(ranges, ranges[1:]):
            assert a.slice_end == b.slice_begin
        sizes = [r.slice_end - r.slice_begin for r in ranges]
        assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_dedup_partition(world):
    torch.manual_seed(world)
    ids = torch.randint(-5, 2000, (5000,), dtype=torch.int64) * 7919
    uniq, rev, counts, offs = C.dedup_partition(ids, world)
    nu = int(offs[-1])
    assert nu == ids.unique().numel()
    assert torch.equal(uniq[:nu][rev.long()], ids)
    assert torch.equal(offs[1:] - offs[:-1], counts)
    # every unique id sits in the bucket of its owner rank
    for r in range(world):
        sl = gen_slice(r, world)
        seg = uniq[offs[r]:offs[r + 1]] & 0xFFFF
        assert bool(((seg >= sl.slice_begin) & (seg < sl.slice_end)).all())


def test_store_insert_find_erase_grow():
    st = make_store(dim=8, cap=16)
    ids = torch.arange(1, 3001, dtype=torch.int64) * 104729
    rows = st.lookup_or_insert(ids, None, None, 1)
    assert rows.min() >= 0 and rows.unique().numel() == 3000
    assert st.size() == 3000 and st.capacity() >= 3000
    assert torch.equal(st.find(ids, None), rows)
    assert int(st.find(torch.tensor([5, -1, -2]), None).max()) == -1
    # values are a function of the id: a second store with another insertion order agrees
    st2 = make_store(dim=8, cap=4096)
    perm = torch.randperm(3000)
    rows2 = st2.lookup_or_insert(ids[perm].contiguous(), None, None, 1)
    e1 = st.emb()[rows.long()][perm]
    e2 = st2.emb()[rows2.long()]
    assert torch.equal(e1, e2)
    assert abs(float(e1.std()) - 0.01) < 1e-3
    erased = st.erase(ids[:1000].contiguous())
    assert torch.equal(erased, rows[:1000])
    assert st.size() == 2000
    assert int(st.find(ids[:1000].contiguous(), None).max()) == -1
    # freed rows are reused before the arena grows
    cap_before = st.capacity()
    new_ids = torch.arange(1, 1001, dtype=torch.int64) * 15485863 + 1
    rows3 = st.lookup_or_insert(new_ids, None, None, 1)
    assert set(rows3.tolist()) == set(rows[:1000].tolist())
    assert st.capacity() == cap_before
    k, r = st.snapshot(False, 0)
    assert k.numel() == 3000


def test_store_count_admission_and_ttl():
    st = make_store()
    ids = torch.tensor([11, 22, 33], dtype=torch.int64)
    step = torch.tensor([1], dtype=torch.int64)
    r1 = st.lookup_or_insert(ids, None, step, 2)
    assert r1.tolist() == [-1, -1, -1] and st.size() == 0
    r2 = st.lookup_or_insert(ids[:2].contiguous(), None, step, 2)
    assert (r2 >= 0).all() and st.size() == 2
    step.fill_(10)
    st.lookup_or_insert(ids[:1].contiguous(), None, step, 2)
    expired, _ = st.snapshot(True, 5)   # last_seen < 5
    assert expired.tolist() == [22]


@pytest.mark.parametrize("dim", [1, 3, 8, 16, 64, 128, 200])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_pool_and_grad_reduce_match_torch(dim, mode):
    torch.manual_seed(dim * 7 + mode)
    U, S = 37, 23
    emb = torch.randn(U, dim)
    lens = torch.randint(0, 6, (S,))
    offsets = torch.zeros(S + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(lens, 0)
    n = int(offsets[-1])
    rev = torch.randint(0, U, (n,), dtype=torch.int32)
    rev[:U] = torch.arange(U, dtype=torch.int32)[: min(U, n)] if n >= U else rev[:U]
    w = torch.rand(n) + 0.5
    out, gsrc, gscale = C.pool_forward(emb, None, rev, offsets, w, mode, 0, 0, True)
    ref = torch.zeros(S, dim)
    seg = torch.repeat_interleave(torch.arange(S), lens)
    ref.index_add_(0, seg, emb[rev.long()] * w[:, None])
    if mode == 1:
        ref = ref / lens.clamp(min=1)[:, None]
    elif mode == 2:
        ws = torch.zeros(S).index_add_(0, seg, w)
        ref = torch.where(ws[:, None] != 0, ref / ws[:, None].clamp(min=1e-30), ref)
    assert torch.allclose(out, ref, atol=1e-5, rtol=1e-5)
    # backward structure
    if n == 0:
        return
    dense_rev = torch.unique(rev, return_inverse=True)[1].to(torch.int32)   # dense unique indices, as dedup gives
    out2, gsrc, gscale = C.pool_forward(emb, None, dense_rev, offsets, w, mode, 0, 0, True)
    csr_u, csr_e, start = C.build_csr(dense_rev)
    go = torch.randn(S, dim)
    nu = int(dense_rev.max()) + 1
    gu = C.grad_reduce(go, gsrc, gscale, csr_u, csr_e, start, dim, None, False, 2, 0, 0, 0, 0, 1, 0, 1.0, None, None, None, nu)
    ref_gu = torch.zeros(nu, dim).index_add_(0, dense_rev.long(), go[gsrc.long()] * gscale[:, None])
    assert torch.allclose(gu, ref_gu, atol=1e-5, rtol=1e-5)


def test_tile_forward():
    torch.manual_seed(0)
    emb = torch.randn(10, 4)
    offsets = torch.tensor([0, 2, 2, 7], dtype=torch.int32)
    rev = torch.tensor([0, 1, 2, 3, 4, 5, 6], dtype=torch.int32)
    out, gsrc, gscale = C.tile_forward(emb, None, rev, offsets, None, 3, True)
    assert out.shape == (3, 12)
    assert torch.equal(out[0, :8].view(2, 4), emb[:2]) and float(out[0, 8:].abs().sum()) == 0
    assert float(out[1].abs().sum()) == 0
    assert torch.equal(out[2].view(3, 4), emb[2:5])
    assert gsrc.tolist() == [0, 1, 6, 7, 8, -1, -1]


def _adam_ref(w, m, v, g, lr, b1, b2, eps, decay, t):
    alpha = -lr * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    return w * decay + alpha * m / (v.sqrt() + eps), m, v


@pytest.mark.parametrize("opt_cls,decay_fn", [
    (SparseAdam, lambda lr, wd: 1.0), (SparseAdamW, lambda lr, wd: 1 - lr * wd), (SparseAdamWTF, lambda lr, wd: 1 - wd)])
def test_sparse_adam_family_matches_reference_math(opt_cls, decay_fn):
    torch.manual_seed(0)
    ht = HashTable([8], initializer=NormalInitializer(0, 0.1), name="t_adam", device="cpu")
    ht._worker_num = 1
    opt = opt_cls(filter_out_sparse_param(ht), lr=0.01, weight_decay=0.01)
    ids = torch.tensor([5, 9, 5, 7, 9, 5])
    w = {}
    state = {}
    for t in range(1, 4):
        emb = ht(ids)
        if t == 1:
            for i, e in zip(ids.tolist(), emb.detach()):
                w[i] = e.clone(); state[i] = (torch.zeros(8), torch.zeros(8))
        coef = torch.arange(1, 7, dtype=torch.float32)[:, None] * t
        loss = (emb * coef).sum()
        opt.zero_grad(); loss.backward(); opt.step()
        for i in set(ids.tolist()):
            g = sum(coef[j] for j, x in enumerate(ids.tolist()) if x == i).expand(8)
            w[i], m, v = _adam_ref(w[i], *state[i], g, 0.01, 0.9, 0.999, 1e-8, decay_fn(0.01, 0.01), t)
            state[i] = (m, v)
    ht.eval()
    final = ht(torch.tensor([5, 9, 7]))
    ref = torch.stack([w[5], w[9], w[7]])
    assert torch.allclose(final, ref, atol=1e-6, rtol=1e-5)


def test_sparse_adagrad_matches_dense_torch_adagrad():
    torch.manual_seed(0)
    V, D = 20, 8
    ht = HashTable([D], initializer=NormalInitializer(0, 0.1), name="t_adagrad", device="cpu")
    ht._worker_num = 1
    opt = SparseAdagrad(filter_out_sparse_param(ht), lr=0.05, eps=1e-10)
    all_ids = torch.arange(V)
    ht.eval(); dense_w = ht(all_ids).detach().clone(); ht.train()
    # ids are inserted by the eval lookup? no: eval is read-only, so insert explicitly through a training lookup
    ht(all_ids)
    ht.impl.clear_grad()
    ht.eval(); dense_w = ht(all_ids).detach().clone(); ht.train()
    dense = torch.nn.Parameter(dense_w.clone())
    ref_opt = torch.optim.Adagrad([dense], lr=0.05, eps=1e-10)
    for t in range(5):
        ids = torch.randint(0, V, (16,))
        coef = torch.randn(16, D)
        loss = (ht(ids) * coef).sum()
        opt.zero_grad(); loss.backward(); opt.step()
        ref_loss = (dense[ids] * coef).sum()
        ref_opt.zero_grad(); ref_loss.backward()
        # torch's dense Adagrad also "updates" untouched rows with zero gradient: a no-op, same as skipping them
        ref_opt.step()
    ht.eval()
    assert torch.allclose(ht(all_ids), dense.detach(), atol=1e-6, rtol=1e-5)


def test_embedding_engine_merges_and_matches_embedding_bag():
    torch.manual_seed(0)
    D, B = 16, 12
    init = NormalInitializer(0, 0.05)
    opts = {
        "a": EmbeddingOption(embedding_dim=D, shared_name="a", combiner="sum", initializer=init, device="cpu"),
        "b": EmbeddingOption(embedding_dim=D, shared_name="b", combiner="sum", initializer=init, device="cpu"),
        "a_mean": EmbeddingOption(embedding_dim=D, shared_name="a", combiner="mean", initializer=init, device="cpu"),
        "c8": EmbeddingOption(embedding_dim=8, shared_name="c8", combiner="sum", initializer=init, device="cpu"),
    }
    eng = EmbeddingEngine(opts)
    assert len(eng.tables()) == 2          # dim 16 (a, b merged) and dim 8
    t16 = eng.table_of("a")
    assert t16 is eng.table_of("b") and t16 is eng.table_of("a_mean")
    assert t16.impl.children_info().children() == ["a", "b"]

    def ragged(maxid):
        lens = torch.randint(1, 5, (B,))
        off = torch.zeros(B + 1, dtype=torch.int32); off[1:] = torch.cumsum(lens, 0)
        return RaggedTensor(torch.randint(0, maxid, (int(off[-1]),)), [off])

    feats = {"a": ragged(30), "b": ragged(30), "a_mean": ragged(30), "c8": torch.randint(0, 10, (B, 3)), "x": torch.randn(B, 2)}
    out = eng(feats)
    assert out["a"].shape == (B, D) and out["c8"].shape == (B, 8) and out["x"] is feats["x"]
    # same raw id in features a and b are different rows (different child prefix); a and a_mean share rows
    ids_a = feats["a"].values()
    ht = t16.table; ht.eval()
    enc = lambda ids, child: (ids & ((1 << 52) - 1)) | (child << 52)
    ea = ht(enc(ids_a, 0)); eb = ht(enc(ids_a, 1))
    assert not torch.allclose(ea, eb)
    lens = feats["a"].offsets()[0][1:] - feats["a"].offsets()[0][:-1]
    seg = torch.repeat_interleave(torch.arange(B), lens.long())
    ref_a = torch.zeros(B, D).index_add_(0, seg, ea)
    assert torch.allclose(out["a"], ref_a, atol=1e-6)
    ids_m = feats["a_mean"].values()
    lens_m = (feats["a_mean"].offsets()[0][1:] - feats["a_mean"].offsets()[0][:-1]).long()
    seg_m = torch.repeat_interleave(torch.arange(B), lens_m)
    ref_m = torch.zeros(B, D).index_add_(0, seg_m, ht(enc(ids_m, 0))) / lens_m[:, None]
    assert torch.allclose(out["a_mean"], ref_m, atol=1e-6)


def test_engine_training_matches_dense_oracle():
    """Two steps of sum-pooled training equal the same steps on an nn.Embedding initialised with the table's rows."""
    torch.manual_seed(0)
    D, B, V = 8, 16, 40
    opts = {"f": EmbeddingOption(embedding_dim=D, shared_name="f", combiner="sum", initializer=NormalInitializer(0, 0.1),
                                 device="cpu", use_weight=False)}
    eng = EmbeddingEngine(opts)
    opt = SparseAdagrad(filter_out_sparse_param(eng), lr=0.1, eps=1e-10)
    table = eng.table_of("f").table
    table(torch.arange(V)); table.impl.clear_grad()
    table.eval(); w0 = table(torch.arange(V)).detach().clone(); table.train()
    dense = torch.nn.Embedding(V, D); dense.weight.data.copy_(w0)
    ref_opt = torch.optim.Adagrad(dense.parameters(), lr=0.1, eps=1e-10)
    for t in range(3):
        ids = torch.randint(0, V, (B, 5))
        coef = torch.randn(B, D)
        loss = (eng({"f": ids})["f"] * coef).sum()
        opt.zero_grad(); loss.backward(); opt.step()
        ref = (dense(ids).sum(1) * coef).sum()
        ref_opt.zero_grad(); ref.backward(); ref_opt.step()
    table.eval()
    assert torch.allclose(table(torch.arange(V)), dense.weight.detach(), atol=1e-5, rtol=1e-5)


def test_readonly_and_eval_do_not_insert():
    ht = HashTable([4], initializer=ConstantInitializer(1.0), name="t_ro", device="cpu")
    out = ht(torch.tensor([1, 2, 3]), admit_hook=AdmitHook("ReadOnly"))
    assert float(out.abs().sum()) == 0 and ht.impl.size() == 0
    ht.eval()
    assert float(ht(torch.tensor([1, 2])).abs().sum()) == 0 and ht.impl.size() == 0
    ht.train()
    assert torch.equal(ht(torch.tensor([1, 2])), torch.ones(2, 4)) and ht.impl.size() == 2


def test_filter_hook_evicts_stale_rows():
    ht = HashTable([4], initializer=ConstantInitializer(1.0), name="t_ttl", device="cpu",
                   filter_hook=FilterHook("GlobalStepFilter", {"filter_step": 2}))
    hook = ht._filter_hook_impl
    ht(torch.tensor([1, 2, 3]))
    for _ in range(4):
        hook.update_step()
        ht(torch.tensor([1]))
    assert hook.do_filter() == 2
    assert sorted(ht.ids().tolist()) == [1]


@pytest.mark.parametrize("init,check", [
    (ConstantInitializer(0.5), lambda e: bool((e == 0.5).all())),
    (UniformInitializer(-1, 1), lambda e: float(e.min()) >= -1 and float(e.max()) <= 1 and abs(float(e.mean())) < 0.05),
    (NormalInitializer(1.0, 2.0), lambda e: abs(float(e.mean()) - 1) < 0.1 and abs(float(e.std()) - 2) < 0.1),
    (TruncNormalInitializer(0, 1, -1, 1), lambda e: float(e.abs().max()) <= 1.0 and 0.45 < float(e.std()) < 0.62),
])
def test_initializers_distribution(init, check):
    ht = HashTable([16], initializer=init, name=f"t_init_{type(init).__name__}", device="cpu")
    e = ht(torch.arange(2000))
    assert check(e.detach())


@pytest.mark.parametrize("decoupled", [False, True])
def test_dense_adam_cpu_matches_torch(decoupled):
    from recis_b200.optim import DenseAdam
    torch.manual_seed(0)
    a = [torch.randn(5, 3).requires_grad_(), torch.randn(7).requires_grad_()]
    b = [p.detach().clone().requires_grad_() for p in a]
    o1 = DenseAdam(a, lr=1e-2, weight_decay=0.01, decoupled=decoupled)
    o2 = (torch.optim.AdamW if decoupled else torch.optim.Adam)(b, lr=1e-2, weight_decay=0.01)
    for _ in range(4):
        for x, y in zip(a, b):
            g = torch.randn_like(x)
            x.grad = g.clone()
            y.grad = g.clone()
        o1.step()
        o2.step()
    for x, y in zip(a, b):
        torch.testing.assert_close(x, y, rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("world,dim", [(2, 16), (3, 8), (4, 128), (8, 64)])
def test_exchange_host_twins_loopback(world, dim):
    """All logical ranks of one exchange step in this process, through the host twins of the exchange kernels (the same harness
    drives the device kernels on one GPU)."""
    from loopback_case import run_loopback
    run_loopback(torch.device("cpu"), world, dim)


@pytest.mark.parametrize("world,dim", [(3, 8), (4, 32)])
def test_exchange_host_twins_overflow_is_clamped(world, dim):
    """Every id goes to logical rank 0, whose receive window is too small: boundaries are clamped, guard rows stay untouched."""
    from loopback_case import run_loopback_overflow
    run_loopback_overflow(torch.device("cpu"), world, dim)


def test_erased_index_slots_are_reused_by_inserts_of_distinct_ids():
    """Steady eviction must not fill the index with tombstones: new ids (distinct within a call) take erased slots on their
    probe path, so churn of a fixed working set leaves the tombstone count near zero instead of growing by the set size per round."""
    C = recis_b200.native()
    store = C.EmbeddingStore(8, 4096, "cpu", 0, 0.0, 0.0, 0.0, 0.0, 1, True, True, None)
    live = torch.arange(0, 3000, dtype=torch.int64)
    store.lookup_or_insert(live, None, None, 1, True)
    slots0 = store.keys().numel()
    for rnd in range(1, 30):
        store.erase(live[:1500].contiguous())
        assert store.counters()[5] == 1500 or rnd > 1                      # tombstones right after an eviction
        fresh = torch.arange(100_000 * rnd, 100_000 * rnd + 1500, dtype=torch.int64)
        rows = store.lookup_or_insert(fresh, None, None, 1, True)
        assert int(rows.min()) >= 0
        assert torch.equal(store.find(fresh), rows)
        live = torch.cat([fresh, live[1500:]])
        assert store.size() == 3000
        assert torch.all(store.find(live) >= 0)
    c = store.counters()
    # 29 rounds erased 43,500 ids: without reuse and clean-up the index would hold as many tombstones (and would have doubled
    # several times); it keeps its size and the erased slots stay a fraction of it
    assert c[5] < 0.65 * slots0 and store.keys().numel() == slots0, (c[5], store.keys().numel())


def test_debug_bounds_mode_rejects_bad_row_indices_before_the_kernel_runs():
    """With RECIS_DEBUG_BOUNDS=1 the bindings of the row-indexing kernels validate their index tensors and raise; nothing reads
    or writes outside its buffers. The switch is read once per process, so the check runs in a child."""
    import subprocess
    import sys
    code = r"""
import torch, recis_b200
C = recis_b200.native()
src = torch.arange(12, dtype=torch.float32).view(4, 3)
ok = C.gather_rows(src, torch.tensor([0, -1, 3], dtype=torch.int32), None)
assert ok[1].abs().sum() == 0 and torch.equal(ok[2], src[3])
def raises(fn, what):
    try:
        fn()
    except RuntimeError as e:
        assert what in str(e), str(e)
        return
    raise AssertionError("no error for " + what)
raises(lambda: C.gather_rows(src, torch.tensor([0, 4], dtype=torch.int32), None), "gather_rows: rows")
raises(lambda: C.scatter_rows(src.clone(), torch.tensor([7], dtype=torch.int32), torch.zeros(1, 3), False), "scatter_rows: rows")
# entries past the device-side count are not looked at
n_dev = torch.tensor([1], dtype=torch.int32)
C.gather_rows(src, torch.tensor([2, 99], dtype=torch.int32), n_dev)
rev = torch.tensor([0, 1, 5], dtype=torch.int32)
offs = torch.tensor([0, 2, 3], dtype=torch.int32)
raises(lambda: C.pool_forward(src, torch.tensor([0, 1], dtype=torch.int32), rev, offs, None, 0, 0, 0, False, None, 0, 0), "pool_forward: reverse index")
raises(lambda: C.pool_forward(src, torch.tensor([0, 9], dtype=torch.int32), torch.tensor([0, 1, 1], dtype=torch.int32), offs, None, 0, 0, 0, False,
                              None, 0, 0), "pool_forward: table rows")
print("ok")
"""
    import os
    env = dict(os.environ, RECIS_DEBUG_BOUNDS="1")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stdout + out.stderr
