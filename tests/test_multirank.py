"""Sharded embedding training on several ranks equals the same training in one process.

CPU: gloo ranks drive the collective (all_to_all) path. GPU (>= 2 devices): the fused peer-memory path and the NCCL path
are both compared with the single-process oracle, and the peer-memory dense all-reduce with a plain mean.
"""
import os

import pytest
import torch

from multirank import run_ranks

D = 16
STEPS = 3


def _batch(rank, step, device):
    from recis_b200.ragged import RaggedTensor
    g = torch.Generator().manual_seed(1000 * step + rank)
    feats, coefs = {}, {}
    for name in ("a", "b"):
        lens = torch.randint(0, 6, (32,), generator=g)
        off = torch.zeros(33, dtype=torch.int32); off[1:] = torch.cumsum(lens, 0)
        vals = torch.randint(0, 200, (int(off[-1]),), generator=g) * 7919        # spreads over the 65536 slices
        w = torch.rand(int(off[-1]), generator=g)
        feats[name] = RaggedTensor(vals.to(device), [off.to(device)], weight=w.to(device))
        coefs[name] = torch.randn(32, D, generator=g).to(device)
    return feats, coefs


def _train(rank, world, device_kind, batch_ranks):
    """Train STEPS steps. ``batch_ranks``: which ranks' batches this process consumes each step (oracle: all of them)."""
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseAdam
    device = torch.device("cuda", rank) if device_kind == "cuda" else torch.device("cpu")
    torch.manual_seed(7)            # the row initializer takes its seed from torch's: same in every process
    init = NormalInitializer(0, 0.05)
    opts = {"a": EmbeddingOption(embedding_dim=D, shared_name="a", combiner="sum", initializer=init, device=device),
            "b": EmbeddingOption(embedding_dim=D, shared_name="b", combiner="mean", initializer=init, device=device)}
    eng = EmbeddingEngine(opts)
    opt = SparseAdam(filter_out_sparse_param(eng), lr=0.01)
    n_total = max(world, len(batch_ranks))
    outs = []
    for step in range(STEPS):
        loss = 0.0
        step_out = {}
        opt.zero_grad()
        for br in batch_ranks:
            feats, coefs = _batch(br, step, device)
            out = eng(feats)
            loss = loss + sum((out[k] * coefs[k]).sum() for k in out) / (n_total if world == 1 else 1)
            step_out[br] = {k: v.detach().cpu() for k, v in out.items()}
        loss.backward()
        opt.step()
        outs.append(step_out)
    table = {}
    for ht in eng.tables().values():
        ids, rows = ht.impl.ids_map()
        emb = ht.impl.store.emb()[rows]
        for i, e in zip(ids.tolist(), emb.cpu()):
            table[i] = e
        ex = getattr(ht, "fused", None)
        if world > 1 and os.environ.get("RECIS_COMM") == "fused":
            assert ex is not None and len(ex.lanes) == 2, "the fused exchange did not run"      # one lane per runtime group
        if ex is not None:
            ex.check()
            assert ex.staged_serves == (STEPS * 2 if os.environ.get("RECIS_STAGE_EXCHANGE") == "1" else 0)
    return {"outs": outs, "table": table}


def _rank_fn(rank, world, device_kind):
    return _train(rank, world, device_kind, [rank])


def _oracle(world):
    from recis_b200.nn.modules.hashtable import HashtableRegister
    HashtableRegister().clear()
    os.environ.pop("WORLD_SIZE", None)
    # one process, every rank's batch per step; the worker-mean (1/world) is applied to the loss instead
    return _train(0, 1, "cpu", list(range(world)))


def _compare(results, oracle, world):
    merged = {}
    for r in results:
        assert not (set(r["table"]) & set(merged)), "an id lives on two shards"
        merged.update(r["table"])
    assert set(merged) == set(oracle["table"])
    for step in range(STEPS):
        for r in range(world):
            for k in ("a", "b"):
                assert torch.allclose(results[r]["outs"][step][r][k], oracle["outs"][step][r][k], atol=2e-5, rtol=1e-4), (step, r, k)
    a = torch.stack([merged[i] for i in sorted(merged)])
    b = torch.stack([oracle["table"][i] for i in sorted(merged)])
    assert torch.allclose(a, b, atol=1e-4, rtol=1e-3)


@pytest.mark.parametrize("world", [2, 3, 8])
def test_gloo_ranks_match_single_process(world):
    results = run_ranks(_rank_fn, world, "gloo", args=("cpu",))
    _compare(results, _oracle(world), world)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_fused_exchange_on_cpu_ranks_matches_single_process(world):
    """The fused exchange (windows, flags, id pull, row push, gradient push, owner reduce + update) through its shared-memory CPU
    twin: same Python path as on GPUs, every world size, against the single-process oracle."""
    results = run_ranks(_rank_fn, world, "gloo", args=("cpu",), env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    _compare(results, _oracle(world), world)


def test_staged_fused_exchange_on_cpu_ranks():
    """RECIS_STAGE_EXCHANGE=1: the requester half of both groups' id phases runs before the first wait; same results."""
    results = run_ranks(_rank_fn, 3, "gloo", args=("cpu",), env={"RECIS_COMM": "fused", "RECIS_STAGE_EXCHANGE": "1", "RECIS_WAIT_TIMEOUT_S": "60"})
    _compare(results, _oracle(3), 3)


def _fused_variants_fn(rank, world):
    """Gradient accumulation (two micro-batches per update), mean-by-id across requesters, and an eval lookup, on the fused
    exchange; every rank also computes the single-process answer from all ranks' batches."""
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.nn.modules.hashtable import HashtableRegister
    from recis_b200.optim import SparseSGD

    def batch(r, step):
        g = torch.Generator().manual_seed(100 * step + r)
        return torch.randint(0, 40, (16, 3), generator=g) * 7919, torch.randn(16, 8, generator=g)

    def run(world_here, ranks, name):
        torch.manual_seed(5)
        eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name=name, combiner="sum", grad_reduce_by="id",
                                                    initializer=NormalInitializer(0, 0.05))})
        opt = SparseSGD(filter_out_sparse_param(eng), lr=0.1)
        opt.set_grad_accum_steps(2)
        for step in range(4):                       # two updates of two micro-batches each
            opt.zero_grad()
            loss = 0.0
            for r in ranks:
                ids, coef = batch(r, step)
                loss = loss + (eng({"a": ids})["a"] * coef).sum()
            loss.backward()
            opt.step()
        eng.eval()
        probe = torch.arange(0, 40).view(-1, 1) * 7919
        with torch.no_grad():
            return eng({"a": probe})["a"].clone(), eng

    got, eng = run(world, [rank], "variants")
    (table,) = eng.tables().values()
    assert table.fused is not None
    table.fused.check()
    return got


def test_fused_exchange_accumulation_and_mean_by_id_on_cpu_ranks():
    world = 2
    res = run_ranks(_fused_variants_fn, world, "gloo", env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    col = run_ranks(_fused_variants_fn_collective, world, "gloo")
    for a, b in zip(res, col):
        assert torch.allclose(a, b, atol=1e-5), float((a - b).abs().max())
    assert torch.allclose(res[0], res[1], atol=1e-6)            # every rank reads the same rows back
    assert float(res[0].abs().sum()) > 0


def _fused_variants_fn_collective(rank, world):
    """The same program on the collective (all-to-all) path."""
    os.environ["RECIS_COMM"] = "nccl"
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseSGD
    torch.manual_seed(5)
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name="variants", combiner="sum", grad_reduce_by="id",
                                                initializer=NormalInitializer(0, 0.05))})
    opt = SparseSGD(filter_out_sparse_param(eng), lr=0.1)
    opt.set_grad_accum_steps(2)
    for step in range(4):
        opt.zero_grad()
        g = torch.Generator().manual_seed(100 * step + rank)
        ids, coef = torch.randint(0, 40, (16, 3), generator=g) * 7919, torch.randn(16, 8, generator=g)
        (eng({"a": ids})["a"] * coef).sum().backward()
        opt.step()
    eng.eval()
    (table,) = eng.tables().values()
    assert table.fused is None
    with torch.no_grad():
        return eng({"a": torch.arange(0, 40).view(-1, 1) * 7919})["a"].clone()


def _missing_peer_fn(rank, world):
    """Step 1 runs on both ranks (it creates the windows); at step 2 rank 1 never shows up: rank 0's bounded waits run out, the
    status word says so, and check() raises - nothing hangs."""
    import time
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption
    from recis_b200.nn.initializers import NormalInitializer
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name="missing_peer", initializer=NormalInitializer(0, 0.05))})
    ids = torch.arange(20).view(-1, 1) * 7919 + rank
    eng({"a": ids})
    (table,) = eng.tables().values()
    table.fused.check()
    if rank == 1:
        time.sleep(6.0)                           # alive, but absent from the step
        return "absent"
    t0 = time.monotonic()
    eng({"a": ids})                               # two waits of one second each run out
    took = time.monotonic() - t0
    try:
        table.fused.check()
        return ("no error", took)
    except RuntimeError as e:
        return (str(e), took)


def test_missing_peer_ends_in_a_timeout_status_not_a_hang():
    res = run_ranks(_missing_peer_fn, 2, "gloo", env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "1"}, timeout=120)
    msg, took = res[0]
    assert "did not signal" in msg and took < 5.0
    assert res[1] == "absent"


def _capacity_fn(rank, world, mode):
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption
    from recis_b200.nn.initializers import NormalInitializer
    cap = {"uneven": 300 + 200 * rank, "tiny": 8}[mode]          # per-rank window capacity in unique ids
    torch.manual_seed(1)
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name=f"cap_{mode}", initializer=NormalInitializer(0, 0.05),
                                                exchange_capacity=cap)})
    g = torch.Generator().manual_seed(rank)
    ids = torch.randint(0, 150, (40, 2), generator=g) * 7919
    out = eng({"a": ids})["a"].detach().clone()
    (table,) = eng.tables().values()
    (lane,) = table.fused.lanes.values()
    try:
        table.fused.check()
        err = None
    except RuntimeError as e:
        err = str(e)
    # what the rows should be: the initializer is a pure function of (seed, id, column), so any table gives the reference values
    torch.manual_seed(1)
    from recis_b200.nn.modules.hashtable import HashtableRegister
    os.environ["RECIS_COMM"] = "nccl"
    ref_eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name=f"cap_{mode}_ref", initializer=NormalInitializer(0, 0.05))})
    ref = ref_eng({"a": ids})["a"].detach().clone()
    return {"send_cap": lane.send_cap, "err": err, "same": bool(torch.allclose(out, ref, atol=1e-6))}


def test_window_capacity_is_agreed_across_ranks_and_overflow_is_reported():
    res = run_ranks(_capacity_fn, 3, "gloo", args=("uneven",), env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    assert {r["send_cap"] for r in res} == {700}                 # the largest request wins on every rank: identical layouts
    assert all(r["err"] is None and r["same"] for r in res)
    res = run_ranks(_capacity_fn, 2, "gloo", args=("tiny",), env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    assert all(r["err"] is not None and "overflow" in r["err"] for r in res)      # flagged, nothing written out of bounds


def _lanes_fn(rank, world, lanes):
    """Four features of one runtime group, optionally split into two exchange lanes; two training steps; returns outputs + rows."""
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseAdam
    torch.manual_seed(11)
    init = NormalInitializer(0, 0.05)
    names = ["f0", "f1", "f2", "f3"]
    eng = EmbeddingEngine({n: EmbeddingOption(embedding_dim=8, shared_name=n, combiner="sum", initializer=init) for n in names},
                          interleave=True, exchange_lanes=lanes)
    opt = SparseAdam(filter_out_sparse_param(eng), lr=0.05)
    outs = []
    for step in range(2):
        g = torch.Generator().manual_seed(10 * step + rank)
        feats = {n: torch.randint(0, 60, (12, 2), generator=g) * 7919 for n in names}
        coef = {n: torch.randn(12, 8, generator=g) for n in names}
        opt.zero_grad()
        out = eng(feats)
        sum((out[n] * coef[n]).sum() for n in names).backward()
        opt.step()
        outs.append({n: out[n].detach().clone() for n in names})
    (table,) = eng.tables().values()
    if table.fused is not None:
        table.fused.check()
        assert len(table.fused.lanes) == max(lanes, 1)
    ids, rows = table.impl.ids_map()
    order = torch.argsort(ids)
    return {"outs": outs, "ids": ids[order], "emb": table.impl.store.emb()[rows[order]].clone()}


def test_exchange_lanes_on_cpu_ranks_equal_the_single_lane_run():
    env = {"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"}
    two = run_ranks(_lanes_fn, 2, "gloo", args=(2,), env=env)
    one = run_ranks(_lanes_fn, 2, "gloo", args=(1,), env=env)
    for a, b in zip(two, one):
        assert torch.equal(a["ids"], b["ids"]) and torch.allclose(a["emb"], b["emb"], atol=1e-6)
        for x, y in zip(a["outs"], b["outs"]):
            assert all(torch.allclose(x[n], y[n], atol=1e-6) for n in x)


def _shared_child_lanes_fn(rank, world, lanes, interleave, device_kind="cpu"):
    """Six features over four child tables: f1 and f2 share ``s1``, f4 and f5 share ``s3``. Lanes must keep the features of one
    child together; a row that landed in two lanes would be updated twice per step."""
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseAdam
    torch.manual_seed(13)
    dev = torch.device("cuda", rank) if device_kind == "cuda" else torch.device("cpu")
    init = NormalInitializer(0, 0.05)
    shared = {"f0": "s0", "f1": "s1", "f2": "s1", "f3": "s2", "f4": "s3", "f5": "s3"}
    eng = EmbeddingEngine({n: EmbeddingOption(embedding_dim=8, shared_name=sn, combiner="sum", initializer=init, device=dev)
                           for n, sn in shared.items()}, interleave=interleave, exchange_lanes=lanes)
    opt = SparseAdam(filter_out_sparse_param(eng), lr=0.05)
    outs = []
    for step in range(3):
        g = torch.Generator().manual_seed(10 * step + rank)
        feats = {n: (torch.randint(0, 40, (12, 2), generator=g) * 7919).to(dev) for n in shared}   # small id range: f1/f2 and f4/f5 collide a lot
        coef = {n: torch.randn(12, 8, generator=g).to(dev) for n in shared}
        opt.zero_grad()
        out = eng(feats)
        sum((out[n] * coef[n]).sum() for n in shared).backward()
        opt.step()
        outs.append({n: out[n].detach().cpu().clone() for n in shared})
    (table,) = eng.tables().values()
    n_lanes = len(table.fused.lanes)
    table.fused.check()
    ids, rows = table.impl.ids_map()
    order = torch.argsort(ids)
    return {"outs": outs, "ids": ids[order].cpu(), "emb": table.impl.store.emb()[rows[order]].cpu().clone(), "n_lanes": n_lanes}


@pytest.mark.parametrize("interleave", [True, False])
def test_lanes_keep_features_of_one_shared_name_together(interleave):
    env = {"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"}
    three = run_ranks(_shared_child_lanes_fn, 2, "gloo", args=(3, interleave), env=env)
    one = run_ranks(_shared_child_lanes_fn, 2, "gloo", args=(1, interleave), env=env)
    assert all(r["n_lanes"] == 3 for r in three) and all(r["n_lanes"] == 1 for r in one)
    for a, b in zip(three, one):
        assert torch.equal(a["ids"], b["ids"]) and torch.allclose(a["emb"], b["emb"], atol=1e-6)
        for x, y in zip(a["outs"], b["outs"]):
            assert all(torch.allclose(x[n], y[n], atol=1e-6) for n in x)


def test_lane_ranges_never_split_a_child():
    from recis_b200.nn.modules.embedding_engine import EmbeddingEngine
    f = EmbeddingEngine._lane_ranges
    assert f([0, 1, 2, 3], 2) == [0, 2, 4]
    ch = [0, 1, 1, 2, 3, 3]
    b = f(ch, 3)
    assert len(b) == 4 and b[0] == 0 and b[-1] == 6
    parts = [set(ch[x:y]) for x, y in zip(b, b[1:])]
    assert all(not (parts[i] & parts[j]) for i in range(3) for j in range(i + 1, 3))
    assert f([0, 1, 0, 1], 2) == [0, 4]                    # interleaved children: no legal cut, one lane
    assert f([0, 0, 0], 4) == [0, 3]
    b = f(list(range(26)), 4)
    assert b[0] == 0 and b[-1] == 26 and len(b) == 5 and all(y > x for x, y in zip(b, b[1:]))


def _skewed_ids_fn(rank, world, strict, device_kind="cpu"):
    """Every id is a multiple of 65536, so rank 0 owns all of them: the receive window of rank 0 is asked for world times what
    a balanced batch would bring. Step 1 sizes the windows from a small batch, step 2 is four times larger."""
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption
    from recis_b200.nn.initializers import NormalInitializer
    torch.manual_seed(3)
    dev = torch.device("cuda", rank) if device_kind == "cuda" else torch.device("cpu")
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name=f"skewed_{strict}", initializer=NormalInitializer(0, 0.05),
                                                exchange_strict=strict, device=dev)})
    (table,) = eng.tables().values()
    outs, refs, errs = [], [], []
    os.environ["RECIS_COMM"] = "nccl"
    torch.manual_seed(3)
    ref_eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name=f"skewed_{strict}_ref", initializer=NormalInitializer(0, 0.05),
                                                    device=dev)})
    for step, n in enumerate((600, 2400, 2400, 2400, 2400)):
        g = torch.Generator().manual_seed(100 * step + rank)
        ids = ((torch.randperm(4000, generator=g)[:n] + 4000 * rank).view(-1, 2) * 65536).to(dev)
        outs.append(eng({"a": ids})["a"].detach().cpu().clone())
        refs.append(ref_eng({"a": ids})["a"].detach().cpu().clone())
        try:
            table.fused.check()
            errs.append(None)
        except RuntimeError as e:
            errs.append(str(e))
    (lane,) = table.fused.lanes.values()
    return {"same": [bool(torch.allclose(o, r, atol=1e-6)) for o, r in zip(outs, refs)], "errs": errs, "grown": lane.grown,
            "caps": (lane.send_cap, lane.in_cap)}


@pytest.mark.parametrize("world", [3, 4])
def test_skewed_ids_overflow_is_memory_safe_then_windows_grow(world):
    """Default mode: the step that outgrows the windows is flagged (ids dropped, nothing indexed out of bounds - the CPU twin
    runs the same clamps), the measured demand makes every rank grow its windows two lookups later, and from then on the
    results are exact again."""
    res = run_ranks(_skewed_ids_fn, world, "gloo", args=(False,), env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    for r in res:
        assert r["same"][0] and r["errs"][0] is None
        assert r["errs"][1] is not None and "overflow" in r["errs"][1]
        assert r["grown"] >= 1 and r["same"][-1] and r["errs"][-1] is None
    assert len({r["caps"] for r in res}) == 1                      # identical layouts on every rank after growing


def test_strict_exchange_repeats_the_id_phase_instead_of_dropping_ids():
    res = run_ranks(_skewed_ids_fn, 3, "gloo", args=(True,), env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    for r in res:
        assert all(r["same"]) and all(e is None for e in r["errs"]) and r["grown"] >= 1


def _bf16_rows_fn(rank, world, lanes):
    """bf16 rows through the exchange: the wire format of a row is its 2-byte storage format."""
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseAdam
    torch.manual_seed(17)
    init = NormalInitializer(0, 0.05)
    names = ["h0", "h1", "h2"]
    eng = EmbeddingEngine({n: EmbeddingOption(embedding_dim=8, shared_name=n, combiner="sum", initializer=init, dtype=torch.bfloat16)
                           for n in names}, interleave=True, exchange_lanes=lanes)
    opt = SparseAdam(filter_out_sparse_param(eng), lr=0.05)
    outs = []
    for step in range(3):
        g = torch.Generator().manual_seed(10 * step + rank)
        feats = {n: torch.randint(0, 60, (12, 2), generator=g) * 7919 for n in names}
        coef = {n: torch.randn(12, 8, generator=g) for n in names}
        opt.zero_grad()
        out = eng(feats)
        sum((out[n].float() * coef[n]).sum() for n in names).backward()
        opt.step()
        outs.append({n: out[n].detach().float().clone() for n in names})
    (table,) = eng.tables().values()
    if table.fused is not None:
        table.fused.check()
        (lane, *_rest) = table.fused.lanes.values()
        assert lane.heap["uemb"].tensor.dtype == torch.bfloat16
    assert table.impl.store.emb().dtype == torch.bfloat16
    ids, rows = table.impl.ids_map()
    order = torch.argsort(ids)
    return {"outs": outs, "ids": ids[order], "emb": table.impl.store.emb()[rows[order]].float().clone()}


def test_bf16_rows_through_the_fused_exchange_match_the_collective_exchange():
    fused = run_ranks(_bf16_rows_fn, 2, "gloo", args=(2,), env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    coll = run_ranks(_bf16_rows_fn, 2, "gloo", args=(1,), env={"RECIS_COMM": "nccl"})
    for a, b in zip(fused, coll):
        assert torch.equal(a["ids"], b["ids"]) and torch.allclose(a["emb"], b["emb"], atol=2e-3)
        for x, y in zip(a["outs"], b["outs"]):
            assert all(torch.allclose(x[n], y[n], atol=2e-2) for n in x)


def _skewed_fn(rank, world, jitter):
    """Many short steps with random delays in front of every flag signal and every pull / push: the ranks drift apart as far as
    the protocol lets them. Returns the final rows."""
    import random
    import time
    import torch
    import recis_b200.parallel.fused_exchange as fx
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseAdagrad
    if jitter:
        real = fx.native()
        rnd = random.Random(1234 + rank)

        class Slow:
            def __getattr__(self, name):
                fn = getattr(real, name)
                if name in ("comm_signal", "comm_pull_ids", "comm_push_emb", "comm_grad_reduce_push", "comm_owner_reduce"):
                    def delayed(*a, **k):
                        time.sleep(rnd.random() * 0.004)
                        return fn(*a, **k)
                    return delayed
                return fn
        slow = Slow()
        fx.native = lambda: slow
    torch.manual_seed(21)
    init = NormalInitializer(0, 0.05)
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name="skew_a", combiner="sum", initializer=init),
                           "b": EmbeddingOption(embedding_dim=8, shared_name="skew_b", combiner="mean", initializer=init)})
    opt = SparseAdagrad(filter_out_sparse_param(eng), lr=0.05)
    for step in range(15):
        g = torch.Generator().manual_seed(1000 * step + rank)
        feats = {n: torch.randint(0, 80, (10, 3), generator=g) * 7919 for n in ("a", "b")}
        opt.zero_grad()
        out = eng(feats)
        sum(v.square().sum() for v in out.values()).backward()
        opt.step()
    rows = {}
    for table in eng.tables().values():
        if table.fused is not None:
            table.fused.check()
        ids, r = table.impl.ids_map()
        for i, e in zip(ids.tolist(), table.impl.store.emb()[r]):
            rows[i] = e.clone()
    return rows


def test_fused_exchange_under_random_skew_between_ranks():
    """15 training steps on three CPU ranks with random delays before every signal, pull and push give the same rows."""
    env = {"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"}
    skewed = run_ranks(_skewed_fn, 3, "gloo", args=(True,), env=env)
    calm = run_ranks(_skewed_fn, 3, "gloo", args=(False,), env=env)
    for a, b in zip(skewed, calm):
        assert a.keys() == b.keys()
        assert all(torch.allclose(a[k], b[k], atol=1e-6) for k in a)


def _wait_stats_fn(rank, world):
    """RECIS_WAIT_STATS=1: rank 1 arrives 0.3 s late at one step; rank 0's accounted wait on the ids channel shows it."""
    import time
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption
    from recis_b200.nn.initializers import NormalInitializer
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name="wait_stats", initializer=NormalInitializer(0, 0.05))})
    ids = torch.arange(30).view(-1, 1) * 7919 + rank
    eng({"a": ids})
    if rank == 1:
        time.sleep(0.3)
    eng({"a": ids})
    (table,) = eng.tables().values()
    table.fused.check()
    return table.fused.exposed_wait_ms()


def test_wait_accounting_on_cpu_ranks():
    res = run_ranks(_wait_stats_fn, 2, "gloo", env={"RECIS_COMM": "fused", "RECIS_WAIT_STATS": "1", "RECIS_WAIT_TIMEOUT_S": "60"})
    assert set(res[0]) >= {"ids", "emb"}
    assert res[0]["ids"] > 100.0                      # mean over two waits, one of which lasted about 300 ms
    assert res[1]["ids"] < res[0]["ids"]              # the late rank itself hardly waited


def _combiner_fn(rank, world):
    """tile and weighted-mean combiners, count-based admission and a read-only (eval) lookup; two steps; returns all outputs."""
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.hashtable_hook import AdmitHook
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseSGD
    from recis_b200.ragged import RaggedTensor
    torch.manual_seed(31)
    init = NormalInitializer(0, 0.05)
    eng = EmbeddingEngine({
        "seq": EmbeddingOption(embedding_dim=8, shared_name="cmb_seq", combiner="tile", combiner_kwargs={"tile_len": 3}, initializer=init),
        "wm": EmbeddingOption(embedding_dim=8, shared_name="cmb_wm", combiner="mean", use_weight=True, initializer=init),
        "adm": EmbeddingOption(embedding_dim=8, shared_name="cmb_adm", combiner="sum", initializer=init,
                               admit_hook=AdmitHook("CountAdmit", {"threshold": 2})),
    })
    opt = SparseSGD(filter_out_sparse_param(eng), lr=0.1)
    outs = []
    for step in range(3):
        g = torch.Generator().manual_seed(7 * step + rank)
        lens = torch.randint(0, 5, (10,), generator=g)
        off = torch.zeros(11, dtype=torch.int32); off[1:] = lens.cumsum(0)
        n = int(off[-1])
        feats = {"seq": RaggedTensor(torch.randint(0, 50, (n,), generator=g) * 7919, [off]),
                 "wm": RaggedTensor(torch.randint(0, 50, (n,), generator=g) * 7919, [off], weight=torch.rand(n, generator=g) + 0.1),
                 # many of these ids are asked for by both ranks in the same step: one sighting per id and step on either exchange
                 "adm": torch.randint(0, 30, (10, 2), generator=g) * 7919}
        opt.zero_grad()
        out = eng(feats)
        sum(v.square().sum() for v in out.values()).backward()
        opt.step()
        outs.append({k: v.detach().clone() for k, v in out.items()})
    eng.eval()
    with torch.no_grad():
        probe = eng({"adm": torch.arange(0, 30).view(-1, 1) * 7919})["adm"].clone()      # read-only: never-admitted ids read as zeros
    for t in eng.tables().values():
        if t.fused is not None:
            t.fused.check()
    return {"outs": outs, "probe": probe, "fused": any(t.fused is not None for t in eng.tables().values())}


def test_combiners_and_admission_agree_between_the_fused_and_the_collective_exchange():
    fused = run_ranks(_combiner_fn, 2, "gloo", env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    coll = run_ranks(_combiner_fn, 2, "gloo", env={"RECIS_COMM": "nccl"})
    assert all(r["fused"] for r in fused) and not any(r["fused"] for r in coll)
    for a, b in zip(fused, coll):
        assert torch.allclose(a["probe"], b["probe"], atol=1e-6)
        for x, y in zip(a["outs"], b["outs"]):
            for k in x:
                assert x[k].shape == y[k].shape and torch.allclose(x[k], y[k], atol=1e-6), k
    assert float(fused[0]["probe"].abs().sum()) > 0 and bool((fused[0]["probe"].abs().sum(1) == 0).any())   # some admitted, some not


def _two_lookups_fn(rank, world):
    """The same feature group is looked up TWICE before the backward (two towers sharing an engine): fine on the collective
    exchange; the fused exchange, whose windows belong to one lookup per step, must say so instead of mixing gradients up. A
    read-only lookup between a training forward and its backward is allowed on both."""
    import torch
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseSGD
    torch.manual_seed(41)
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name="twice", initializer=NormalInitializer(0, 0.05))})
    opt = SparseSGD(filter_out_sparse_param(eng), lr=0.1)
    g = torch.Generator().manual_seed(rank)
    left, right = (torch.randint(0, 40, (8, 2), generator=g) * 7919 for _ in range(2))
    # a training forward, a read-only forward of the same group, then the backward of the first: allowed
    opt.zero_grad()
    out = eng({"a": left})["a"]
    eng.eval()
    with torch.no_grad():
        eng({"a": right})
    eng.train()
    out.square().sum().backward()
    opt.step()
    # two training forwards before the backward
    opt.zero_grad()
    out = eng({"a": left})["a"] + eng({"a": right})["a"]
    try:
        out.square().sum().backward()
        opt.step()
        return "ok"
    except RuntimeError as e:
        return str(e)


def test_two_training_lookups_of_one_group_before_the_backward():
    coll = run_ranks(_two_lookups_fn, 2, "gloo", env={"RECIS_COMM": "nccl"})
    assert coll == ["ok", "ok"]
    fused = run_ranks(_two_lookups_fn, 2, "gloo", env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "30", "RB_NO_FINAL_BARRIER": "1"})
    assert all("looked up again before the gradients" in r for r in fused), fused


def _need_gpus(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.gpu
@pytest.mark.parametrize("comm", ["fused", "nccl"])
def test_gpu_ranks_match_single_process(comm):
    _need_gpus(2)
    world = min(torch.cuda.device_count(), int(os.environ.get("RECIS_TEST_GPU_RANKS", "2")))   # 2 ranks by default; more on request
    results = run_ranks(_rank_fn, world, "nccl", args=("cuda",), env={"RECIS_COMM": comm, "NCCL_NVLS_ENABLE": "0"})
    _compare(results, _oracle(world), world)


@pytest.mark.gpu
@pytest.mark.parametrize("interleave", [True, False])
def test_gpu_exchange_lanes_pipeline_matches_single_lane_cpu_ranks(interleave):
    """Three lanes on two CUDA streams (link stream for the NVLink-bound kernels) on real peers against the single-lane run of
    the exchange's host twin."""
    _need_gpus(2)
    gpu = run_ranks(_shared_child_lanes_fn, 2, "nccl", args=(3, interleave, "cuda"), env={"RECIS_COMM": "fused", "NCCL_NVLS_ENABLE": "0"})
    cpu = run_ranks(_shared_child_lanes_fn, 2, "gloo", args=(1, interleave), env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    assert all(r["n_lanes"] == 3 for r in gpu)
    for a, b in zip(gpu, cpu):
        assert torch.equal(a["ids"], b["ids"]) and torch.allclose(a["emb"], b["emb"], atol=1e-5)
        for x, y in zip(a["outs"], b["outs"]):
            assert all(torch.allclose(x[n], y[n], atol=1e-5) for n in x)


@pytest.mark.gpu
def test_gpu_exchange_windows_grow_and_strict_mode_on_real_peers():
    _need_gpus(2)
    for strict in (False, True):
        res = run_ranks(_skewed_ids_fn, 2, "nccl", args=(strict, "cuda"), env={"RECIS_COMM": "fused", "NCCL_NVLS_ENABLE": "0"})
        for r in res:
            assert r["grown"] >= 1 and r["same"][-1] and r["errs"][-1] is None
            if strict:
                assert all(r["same"]) and all(e is None for e in r["errs"])


def _allreduce_fn(rank, world, device_kind="cuda"):
    import torch
    from recis_b200.parallel.dense_reducer import DenseGradReducer
    dev = torch.device("cuda", rank) if device_kind == "cuda" else torch.device("cpu")
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.zeros(s, device=dev)) for s in ((1000, 37), (513,), (64, 64))]
    red = DenseGradReducer(params, world)
    assert red.p2p
    outs = []
    for it in range(3):
        g = torch.Generator(device="cpu").manual_seed(100 * it + rank)
        for p in params:
            p.grad.copy_(torch.randn(p.shape, generator=g).to(dev))
        red.all_reduce()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        outs.append([p.grad.detach().cpu().clone() for p in params])
    red.check()
    return outs


def _check_allreduce(results, world):
    shapes = ((1000, 37), (513,), (64, 64))
    for it in range(3):
        per_rank = []
        for r in range(world):
            g = torch.Generator().manual_seed(100 * it + r)
            per_rank.append([torch.randn(s, generator=g) for s in shapes])
        for k in range(len(shapes)):
            mean = sum(per_rank[r][k] for r in range(world)) / world
            for r in range(world):
                assert torch.allclose(results[r][it][k], mean, atol=1e-6)


@pytest.mark.parametrize("world", [2, 3])
def test_two_shot_dense_allreduce_on_cpu_ranks(world):
    """The flat-buffer two-shot all-reduce (signal, wait, reduce my slice from all peers, write it back to all, signal, wait)
    through the shared-memory twin: 3 ranks exercise the padding of the buffer to a multiple of 4 * world."""
    results = run_ranks(_allreduce_fn, world, "gloo", args=("cpu",), env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    _check_allreduce(results, world)


@pytest.mark.gpu
def test_p2p_dense_allreduce():
    _need_gpus(2)
    world = min(torch.cuda.device_count(), int(os.environ.get("RECIS_TEST_GPU_RANKS", "2")))   # 2 ranks by default; more on request
    results = run_ranks(_allreduce_fn, world, "nccl", env={"RECIS_COMM": "fused", "NCCL_NVLS_ENABLE": "0"})
    _check_allreduce(results, world)


def _bucketed_backward_fn(rank, world, device_kind, comm):
    """A four-layer tower whose gradients are averaged bucket by bucket from backward's hooks; one parameter takes no part in
    the graph, and the second step is an accumulation of two micro-batches with the division folded into the average."""
    import torch
    from recis_b200.parallel.dense_reducer import DenseGradReducer
    dev = torch.device("cuda", rank) if device_kind == "cuda" else torch.device("cpu")
    torch.manual_seed(1)
    layers = torch.nn.ModuleList([torch.nn.Linear(24, 40), torch.nn.Linear(40, 40), torch.nn.Linear(40, 33), torch.nn.Linear(33, 1)]).to(dev)
    unused = torch.nn.Parameter(torch.ones(7, device=dev))
    params = list(layers.parameters()) + [unused]
    red = DenseGradReducer(params, world, bucket_mb=40 * 40 * 4 / (1 << 20))
    assert red.p2p == (comm == "fused") and len(red.buckets) >= 3

    def loss_of(step, r, micro):
        g = torch.Generator().manual_seed(1000 * step + 10 * r + micro)
        x = torch.randn(16, 24, generator=g).to(dev)
        for l in layers[:-1]:
            x = torch.relu(l(x))
        return layers[-1](x).square().mean()

    out = []
    for step, accum in ((0, 1), (1, 1), (2, 2)):
        red.flat.zero_()
        red.grad_scale = 1.0 / accum
        for micro in range(accum):
            red.armed = micro == accum - 1
            loss_of(step, rank, micro).backward()
        started_in_backward = sum(b.launched for b in red.buckets)
        red.all_reduce_async()
        red.wait()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        got = [p.grad.detach().cpu().clone() for p in params]
        # the oracle: every rank's gradients computed here, without the reducer
        red.armed = False
        for p in params:
            p.grad = None
        want = [torch.zeros(p.shape) for p in params]
        for r in range(world):
            for micro in range(accum):
                loss_of(step, r, micro).backward()
        for k, p in enumerate(params):
            if p.grad is not None:
                want[k] = p.grad.detach().cpu() / (world * accum)
        out.append((got, want, started_in_backward))
        # back to views of the flat buffer for the next step
        for p, start in red._placement:
            p.grad = red.flat[start:start + p.numel()].view_as(p)
    red.check()
    return out


@pytest.mark.parametrize("comm", ["fused", "nccl"])
def test_dense_buckets_start_from_backward_hooks_on_cpu_ranks(comm):
    results = run_ranks(_bucketed_backward_fn, 2, "gloo", args=("cpu", comm), env={"RECIS_COMM": comm, "RECIS_WAIT_TIMEOUT_S": "60"})
    for res in results:
        for step, (got, want, started) in enumerate(res):
            assert started == 0 if step == 0 else started >= 3      # the first step learns which parameters get gradients
            for a, b in zip(got, want):
                assert torch.allclose(a, b, atol=1e-6), float((a - b).abs().max())


@pytest.mark.gpu
def test_gpu_dense_buckets_start_from_backward_hooks():
    _need_gpus(2)
    results = run_ranks(_bucketed_backward_fn, 2, "nccl", args=("cuda", "fused"), env={"RECIS_COMM": "fused", "NCCL_NVLS_ENABLE": "0"})
    for res in results:
        for step, (got, want, started) in enumerate(res):
            assert started == 0 if step == 0 else started >= 3
            for a, b in zip(got, want):
                assert torch.allclose(a, b, atol=1e-5), float((a - b).abs().max())


def _staged_fn(rank, world):
    """Two tables looked up through the three-stage interface with both id exchanges started before either is finished."""
    import torch
    from recis_b200.nn import DynamicEmbedding, EmbeddingOption
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.ragged import RaggedTensor
    torch.manual_seed(3)
    init = NormalInitializer(0, 0.05)
    tabs = [DynamicEmbedding(EmbeddingOption(embedding_dim=8, shared_name=f"staged_{i}", combiner="sum", initializer=init)) for i in range(2)]
    g = torch.Generator().manual_seed(rank)
    data = []
    for _ in tabs:
        lens = torch.randint(0, 5, (16,), generator=g)
        off = torch.zeros(17, dtype=torch.int32); off[1:] = torch.cumsum(lens, 0)
        data.append((torch.randint(0, 300, (int(off[-1]),), generator=g) * 7919, off))
    started = [t.exchange_ids(ids, off) for t, (ids, off) in zip(tabs, data)]        # both id phases in flight
    assert all(s.prepared is not None for s in started)
    staged = [t.emb_reduce(t.lookup_exchange_emb(s), None, "sum") for t, s in zip(tabs, started)]
    direct = [t(RaggedTensor(ids, [off])) for t, (ids, off) in zip(tabs, data)]
    return [bool(torch.allclose(a.view_as(b), b)) for a, b in zip(staged, direct)]


def test_staged_interface_on_gloo_ranks():
    results = run_ranks(_staged_fn, 2, "gloo")
    assert all(all(r) for r in results)
