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
        for ex in [getattr(ht, "fused", None)]:
            if ex is not None:
                ex.check()
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


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_gloo_ranks_match_single_process(world):
    results = run_ranks(_rank_fn, world, "gloo", args=("cpu",))
    _compare(results, _oracle(world), world)


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


def _allreduce_fn(rank, world):
    import torch
    from recis_b200.parallel.dense_reducer import DenseGradReducer
    dev = torch.device("cuda", rank)
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
        torch.cuda.synchronize()
        outs.append([p.grad.detach().cpu().clone() for p in params])
    red.check()
    return outs


@pytest.mark.gpu
def test_p2p_dense_allreduce():
    _need_gpus(2)
    world = min(torch.cuda.device_count(), int(os.environ.get("RECIS_TEST_GPU_RANKS", "2")))   # 2 ranks by default; more on request
    results = run_ranks(_allreduce_fn, world, "nccl", env={"RECIS_COMM": "fused", "NCCL_NVLS_ENABLE": "0"})
    shapes = ((1000, 37), (513,), (64, 64))
    for it in range(3):
        expect = []
        for s in shapes:
            acc = torch.zeros(s)
            for r in range(world):
                pass
            expect.append(acc)
        # regenerate every rank's gradients in the same order as the workers did
        per_rank = []
        for r in range(world):
            g = torch.Generator().manual_seed(100 * it + r)
            per_rank.append([torch.randn(s, generator=g) for s in shapes])
        for k in range(len(shapes)):
            mean = sum(per_rank[r][k] for r in range(world)) / world
            for r in range(world):
                assert torch.allclose(results[r][it][k], mean, atol=1e-6)


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
