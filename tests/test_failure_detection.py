"""Failure detection without touching a GPU: ranks are CPU processes (gloo); the failures are made on the host - a rank that
stops sending heartbeats, a rank that exits, a collective that a peer never joins, a checkpoint shard cut short."""
import os
import time

import pytest
import torch
import torch.distributed as dist

from multirank import run_ranks


def _heartbeat_case(rank, world, mode):
    from recis_b200.framework.health import PeerLostError, PeerMonitor
    mon = PeerMonitor(rank, world, interval=0.1, timeout=1.0).start()
    dist.barrier()
    out = {"rank": rank}
    if mode == "stall" and rank == 1:
        mon.pause()                       # a hung process: alive, but silent
        time.sleep(4.0)
    elif mode == "leave" and rank == 1:
        mon.leave()                       # clean exit between steps
        time.sleep(3.0)
    else:
        t0 = time.monotonic()
        lost = None
        while time.monotonic() - t0 < 3.0:
            try:
                mon.check()
            except PeerLostError as e:
                lost = (e.rank, time.monotonic() - t0)
                break
            time.sleep(0.05)
        out["lost"] = lost
        out["alive"] = mon.alive()
        if lost is None:
            time.sleep(max(0.0, 3.2 - (time.monotonic() - t0)))
        else:
            time.sleep(max(0.0, 4.2 - (time.monotonic() - t0)))    # keep the store's host alive until the stalled rank wakes up
    mon.leave()
    return out


def test_stalled_rank_is_detected_by_heartbeat():
    res = run_ranks(_heartbeat_case, 3, "gloo", args=("stall",))
    for r in (0, 2):
        lost_rank, after = res[r]["lost"]
        assert lost_rank == 1 and after < 2.5


def test_clean_leave_is_not_a_failure():
    res = run_ranks(_heartbeat_case, 3, "gloo", args=("leave",))
    for r in (0, 2):
        assert res[r]["lost"] is None and 1 not in res[r]["alive"]


def _collective_timeout_case(rank, world):
    from datetime import timedelta
    # a second group with a short timeout: rank 1 never joins the all-reduce, the others must get an error, not a hang
    g = dist.new_group(ranks=list(range(world)), backend="gloo", timeout=timedelta(seconds=2))
    t = torch.ones(4)
    if rank == 1:
        time.sleep(5.0)
        return {"joined": False}
    t0 = time.monotonic()
    try:
        dist.all_reduce(t, group=g)
        err = None
    except RuntimeError as e:
        err = str(e)[:200]
    return {"joined": True, "error": err, "after": time.monotonic() - t0}


def test_collective_with_missing_peer_times_out_with_an_error():
    try:
        res = run_ranks(_collective_timeout_case, 2, "gloo")
    except RuntimeError as e:            # gloo may tear the pair down while rank 1 still sleeps; the helper's final barrier then fails
        assert "rank 0" not in str(e) or "timed out" not in str(e)
        return
    assert res[0]["error"] is not None and res[0]["after"] < 4.5


def test_truncated_checkpoint_shard_is_a_clean_error(tmp_path):
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.modules.hashtable import HashtableRegister
    from recis_b200.serialize import Loader, Saver
    HashtableRegister().clear()
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu")})
    eng({"a": torch.arange(100)})
    Saver(0, 1, 1, str(tmp_path), filter_out_sparse_param(eng), {}).save()
    shard = [f for f in os.listdir(tmp_path) if f.endswith(".safetensors")][0]
    size = os.path.getsize(tmp_path / shard)
    with open(tmp_path / shard, "r+b") as fh:
        fh.truncate(size - 64)
    HashtableRegister().clear()
    eng2 = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu")})
    with pytest.raises((RuntimeError, ValueError, OSError)):
        Loader(str(tmp_path), filter_out_sparse_param(eng2), {}).load()


def _trainer_case(rank, world, mode):
    """Two ranks train DeepFM through the Trainer with heartbeats on; in ``mode == "die"`` rank 1 stops after two steps."""
    import tempfile

    from recis_b200.framework import Trainer, TrainingArguments
    from recis_b200.framework.health import PeerLostError
    from recis_b200.io import SparseFieldSpec, StateDataset, SyntheticDataset, SyntheticSpec, WrapEndDataset
    from recis_b200.models.deepfm import DeepFM
    from recis_b200.nn import filter_out_sparse_param
    from recis_b200.optim import DenseAdam, SparseAdagrad
    torch.manual_seed(0)
    fields = ["c0", "c1", "c2"]
    spec = SyntheticSpec(batch=32, dense_dim=13, label_rate=0.3, seed=rank,
                         sparse=[SparseFieldSpec(f, zipf_a=1.1, id_bits=20, universe=500, length="fixed", mean_len=1) for f in fields])
    model = DeepFM(fields, device="cpu", compute_dtype=torch.float32, hidden=(16,))

    class Loss(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m
            self.calls = 0

        def forward(self, batch):
            self.calls += 1
            if mode == "die" and rank == 1 and self.calls == 3:
                os._exit(0)                      # a crashed rank: no clean-up, no further heartbeats, between two steps
            return self.m(batch)[0]

    steps = 4 if mode == "ok" else 400
    args = TrainingArguments(output_dir=tempfile.mkdtemp(), log_steps=100, train_steps=steps, save_steps=10_000, heartbeat_timeout=1.5,
                             stop_check_interval=10_000)
    wrapped = Loss(model)
    trainer = Trainer(model=wrapped, args=args, train_dataset=WrapEndDataset(StateDataset(SyntheticDataset(spec, steps=steps), save_interval=50)),
                      dense_optimizers=(DenseAdam([p for p in model.parameters() if p.requires_grad], lr=1e-3), None),
                      sparse_optimizer=SparseAdagrad(filter_out_sparse_param(model), lr=0.01))
    assert trainer.peer_monitor is not None
    try:
        trainer.train()
        return {"done": True, "steps": wrapped.calls}
    except PeerLostError as e:
        return {"done": False, "lost": e.rank, "steps": wrapped.calls}
    except RuntimeError as e:                 # the collective inside a step noticed first (connection closed by the dead peer)
        return {"done": False, "lost": None, "error": str(e)[:120], "steps": wrapped.calls}


def test_trainer_with_heartbeats_runs_clean_on_two_ranks():
    res = run_ranks(_trainer_case, 2, "gloo", args=("ok",))
    assert all(r["done"] and r["steps"] == 4 for r in res)


def test_trainer_reports_a_rank_that_died_between_steps():
    res = run_ranks(_trainer_case, 2, "gloo", args=("die",), env={"RB_NO_FINAL_BARRIER": "1"}, allow_missing=True, timeout=120)
    assert res[1] is None                                   # the dead rank left nothing
    survivor = res[0]
    assert survivor is not None and survivor["done"] is False and survivor["steps"] < 400
    assert survivor.get("lost") == 1 or survivor.get("error")


def test_peer_that_starts_late_is_not_reported_lost():
    """A fake store in one process: a peer whose first heartbeat arrives later than ``timeout`` after this rank's monitor was
    created is given the start-up allowance; once seen, going silent for ``timeout`` reports it; never appearing at all reports
    it after the start-up allowance."""
    from recis_b200.framework.health import PeerLostError, PeerMonitor

    class FakeStore(dict):
        def set(self, k, v):
            self[k] = v

        def check(self, keys):
            return all(k in self for k in keys)

        def get(self, k):
            return self[k].encode()

    store = FakeStore()
    mon = PeerMonitor(0, 2, store=store, interval=0.0, timeout=0.2, startup_timeout=1.0)
    time.sleep(0.3)
    mon.check()                                   # peer 1 has published nothing yet: within the start-up allowance
    store.set("recis_b200/hb/1", "0")
    mon.check()                                   # first sight
    time.sleep(0.1)
    store.set("recis_b200/hb/1", "1")
    mon.check()
    time.sleep(0.3)
    with pytest.raises(PeerLostError) as e:
        mon.check()                               # silent for longer than the timeout after having been seen
    assert e.value.rank == 1
    late = PeerMonitor(0, 2, store=FakeStore(), interval=0.0, timeout=0.1, startup_timeout=0.3)
    late.check()
    time.sleep(0.4)
    with pytest.raises(PeerLostError):
        late.check()                              # never showed up at all


def test_trainer_on_two_cpu_ranks_with_the_fused_exchange():
    """The same two-rank Trainer run with the embedding exchange and the dense all-reduce on their shared-memory paths."""
    res = run_ranks(_trainer_case, 2, "gloo", args=("ok",), env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "60"})
    assert all(r["done"] and r["steps"] == 4 for r in res)


def test_trainer_survivor_on_the_fused_exchange_gets_an_error_not_a_hang():
    """Rank 1 dies between steps while the exchange runs over shared memory: rank 0's device-style waits run out (one second each)
    instead of blocking, and the heartbeat monitor names the lost rank before a later step."""
    res = run_ranks(_trainer_case, 2, "gloo", args=("die",), allow_missing=True, timeout=180,
                    env={"RB_NO_FINAL_BARRIER": "1", "RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "1"})
    assert res[1] is None
    survivor = res[0]
    assert survivor is not None and survivor["done"] is False and survivor["steps"] < 400
    assert survivor.get("lost") == 1 or survivor.get("error")


def _overflow_trainer_fn(rank, world):
    """Exchange windows far too small for the batches: the Trainer's periodic status check ends the run with an error."""
    import tempfile
    from recis_b200.framework import Trainer, TrainingArguments
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseSGD

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name="overflow_tab", exchange_capacity=4,
                                                             initializer=NormalInitializer(0, 0.05))})
            self.lin = torch.nn.Linear(8, 1)

        def forward(self, batch):
            return self.lin(self.emb({"a": batch["a"]})["a"]).square().mean()
    m = M()
    data = [{"a": torch.arange(64).view(-1, 1) * 7919 + rank} for _ in range(6)]
    args = TrainingArguments(output_dir=tempfile.mkdtemp(), log_steps=2, train_steps=6, save_steps=1000, stop_check_interval=1000)
    trainer = Trainer(model=m, args=args, train_dataset=data, dense_optimizers=(torch.optim.SGD(m.lin.parameters(), lr=0.1), None),
                      sparse_optimizer=SparseSGD(filter_out_sparse_param(m), lr=0.1))
    try:
        trainer.train()
        return "no error"
    except RuntimeError as e:
        return str(e)


def test_trainer_stops_on_an_exchange_window_overflow():
    res = run_ranks(_overflow_trainer_fn, 2, "gloo", env={"RECIS_COMM": "fused", "RECIS_WAIT_TIMEOUT_S": "30"})
    assert all("overflow" in r for r in res), res


def _param_sync_fn(rank, world):
    """Ranks build their dense towers from different seeds; the Trainer starts all of them from rank 0's weights."""
    import tempfile
    from recis_b200.framework import Trainer, TrainingArguments
    torch.manual_seed(100 + rank)
    m = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.BatchNorm1d(3))
    before = m[0].weight.detach().clone()
    Trainer(model=m, args=TrainingArguments(output_dir=tempfile.mkdtemp()), train_dataset=[],
            dense_optimizers=(torch.optim.SGD(m.parameters(), lr=0.1), None))
    return before, m[0].weight.detach().clone(), m[1].running_mean.clone()


def test_trainer_starts_every_rank_from_rank_zero_dense_weights():
    res = run_ranks(_param_sync_fn, 2, "gloo")
    assert not torch.equal(res[0][0], res[1][0])                 # they were built differently
    assert torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][1], res[0][0])      # rank 0's values everywhere
    assert torch.equal(res[0][2], res[1][2])
