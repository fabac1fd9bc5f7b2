"""Trainer, checkpoint manager, hooks, metrics and datasets on CPU (DeepFM on synthetic data, 1 process)."""
import os

import pytest
import torch

from recis_b200.framework import Trainer, TrainingArguments
from recis_b200.framework.metrics import add_metric, get_global_metrics
from recis_b200.hooks import HashTableFilterHook, Hook, LoggerHook
from recis_b200.io import (SparseFieldSpec, StateDataset, SyntheticDataset, SyntheticSpec, TensorDataset, WrapEndDataset)
from recis_b200.metrics.auroc import AUROC
from recis_b200.metrics.gauc import Gauc
from recis_b200.models.deepfm import DeepFM
from recis_b200.nn import filter_out_sparse_param
from recis_b200.nn.modules.hashtable import HashtableRegister
from recis_b200.optim import AdamWTF, SparseAdagrad
from recis_b200.utils.parser import ArgumentParser


def _spec(batch=64):
    fields = [f"c{i}" for i in range(6)]
    return fields, SyntheticSpec(batch=batch, dense_dim=13, label_rate=0.25, seed=0,
                                 sparse=[SparseFieldSpec(f, zipf_a=1.1, id_bits=20, universe=2000, length="fixed", mean_len=1) for f in fields])


def _build(tmp, steps, save_steps=5):
    HashtableRegister().clear()
    torch.manual_seed(0)
    fields, spec = _spec()
    model = DeepFM(fields, device="cpu", compute_dtype=torch.float32, hidden=(32, 16))
    sparse_opt = SparseAdagrad(filter_out_sparse_param(model), lr=0.01)
    dense_opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    ds = WrapEndDataset(StateDataset(SyntheticDataset(spec, steps=steps), save_interval=1))

    class Wrapped(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, batch):
            loss, logit = self.m(batch)
            add_metric("mean_logit", logit.detach().mean())
            return loss

    args = TrainingArguments(output_dir=str(tmp), log_steps=2, train_steps=steps, save_steps=save_steps, max_to_keep=2)
    return Trainer(model=Wrapped(model), args=args, train_dataset=ds, dense_optimizers=(dense_opt, None), sparse_optimizer=sparse_opt), model


def test_trainer_trains_saves_and_resumes(tmp_path):
    class Count(Hook):
        n = 0
        def after_step(self, metrics=None, global_step=0):
            Count.n += 1
            assert "loss" in metrics and "mean_logit" in metrics

    trainer, model = _build(tmp_path, steps=12)
    trainer.add_hook(Count())
    trainer.train()
    assert Count.n == 12
    listing = open(tmp_path / "checkpoint").read().split()
    assert listing == ["ckpt_10", "ckpt_12"]                      # retention keeps the newest two
    assert not os.path.exists(tmp_path / "ckpt_5")
    d = tmp_path / "ckpt_12"
    for f in ("index", "tensorkey.json", "model.pt", "extra.pt", "io_state_0.pt", "io_state_count"):
        assert os.path.exists(d / f), f
    sizes = {n: t.impl.size() for n, t in model.embedding_engine.tables().items()}
    w_ref = model.dnn.layers[0].weight.detach().clone()
    # a fresh process-like restart resumes at step 12 with identical tables and dense weights
    trainer2, model2 = _build(tmp_path, steps=14)
    trainer2.restore()
    assert int(trainer2._global_step) == 12
    assert {n: t.impl.size() for n, t in model2.embedding_engine.tables().items()} == sizes
    assert torch.equal(model2.dnn.layers[0].weight, w_ref)
    assert trainer2.train_dataset.dataset.dataset.dump_io_state()["step"] == 12
    trainer2.train(train_steps=2)
    assert int(trainer2._global_step) == 14


def test_deepfm_loss_decreases_on_cpu():
    HashtableRegister().clear()
    torch.manual_seed(0)
    fields, spec = _spec(batch=256)
    model = DeepFM(fields, device="cpu", compute_dtype=torch.float32, hidden=(64, 32))
    sopt = SparseAdagrad(filter_out_sparse_param(model), lr=0.05)
    dopt = AdamWTF(model.parameters(), lr=1e-2, weight_decay=0.0)
    from recis_b200.io import make_batch
    batch = make_batch(spec, 0)
    losses = []
    for _ in range(30):
        loss, _ = model(batch)
        dopt.zero_grad(); sopt.zero_grad(); loss.backward(); dopt.step(); sopt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0] * 0.8


def test_auroc_matches_exact_and_gauc():
    torch.manual_seed(0)
    y = (torch.rand(5000) < 0.3).float()
    p = (torch.rand(5000) * 0.6 + y * 0.3).clamp(0, 1)
    m = AUROC(num_thresholds=400)
    m.update(p[:2500], y[:2500]); m.update(p[2500:], y[2500:])
    order = torch.argsort(p)
    ranks = torch.empty_like(p); ranks[order] = torch.arange(1, 5001, dtype=torch.float32)
    n1 = y.sum(); n0 = 5000 - n1
    exact = (ranks[y == 1].sum() - n1 * (n1 + 1) / 2) / (n1 * n0)
    assert abs(float(m.compute()) - float(exact)) < 5e-3
    m.reset()
    assert float(m.pos_hist.sum()) == 0
    g = Gauc(dist_sync=False)
    labels = torch.tensor([1.0, 0.0, 1.0, 0.0, 1.0, 1.0, 0.0])
    preds = torch.tensor([0.9, 0.1, 0.2, 0.8, 0.5, 0.6, 0.4])
    groups = torch.tensor([0, 0, 1, 1, 2, 2, 2])
    batch, running = g(labels, preds, groups)
    # group 0: auc 1 (2 samples), group 1: auc 0 (2), group 2: auc 1 (3) -> (2*1 + 2*0 + 3*1) / 7
    assert abs(batch - 5.0 / 7.0) < 1e-9 and abs(running - batch) < 1e-12


def test_datasets_state_and_parser(tmp_path):
    _, spec = _spec(batch=8)
    ds = SyntheticDataset(spec, steps=5)
    it = iter(ds)
    b0 = next(it); b1 = next(it)
    state = ds.dump_io_state()
    b2 = next(it)
    ds2 = SyntheticDataset(spec, steps=5)
    ds2.load_io_state(state)
    c2 = next(iter(ds2))
    assert torch.equal(b2["c0"].values(), c2["c0"].values()) and torch.equal(b2["dense"], c2["dense"])
    assert not torch.equal(b0["c0"].values(), b1["c0"].values())
    td = WrapEndDataset(TensorDataset({"x": torch.arange(10)}, batch_size=4))
    flags = []
    for i, (stop, batch) in enumerate(td):
        flags.append(stop)
        if i == 4:
            break
    assert flags == [False, False, False, True, True]
    parser = ArgumentParser()
    parser.add_arguments(TrainingArguments, dest="train")
    ns = parser.parse_args(["--train.log_steps", "7", "--save_steps", "3", "--output_dir", "/tmp/x"])
    assert ns.train.log_steps == 7 and ns.train.save_steps == 3 and ns.train.output_dir == "/tmp/x" and ns.train.max_to_keep == 5


def test_orc_dataset_parquet(tmp_path):
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    from recis_b200.io import OrcDataset
    table = pa.table({"ids": [[1, 2], [], [3]], "user": ["a", "bb", "a"], "price": [1.0, 2.5, 3.0]})
    path = str(tmp_path / "part-0.parquet")
    pq.write_table(table, path)
    ds = OrcDataset(batch_size=2)
    ds.add_path(path)
    ds.varlen_feature("ids")
    ds.varlen_feature("user", hash_type="farm", hash_bucket=1000)
    ds.fixedlen_feature("price", 0.0)
    batches = list(ds)
    assert len(batches) == 2
    assert batches[0]["ids"].values().tolist() == [1, 2] and batches[0]["ids"].offsets()[0].tolist() == [0, 2, 2]
    assert batches[0]["price"].tolist() == [[1.0], [2.5]]
    u0, u1 = batches[0]["user"].values(), batches[1]["user"].values()
    assert u0[0] == u1[0] and u0[0] != u0[1] and int(u0.max()) < 1000


def test_filter_hook_in_loop():
    HashtableRegister().clear()
    from recis_b200.nn import HashTable
    from recis_b200.nn.hashtable_hook import FilterHook
    ht = HashTable([4], name="ttl_loop", device="cpu", filter_hook=FilterHook("GlobalStepFilter", {"filter_step": 3}))
    hook = HashTableFilterHook(filter_interval=2, model=ht)
    ht(torch.arange(50))
    for step in range(8):
        ht(torch.arange(5))
        hook.after_step({}, step)
    assert ht.impl.size() == 5 and hook.evicted == 45


def test_table_stats_and_hook():
    from recis_b200.hooks import TableStatsHook
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption
    from recis_b200.nn.hashtable_hook import AdmitHook
    HashtableRegister().clear()
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu", capacity=64,
                                                admit_hook=AdmitHook("CountAdmit", {"threshold": 2}))})
    eng.train()
    eng({"a": torch.arange(10)})
    (table,) = eng.tables().values()
    st = table.impl.stats()
    assert st["rows"] == 0 and st["probation"] == 10 and st["status"] == 0          # first sighting: probation only
    eng({"a": torch.arange(6)})
    st = table.impl.stats()
    assert st["rows"] == 6 and st["probation"] == 4 and st["admitted_last_lookup"] == 6
    assert 0 < st["row_load"] <= 1 and 0 < st["index_load"] < 1
    hook = TableStatsHook(eng, interval=1)
    m = {}
    hook.after_step(m, 1)
    assert m["table0/rows"] == 6 and m["table0/rows_delta"] == 6 and m["table0/probation"] == 4


def test_api_parity_helpers(tmp_path):
    import recis_b200
    from recis_b200.features import Feature, Mod
    from recis_b200.hooks import HashTableFilterHook
    from recis_b200.io import TensorDataset
    from recis_b200.io.dataset import get_dir_size
    from recis_b200.nn.modules.hashtable_hook_impl import HashtableHookFactory
    info = recis_b200.get_build_info()
    assert info["cuda_arch"] == "sm_100a" and recis_b200.is_internal_enabled() is False
    f = Feature.from_json({"name": "x", "ops": [{"type": "SelectField", "name": "x"}, {"type": "Mod", "mod_value": 7}]})
    assert len(f.ops) == 2 and isinstance(f.ops[1], Mod) and f.id == id(f)
    h = HashTableFilterHook(filter_interval=10)
    h.reset_filter_interval(3)
    assert h.filter_interval == 3
    fac = HashtableHookFactory()
    with pytest.raises(ValueError):
        fac.regist_filter("GlobalStepFilter", object)
    assert isinstance(fac.get_filters(), dict) and isinstance(fac.get_admits(), dict)
    # map / filter register on the dataset itself (the return value may be ignored); a filter function returning True SKIPS
    ds = TensorDataset({"a": torch.arange(10)}, batch_size=2)
    ds.map(lambda b: {"a": b["a"] * 2})
    ds.filter(lambda b: int(b["a"][0]) % 8 != 0)
    assert [b["a"].tolist() for b in ds] == [[0, 2], [8, 10], [16, 18]]
    from recis_b200.io import FilterDataset, MapDataset
    chained = FilterDataset(MapDataset(TensorDataset({"a": torch.arange(6)}, batch_size=2), [lambda b: {"a": b["a"] + 1}, lambda b: {"a": b["a"] * 10}]),
                            filter_funcs=[lambda b: int(b["a"][0]) == 30])
    assert [b["a"].tolist() for b in chained] == [[10, 20], [50, 60]]
    (tmp_path / "x.bin").write_bytes(b"12345")
    assert get_dir_size(str(tmp_path)) == 5
    m = AUROC(num_thresholds=10)
    tp, fp, tn, fn = m.sync(torch.ones(3), torch.zeros(3), torch.ones(3), torch.zeros(3))
    assert float(tp.sum()) == 3.0


def test_crypto_and_singleton_helpers():
    import base64
    cryptography = pytest.importorskip("cryptography")
    from cryptography.hazmat.primitives import serialization
    from cryptography.hazmat.primitives.asymmetric import rsa
    from recis_b200.common.crypto_utils import decode, encode
    from recis_b200.common.singleton import SingletonMeta
    key = rsa.generate_private_key(public_exponent=65537, key_size=2048)
    pub = base64.b64encode(key.public_key().public_bytes(serialization.Encoding.DER, serialization.PublicFormat.SubjectPublicKeyInfo)).decode()
    priv = base64.b64encode(key.private_bytes(serialization.Encoding.DER, serialization.PrivateFormat.PKCS8, serialization.NoEncryption())).decode()
    assert decode(encode("access-key-123", pub), priv) == "access-key-123"

    class Once(metaclass=SingletonMeta):
        pass
    assert Once() is Once()


def test_span_recorder_accounts_phases_per_step():
    """The communication-span recorder with a fake event class: off by default (no events made), per-label sums per step."""
    from recis_b200.parallel.spans import SpanRecorder

    clock = [0.0]

    class FakeEvent:
        made = 0

        def __init__(self, enable_timing=False):
            FakeEvent.made += 1
            self.t = None

        def record(self):
            clock[0] += 1.0
            self.t = clock[0]

        def elapsed_time(self, other):
            return other.t - self.t

    rec = SpanRecorder(event_cls=FakeEvent)
    assert rec.open("ids") is None and FakeEvent.made == 0          # switched off: nothing is recorded
    rec.close(None)
    rec.start()
    for _ in range(4):
        for label in ("ids", "emb", "ids"):
            tok = rec.open(label)
            clock[0] += 2.5                                          # "device work" between the two events
            rec.close(tok)
    out = rec.stop(steps=4, synchronize=lambda: None)
    assert not rec.enabled
    assert abs(out["ids"] - 2 * 3.5) < 1e-9 and abs(out["emb"] - 3.5) < 1e-9 and abs(out["total"] - 10.5) < 1e-9
    assert rec.stop(steps=1, synchronize=lambda: None) == {"total": 0}


def test_common_config_file_transforms_and_nested_lookup(tmp_path):
    import json
    from recis_b200.common.common_config import get_access_id, get_config, set_config
    p = tmp_path / "conf.json"
    p.write_text(json.dumps({"train": {"lr": 0.1, "table": "$TABLE", "cols": ["a", "$COL", {"deep": "$TABLE"}]}, "name": "job"}))
    conf = set_config(str(p), transforms={"$TABLE": "project.table", "$COL": "b"})
    assert conf["train"]["table"] == "project.table" and conf["train"]["cols"] == ["a", "b", {"deep": "project.table"}]
    assert get_config("train", "lr") == 0.1 and get_config("train", "missing", default=7) == 7 and get_config("name") == "job"
    assert get_config("name", "too_deep", default="d") == "d" and get_config()["name"] == "job"
    set_config({"x": {"y": 1}})
    assert get_config("x", "y") == 1
    set_config('{"z": 2}')
    assert get_config("z") == 2 and set_config() == {} and get_access_id() is None


def test_profiler_hook_writes_a_chrome_trace(tmp_path):
    from recis_b200.hooks import ProfilerHook
    hook = ProfilerHook(wait=0, warmup=1, active=1, repeat=1, output_dir=str(tmp_path))
    assert callable(hook.get_trace_handler())
    x = torch.randn(64, 64)
    for step in range(4):
        (x @ x).sum()
        hook.after_step({}, step)
    hook.end()
    traces = [f for f in os.listdir(tmp_path) if f.endswith(".json")]
    assert len(traces) == 1 and "-timeline-" in traces[0] and os.path.getsize(tmp_path / traces[0]) > 100
    assert hook.traces == [str(tmp_path / traces[0])]


def test_profiler_hook_puts_traces_through_fsspec_for_url_output_dirs():
    """An output directory given as a URL: the trace is exported locally and put through the URL's file system."""
    import fsspec
    from recis_b200.hooks import ProfilerHook
    hook = ProfilerHook(wait=0, warmup=1, active=1, repeat=1, output_dir="memory://traces/job7")
    x = torch.randn(32, 32)
    for step in range(4):
        (x @ x).sum()
        hook.after_step({}, step)
    hook.end()
    fs = fsspec.filesystem("memory")
    files = fs.ls("/traces/job7", detail=False)
    assert len(files) == 1 and files[0].endswith(".json") and "-timeline-" in files[0] and fs.size(files[0]) > 100
    assert hook.traces == [files[0]]
    fs.rm("/traces", recursive=True)


def test_prefetch_dataset_order_errors_and_early_exit():
    import threading
    import time
    from recis_b200.io import PrefetchDataset, TensorDataset
    src = TensorDataset({"a": torch.arange(20)}, batch_size=3)
    assert [b["a"].tolist() for b in PrefetchDataset(src, depth=2)] == [b["a"].tolist() for b in src]

    class Broken:
        def __iter__(self):
            yield {"a": torch.zeros(1)}
            raise OSError("disk went away")
    with pytest.raises(OSError, match="disk went away"):
        list(PrefetchDataset(Broken(), depth=2))
    # a consumer that stops early does not leave the producer thread behind
    before = threading.active_count()
    it = iter(PrefetchDataset(src, depth=1))
    next(it)
    it.close()
    deadline = time.time() + 5
    while threading.active_count() > before and time.time() < deadline:
        time.sleep(0.05)
    assert threading.active_count() <= before


def test_small_helpers_filesystem_logger_pad_info_initializers(tmp_path, capsys):
    from recis_b200.framework.filesystem import get_file_system
    from recis_b200.nn.initializers import KaimingNormalInitializer, KaimingUniformInitializer, XavierNormalInitializer, XavierUniformInitializer
    from recis_b200.ragged.tensor import RaggedPadInfo
    from recis_b200.utils.logger import Logger
    fs = get_file_system(str(tmp_path / "x"))
    with fs.open(str(tmp_path / "x"), "w") as fh:
        fh.write("hello")
    assert fs.exists(str(tmp_path / "x")) and get_file_system("file:///tmp").protocol[0] in ("file", "local")
    log = Logger("helper_test")
    log.error_rank0("an error line")
    log.info_rank0("an info line")
    out = capsys.readouterr()
    assert "an error line" in out.err and "an info line" in out.out          # INFO to stdout, the rest to stderr
    pad = RaggedPadInfo(torch.tensor([1]), torch.tensor([2]), torch.tensor([True]), torch.tensor([False]))
    assert int(pad.drop_nums[0]) == 1 and int(pad.pad_nums[0]) == 2 and "RaggedPadInfo" in repr(pad)
    # fan-based initializers: the standard deviation follows the fan of the [block, dim] shape they are built for
    for cls, want in ((XavierUniformInitializer, (2.0 / (1024 + 64)) ** 0.5), (XavierNormalInitializer, (2.0 / (1024 + 64)) ** 0.5)):
        init = cls()
        init.set_shape([1024, 64])
        init.build()
        e = init.generate()
        assert e.shape == (1024, 64) and abs(float(e.std()) - want) < 0.15 * want
    for cls in (KaimingUniformInitializer, KaimingNormalInitializer):
        init = cls()
        init.set_shape([1024, 64])
        init.build()
        assert 0 < float(init.generate().std()) < 1


def test_trainer_runs_every_epoch_over_the_whole_dataset(tmp_path):
    """``train_epoch=3``: the dataset is iterated three times (an exhausted dataset starts over on the next ``iter``)."""
    HashtableRegister().clear()
    torch.manual_seed(0)
    fields, spec = _spec(batch=32)
    model = DeepFM(fields, device="cpu", compute_dtype=torch.float32, hidden=(16,))

    class LossOnly(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, batch):
            return self.m(batch)[0]

    class Count(Hook):
        steps, epochs = 0, 0

        def after_step(self, metrics=None, global_step=0):
            Count.steps += 1

        def after_epoch(self):
            Count.epochs += 1

    ds = SyntheticDataset(spec, steps=4)
    args = TrainingArguments(output_dir=str(tmp_path), train_epoch=3, train_steps=None, save_steps=1000, log_steps=100)
    trainer = Trainer(model=LossOnly(model), args=args, train_dataset=ds, dense_optimizers=(torch.optim.Adam(model.parameters(), lr=1e-3), None),
                      sparse_optimizer=SparseAdagrad(filter_out_sparse_param(model), lr=0.01), hooks=[Count()])
    trainer.train()
    assert Count.epochs == 3 and Count.steps == 12


def test_trainer_gradient_accumulation_averages_dense_and_sparse_alike(tmp_path):
    """Two micro-batches with accumulation 2 == one step on the mean loss of the two, for dense weights AND embedding rows."""
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.optim import SparseSGD

    class Tiny(torch.nn.Module):
        def __init__(self, name):
            super().__init__()
            self.emb = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name=name, device="cpu", initializer=NormalInitializer(0, 0.1))})
            self.lin = torch.nn.Linear(4, 1)

        def forward(self, batch):
            return self.lin(self.emb({"a": batch["a"]})["a"]).square().mean()

    batches = [{"a": torch.tensor([[1], [2], [3]])}, {"a": torch.tensor([[3], [4], [5]])}]

    def run(accum, name):
        HashtableRegister().clear()
        torch.manual_seed(0)
        m = Tiny(name)
        sopt = SparseSGD(filter_out_sparse_param(m), lr=0.5)
        dopt = torch.optim.SGD(m.lin.parameters(), lr=0.5)
        if accum == 1:
            sopt.zero_grad(); dopt.zero_grad()
            (sum(m(b) for b in batches) / 2).backward()
            sopt.step(); dopt.step()
        else:
            args = TrainingArguments(output_dir=str(tmp_path / name), gradient_accumulation_steps=2, train_steps=2, save_steps=1000)
            Trainer(model=m, args=args, train_dataset=list(batches), dense_optimizers=(dopt, None), sparse_optimizer=sopt).train()
        (t,) = m.emb.tables().values()
        keys, rows = t.impl.ids_map()
        e = t.impl.store.emb()[rows]
        return m.lin.weight.detach().clone(), {int(k): e[i].clone() for i, k in enumerate(keys.tolist())}

    (w1, e1), (w2, e2) = run(1, "ga_one"), run(2, "ga_two")
    assert torch.allclose(w1, w2, atol=1e-6)
    assert e1.keys() == e2.keys() and all(torch.allclose(e1[k], e2[k], atol=1e-6) for k in e1)


def test_final_save_of_an_interval_step_is_listed_once(tmp_path):
    trainer, _model = _build(tmp_path, steps=10, save_steps=5)       # step 10 is saved by the interval and again at the end
    trainer.train()
    assert open(tmp_path / "checkpoint").read().split() == ["ckpt_5", "ckpt_10"]


def test_filter_hook_without_a_model_finds_the_tables_itself():
    """``HashTableFilterHook(filter_interval=n)`` with no model, as the reference is used: the live tables' filters are found
    through the hook factory's registry; a table that is gone drops out of it."""
    import gc
    from recis_b200.nn import HashTable
    from recis_b200.nn.hashtable_hook import FilterHook
    from recis_b200.nn.modules.hashtable_hook_impl import HashtableHookFactory
    HashtableRegister().clear()
    ht = HashTable([4], name="ttl_registry", device="cpu", filter_hook=FilterHook("GlobalStepFilter", {"filter_step": 3}))
    assert "ttl_registry" in HashtableHookFactory().get_filters()
    hook = HashTableFilterHook(filter_interval=2)
    ht(torch.arange(50))
    for step in range(8):
        ht(torch.arange(5))
        hook.after_step({}, step)
    assert ht.impl.size() == 5 and hook.evicted >= 45
    del ht, hook
    gc.collect()
    assert "ttl_registry" not in HashtableHookFactory().get_filters()


def test_jobs_that_span_machines_do_not_use_peer_memory(monkeypatch):
    from recis_b200.parallel.symmetric import single_node
    monkeypatch.delenv("LOCAL_WORLD_SIZE", raising=False)
    assert single_node(8)                                   # ranks spawned by hand on one machine
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    assert single_node(8) and not single_node(16)           # 2 machines x 8 ranks


def test_packed_batch_round_trip_and_prefetcher():
    """A packed host batch (one buffer for all tensors) unpacks to the same batch, directly and through the prefetcher."""
    from recis_b200.io import DevicePrefetcher, PackedBatch, SparseFieldSpec, SyntheticSpec, make_batch
    from recis_b200.ragged import RaggedTensor
    spec = SyntheticSpec(batch=16, dense_dim=5, label_rate=0.3, seed=3,
                         sparse=[SparseFieldSpec(f, zipf_a=1.1, id_bits=20, universe=500, length="poisson", mean_len=3) for f in ("a", "b")])
    batches = [make_batch(spec, i) for i in range(3)]
    batches[1]["w"] = RaggedTensor(torch.arange(6), [torch.tensor([0, 2, 6], dtype=torch.int32)], weight=torch.rand(6))
    batches[1]["note"] = "not a tensor"
    packed = [PackedBatch(b, pin=False) for b in batches]

    def same(x, y):
        if isinstance(x, RaggedTensor):
            assert torch.equal(x.values(), y.values()) and all(torch.equal(a, b) for a, b in zip(x.offsets(), y.offsets()))
            assert (x.weight() is None) == (y.weight() is None) and (x.weight() is None or torch.equal(x.weight(), y.weight()))
            assert x._dense_shape == y._dense_shape
        elif isinstance(x, torch.Tensor):
            assert x.dtype == y.dtype and torch.equal(x, y)
        else:
            assert x == y
    for b, p in zip(batches, packed):
        assert p.payload_bytes <= p.nbytes
        got = p.to("cpu")
        assert list(got) == list(b)
        for k in b:
            same(got[k], b[k])
    for b, got in zip(batches, DevicePrefetcher(packed, "cpu")):
        for k in b:
            same(got[k], b[k])


def test_async_scalar_reader_returns_every_posted_value():
    """Tickets come back with the value posted, in any order within the ring, on the host path (the CUDA path is in the GPU tests)."""
    from recis_b200.utils import AsyncScalarReader
    r = AsyncScalarReader("cpu", slots=4)
    t = [r.post(torch.tensor(float(i) * 0.5)) for i in range(4)]
    assert [r.get(k) for k in reversed(t)] == [1.5, 1.0, 0.5, 0.0]
    t5 = r.post(torch.tensor(7.0))
    assert r.get(t5) == 7.0
    with pytest.raises(AssertionError):
        r.get(t[0])


def test_bf16_weight_copy_bookkeeping_follows_versions_and_storage():
    """The kept bf16 copy of a weight is valid only for the same storage and version counter (the CUDA kernels that use it are
    covered by the GPU tests; the bookkeeping is plain Python)."""
    from recis_b200.ops.dense import bf16_shadow, keep_bf16_shadow
    w = torch.nn.Parameter(torch.randn(8, 16))
    assert bf16_shadow(w) is None
    keep_bf16_shadow(w, w.detach().to(torch.bfloat16))
    assert bf16_shadow(w) is not None
    with torch.no_grad():
        w.add_(1.0)                                   # an in-place change through torch bumps the version counter
    assert bf16_shadow(w) is None
    keep_bf16_shadow(w, w.detach().to(torch.bfloat16))
    w.data = torch.randn(8, 16)                       # new storage under the same Parameter object
    assert bf16_shadow(w) is None


def test_dense_reducer_single_rank_applies_the_accumulation_scale():
    """With one rank there is nothing to reduce, but the division by the accumulation count still happens in the reducer."""
    from recis_b200.parallel import DenseGradReducer
    lin = torch.nn.Linear(4, 3)
    red = DenseGradReducer(list(lin.parameters()), world=1)
    red.grad_scale = 0.5
    for _ in range(2):
        lin(torch.ones(2, 4)).sum().backward()
    red.all_reduce_async()
    red.wait()
    assert torch.allclose(lin.bias.grad, torch.full((3,), 2.0))       # (2 + 2) * 0.5
    assert lin.weight.grad.data_ptr() == red.flat[:0].data_ptr() or lin.weight.grad.untyped_storage().data_ptr() == red.flat.untyped_storage().data_ptr()
