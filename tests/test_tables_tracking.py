"""Row-addressable tables, time-addressable streams and their windowed datasets; sample-level trace tables; experiment tracking;
the model store. All on CPU: the services of the reference's internal build are replaced by files and by fakes registered as
sources."""
import json
import os

import numpy as np
import pyarrow as pa
import pyarrow.dataset as pads
import pyarrow.orc as orc
import pyarrow.parquet as pq
import pytest
import torch

from recis_b200.io import (OdpsDataset, get_table_size, make_lake_stream_window_io, make_odps_sample_io, make_odps_window_io,
                           register_table_source)
from recis_b200.io.window_io import (TableSheet, _build_shard, _parse_proportion, _shard_sheets_by_row_num, _shard_table_by_subprocess,
                                     _str_to_timestamp)


def _write_table(dirname, base, nfiles, rows):
    os.makedirs(dirname, exist_ok=True)
    r = base
    for i in range(nfiles):
        t = pa.table({"uid": pa.array(np.arange(r, r + rows), pa.int64()),
                      "items": pa.array([[int(x), int(x) + 1] for x in range(r, r + rows)], pa.list_(pa.int64())),
                      "score": pa.array(np.arange(r, r + rows, dtype=np.float64))})
        if i % 2 == 0:
            pq.write_table(t, f"{dirname}/part-{i:03d}.parquet")
        else:
            orc.write_table(t, f"{dirname}/part-{i:03d}.orc")
        r += rows


# ------------------------------------------------------------------------------------------------------------ sharding math
def test_build_shard_spreads_the_surplus():
    shards, off = _build_shard(0, 100, 3)
    assert shards == [(0, 34), (34, 67), (67, 100)] and off == 1
    shards, off = _build_shard(100, 100, 3, off)          # the longer shard moves on
    assert [e - s for s, e in shards] == [33, 34, 33] and shards[0][0] == 100 and shards[-1][1] == 200 and off == 2


def test_parse_proportion():
    assert _parse_proportion(6, [(2, 3), (1, 3)]) == ([4, 2], 6)
    assert _parse_proportion(4, [(1, 1)]) == ([4], 4)
    with pytest.raises(ValueError):
        _parse_proportion(4, [(1, 2), (1, 3)])
    with pytest.raises(ValueError):
        _parse_proportion(4, [(2, 3), (2, 3)])


def test_subprocess_shares_cover_each_sheet():
    sheets = [TableSheet("t", 0, 10), TableSheet("t", 10, 17)]
    parts = [_shard_table_by_subprocess(sheets, i, 3) for i in range(3)]
    for k, sh in enumerate(sheets):
        rows = []
        for p in parts:
            s = TableSheet.parse(p[k])
            rows += list(range(s.start, s.end))
        assert rows == list(range(sh.start, sh.end))


def test_row_num_sheets_partition_the_table(tmp_path):
    _write_table(str(tmp_path / "t"), 0, 3, 111)
    rows = []
    for w in range(2):
        sheets, _ = _shard_sheets_by_row_num(str(tmp_path / "t"), w, 2, 2, 50, 0)
        for s in sheets:
            rows += list(range(s.start, s.end))
    assert sorted(rows) == list(range(333))


# ------------------------------------------------------------------------------------------------------------ table dataset
def test_table_dataset_reads_every_row_once_across_workers(tmp_path):
    table = str(tmp_path / "t1")
    _write_table(table, 0, 4, 250)
    assert get_table_size(table) == 1000
    seen = []
    for w in range(2):
        ds = OdpsDataset(64, worker_idx=w, worker_num=2, read_threads_num=2)
        ds.add_path(table)
        ds.varlen_feature("items")
        ds.fixedlen_feature("uid")
        ds.fixedlen_feature("score")
        for b in ds:
            uid = b["uid"].flatten()
            assert torch.equal(b["items"].values().view(-1, 2)[:, 0], uid) and torch.equal(b["score"].flatten().long(), uid)
            seen += uid.tolist()
    assert sorted(seen) == list(range(1000))


def test_table_dataset_resumes_from_io_state(tmp_path):
    table = str(tmp_path / "t1")
    _write_table(table, 0, 2, 300)

    def make():
        ds = OdpsDataset(50, read_threads_num=2)
        ds.add_path(table)
        ds.fixedlen_feature("uid")
        return ds

    full = [b["uid"].flatten().tolist() for b in make()]
    ds = make()
    it = iter(ds)
    head = [next(it)["uid"].flatten().tolist() for _ in range(4)]
    state = ds.dump_io_state()
    ds2 = make()
    ds2.load_io_state(state)
    tail = [b["uid"].flatten().tolist() for b in ds2]
    assert head + tail == full


def test_registered_source_stands_in_for_a_table_service():
    class FakeService:
        def __init__(self):
            self.calls = []

        def size(self, table):
            return 500

        def read(self, table, start, end, columns):
            self.calls.append((table, start, end))
            return pa.table({"uid": pa.array(np.arange(start, end), pa.int64())}).select(columns)

    svc = FakeService()
    register_table_source("faketables", svc)
    ds = OdpsDataset(128, worker_idx=1, worker_num=2, read_threads_num=1)
    ds.add_path("faketables://proj.clicks")
    ds.fixedlen_feature("uid")
    rows = torch.cat([b["uid"].flatten() for b in ds]).tolist()
    assert rows == list(range(250, 500)) and all(c[0] == "proj.clicks" for c in svc.calls)


# ---------------------------------------------------------------------------------------------------------------- windows
def test_window_io_mixes_tables_in_proportion_and_reads_all(tmp_path):
    t1, t2 = str(tmp_path / "t1"), str(tmp_path / "t2")
    _write_table(t1, 0, 4, 250)
    _write_table(t2, 100000, 2, 250)
    ds = make_odps_window_io(split_num=4)(90, read_threads_num=3)
    ds.add_path(t1, (2, 3))
    ds.add_path(t2, (1, 3))
    ds.fixedlen_feature("uid")
    got, windows, shares = [], 0, []
    while True:
        try:
            if ds.next_window():
                continue
        except StopIteration:
            break
        windows += 1
        for b in ds:
            u = b["uid"].flatten()
            got += u.tolist()
            if len(u) == 90:
                shares.append(float((u < 100000).float().mean()))
    assert windows == 4 and sorted(got) == list(range(1000)) + list(range(100000, 100500))
    assert shares and all(abs(s - 2 / 3) < 1e-6 for s in shares)
    ds.reset()
    assert ds.next_window() is False


def test_window_io_state_resumes_at_the_next_window(tmp_path):
    table = str(tmp_path / "t")
    _write_table(table, 0, 2, 200)

    def make():
        ds = make_odps_window_io(row_num=100)(32, read_threads_num=2)
        ds.add_path(table)
        ds.fixedlen_feature("uid")
        return ds

    def drain(ds, limit=None):
        out, n = [], 0
        while limit is None or n < limit:
            try:
                if ds.next_window():
                    continue
            except StopIteration:
                break
            out.append(sorted(torch.cat([b["uid"].flatten() for b in ds]).tolist()))
            n += 1
        return out

    full = drain(make())
    assert sorted(sum(full, [])) == list(range(400))
    a = make()
    first = drain(a, 2)
    b = make()
    b.load_state_dict(a.state_dict())
    assert first + drain(b) == full
    with pytest.raises(ValueError):
        make_odps_window_io(split_num=2, row_num=10)
    with pytest.raises(ValueError):
        make_odps_window_io()


def test_sample_io_reads_one_contiguous_sample(tmp_path):
    table = str(tmp_path / "t")
    _write_table(table, 0, 2, 500)
    ds = make_odps_sample_io(row_num=100, seed=3)(32, read_threads_num=2)
    ds.add_path(table)
    ds.fixedlen_feature("uid")
    assert ds.next_window() is False
    u = torch.cat([b["uid"].flatten() for b in ds])
    assert len(u) == 100 and int(u.max() - u.min()) == 99
    with pytest.raises(StopIteration):
        ds.next_window()


def test_stream_window_moves_forward_in_time(tmp_path):
    stream = str(tmp_path / "stream")
    for hh in range(4):
        _write_table(f"{stream}/20250101{hh:02d}00", hh * 1000, 1, 100)
    ds = make_lake_stream_window_io(step_mins=60, repeat_mins=60)(64)
    ds.add_path(stream, _str_to_timestamp("20250101000000"), 120)
    ds.fixedlen_feature("uid")
    spans = []
    for _ in range(5):
        empty = ds.next_window()
        u = [] if empty else torch.cat([b["uid"].flatten() for b in ds]).tolist()
        spans.append((empty, len(u), (min(u), max(u)) if u else None))
    assert spans[0] == (False, 200, (0, 1099)) and spans[1] == (False, 200, (1000, 2099)) and spans[3] == (False, 100, (3000, 3099))
    assert spans[4] == (True, 0, None)                  # no data there yet: an empty window, not the end of the stream
    # two workers split a window's entries between them
    parts = []
    for w in range(2):
        d2 = make_lake_stream_window_io(step_mins=60)(64, worker_idx=w, worker_num=2)
        d2.add_path(stream, _str_to_timestamp("20250101000000"), 240)
        d2.fixedlen_feature("uid")
        assert d2.next_window() is False
        parts.append(torch.cat([b["uid"].flatten() for b in d2]).tolist())
    assert sorted(parts[0] + parts[1]) == sorted(sum([list(range(h * 1000, h * 1000 + 100)) for h in range(4)], []))
    assert parts[0] and parts[1]


# ------------------------------------------------------------------------------------------------------------- trace table
def test_trace_hook_writes_the_declared_table(tmp_path):
    from recis_b200.hooks import TraceToOdpsHook, add_to_trace
    import recis_b200.hooks.trace_to_odps_hook as same_module
    assert same_module.TraceToOdpsHook is TraceToOdpsHook
    out = str(tmp_path / "trace")
    hook = TraceToOdpsHook({"output_dir": out, "partition": "dt=20250101,hh=10"}, ["uid", "score", "emb", "tag"],
                           ["bigint", "double", "array<float>", "string"], worker_num=2, size_threshold=1000)
    for s in range(5):
        add_to_trace("uid", torch.arange(8) + s * 8)
        add_to_trace("score", np.arange(8, dtype=np.float64) + s * 8)
        add_to_trace("emb", (torch.arange(32).view(8, 4) + s).bfloat16())
        add_to_trace("tag", [f"t{i}" for i in range(8)])
        hook.after_step()
    hook.end()
    t = pads.dataset(os.path.join(out, "dt=20250101", "hh=10"), format="parquet").to_table().sort_by("uid")
    assert t.num_rows == 40 == hook.rows_written and t.schema.names == ["uid", "score", "emb", "tag"]
    assert t["uid"].to_pylist() == list(range(40)) and t["score"].to_pylist() == [float(i) for i in range(40)]
    assert t.schema.field("emb").type == pa.list_(pa.float32()) and t["emb"][9].as_py() == [5.0, 6.0, 7.0, 8.0]
    assert not [f for f in os.listdir(os.path.join(out, "dt=20250101", "hh=10")) if f.endswith(".tmp")]


def test_trace_hook_reports_a_failing_writer(tmp_path):
    from recis_b200.hooks.trace_hook import TraceToOdpsHook, add_to_trace, clear_trace_map

    class BrokenSink:
        def write_block(self, table):
            raise IOError("sink is down")

        def commit(self):
            pass

    import recis_b200.hooks.trace_hook as th
    hook = TraceToOdpsHook({"sink": BrokenSink()}, ["uid"], ["bigint"], size_threshold=1)
    for w in hook.writers:                       # no ten-second pauses between the retries in a test
        w._write_block = lambda table, _w=w: _w.sink.write_block(table)
    add_to_trace("uid", [1, 2, 3])
    hook.after_step()
    for w in hook.writers:
        w.join(timeout=10)
    add_to_trace("uid", [4])
    with pytest.raises(ValueError):
        hook.after_step()
    clear_trace_map()
    with pytest.raises(ValueError):
        th.add_to_trace("x", 3.0)                # only tensors, arrays and lists are rows


def test_trace_rejects_ragged_row_counts():
    from recis_b200.hooks.trace_hook import rows_to_table
    with pytest.raises(ValueError):
        rows_to_table({"a": [1, 2, 3], "b": [1.0]}, ["a", "b"], ["bigint", "double"])
    with pytest.raises(KeyError):
        rows_to_table({"a": [1]}, ["a", "b"], ["bigint", "double"])


@pytest.mark.gpu
def test_trace_takes_device_tensors_without_blocking():
    from recis_b200.hooks.trace_hook import add_to_trace, clear_trace_map, get_trace_map
    x = torch.arange(1 << 16, device="cuda", dtype=torch.float32)
    add_to_trace("x", x * 2)
    got = get_trace_map()["x"]
    assert isinstance(got, np.ndarray) and got[-1] == 2.0 * ((1 << 16) - 1)
    clear_trace_map()


# --------------------------------------------------------------------------------------------------------------- tracking
def test_ml_tracker_hook_logs_steps_to_files(tmp_path):
    from recis_b200.hooks import MLTrackerHook, add_to_ml_tracker
    hook = MLTrackerHook("proj", "run", {"lr": 0.1, "layers": [512, 256]}, id="a1", root=str(tmp_path), log_metrics=True)
    for step in range(3):
        add_to_ml_tracker("loss", torch.tensor(0.5 / (step + 1)))
        add_to_ml_tracker("hist", np.arange(3))
        hook.after_step({"auc": 0.7 + step / 10}, step)
    hook.end()
    run = tmp_path / "proj" / "run-a1"
    lines = [json.loads(l) for l in open(run / "metrics.jsonl")]
    assert [l["step"] for l in lines] == [0, 1, 2] and lines[1]["loss"] == 0.25 and lines[2]["hist"] == [0, 1, 2]
    assert abs(lines[2]["auc"] - 0.9) < 1e-9
    cfg = json.load(open(run / "config.json"))
    assert cfg["config"] == {"lr": 0.1, "layers": [512, 256]} and cfg["id"] == "a1"
    assert json.load(open(run / "finished"))["steps"] == 3


# ------------------------------------------------------------------------------------------------------------ model store
def test_model_uri_parsing():
    from recis_b200.utils.mos import parse_uri
    assert parse_uri("model.rec.user_emb")["level"] == "model"
    v = parse_uri("model.rec.user_emb/version=v1")
    assert (v["level"], v["project"], v["model_name"], v["version"], v["ckpt_id"]) == ("version", "rec", "user_emb", "v1", None)
    c = parse_uri("model.rec.user_emb/version=v1/ckpt_id=ckpt_10")
    assert (c["level"], c["ckpt_id"]) == ("ckpt_id", "ckpt_10")
    assert parse_uri("model.rec.user_emb/version=dt_max_pt/ckpt_id=x")["level"] == "version"
    auto = parse_uri("model.rec.user_emb", auto_version=True)
    assert len(auto["version"]) == 14 and auto["uri"].endswith("/version=" + auto["version"])
    for bad in ("rec.user_emb", "model.rec", "model.rec.user emb", ""):
        with pytest.raises(ValueError):
            parse_uri(bad)


def test_checkpoints_saved_under_a_model_uri_load_back_as_model_bank(tmp_path, monkeypatch):
    from recis_b200.framework.checkpoint_manager import CheckpointManager, Saver
    from recis_b200.utils.mos import Mos
    monkeypatch.setenv("RECIS_MODEL_STORE", str(tmp_path / "store"))
    torch.manual_seed(0)
    model = torch.nn.Linear(4, 3)
    saver = Saver(model, output_dir="model.rec.tower/version=v7", max_keep=2)
    assert saver._output_dir == str(tmp_path / "store" / "rec" / "tower" / "version=v7")
    for step in (10, 20, 30):
        with torch.no_grad():
            model.weight.fill_(float(step))
        saver.save(f"ckpt_{step}")
    store = Mos("model.rec.tower/version=v7", model_bank_path=True)
    assert store.list_ckpts() == ["ckpt_20", "ckpt_30"] and store.real_physical_path.endswith("ckpt_30")
    assert Mos("model.rec.tower", True).uri_info["version"] == "v7"                  # newest version, newest checkpoint
    assert Mos("model.rec.tower/version=v7/ckpt_id=ckpt_20", True).real_physical_path.endswith("ckpt_20")
    with pytest.raises(FileNotFoundError):
        Mos("model.rec.tower/version=v7/ckpt_id=ckpt_10", True)                      # removed by max_keep, and forgotten
    other = torch.nn.Linear(4, 3)
    mgr = CheckpointManager(Saver(other, output_dir=str(tmp_path / "elsewhere")), save_interval=100)
    mgr.load_model_bank([{"path": "model.rec.tower/version=v7/ckpt_id=ckpt_20", "load": ["dense"]}])
    assert float(other.weight.detach()[0, 0]) == 20.0


def test_info_module_matches_the_reference_names():
    import recis_b200.__info__ as info
    assert info.is_internal_enabled() == 0 and isinstance(info.INTERVAL_VERSION, str)


def test_table_export_to_orc_shards_round_trips(tmp_path):
    from recis_b200.io import OrcDataset
    from recis_b200.io.table_to_orc import main
    table = str(tmp_path / "t")
    _write_table(table, 0, 3, 100)
    out = str(tmp_path / "out")
    main(["--table", table, "--output", out, "--nfiles", "4", "--threads", "2"])
    files = sorted(os.listdir(out))
    assert files == [f"part-{i:05d}.orc" for i in range(4)]
    ds = OrcDataset(64, native_reader=False)
    ds.add_paths([os.path.join(out, f) for f in files])
    ds.fixedlen_feature("uid")
    ds.varlen_feature("items")
    rows = torch.cat([b["uid"].flatten() for b in ds]).tolist()
    assert rows == list(range(300))


# ------------------------------------------------------------------------------------------------- trainer over windows
def _window_trainer(tmp_path, table, out, seen, train_steps=None, hooks=()):
    from recis_b200.framework.trainer import Trainer, TrainingArguments
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
    from recis_b200.nn.modules.hashtable import HashtableRegister
    from recis_b200.nn.initializers import ConstantInitializer
    from recis_b200.optim import SparseAdagrad
    HashtableRegister().clear()
    torch.manual_seed(0)

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = EmbeddingEngine({"items": EmbeddingOption(embedding_dim=4, shared_name="items", device="cpu", combiner="sum",
                                                                 initializer=ConstantInitializer(0.1))})
            self.head = torch.nn.Linear(4, 1)

        def forward(self, batch):
            seen.extend(batch["uid"].flatten().tolist())
            e = self.emb({"items": batch["items"]})["items"]
            return (self.head(e).squeeze(-1) - batch["score"].flatten() * 1e-3).pow(2).mean()

    ds = make_odps_window_io(row_num=100)(32, read_threads_num=2)
    ds.add_path(table)
    ds.varlen_feature("items")
    ds.fixedlen_feature("uid")
    ds.fixedlen_feature("score")
    model = Model()
    args = TrainingArguments(output_dir=out, train_steps=train_steps, save_steps=1000, log_steps=1000)
    return Trainer(model=model, args=args, train_dataset=ds, dense_optimizers=(torch.optim.SGD(model.head.parameters(), lr=1e-3), None),
                   sparse_optimizer=SparseAdagrad(filter_out_sparse_param(model), lr=0.01), hooks=list(hooks)), ds


def test_trainer_walks_every_window_and_resumes_at_the_next_one(tmp_path):
    table = str(tmp_path / "t")
    _write_table(table, 0, 2, 200)
    seen = []
    trainer, ds = _window_trainer(tmp_path, table, str(tmp_path / "run_all"), seen)
    trainer.train()
    assert sorted(seen) == list(range(400))                          # four windows of 100 rows, every row once

    # stop after the first window's batches; the checkpoint carries the window position
    first = []
    trainer, ds = _window_trainer(tmp_path, table, str(tmp_path / "run_split"), first, train_steps=4)
    trainer.train()
    assert sorted(first) == list(range(100)) and int(ds.state_dict()["read_offset"][0]) == 2
    rest = []
    trainer, ds = _window_trainer(tmp_path, table, str(tmp_path / "run_split"), rest)
    trainer.train()
    assert sorted(rest) == list(range(100, 400))


def test_trainer_traces_and_tracks_through_hooks(tmp_path):
    from recis_b200.hooks import Hook, MLTrackerHook, TraceToOdpsHook, add_to_ml_tracker, add_to_trace
    table = str(tmp_path / "t")
    _write_table(table, 0, 1, 128)
    seen = []

    class Name(Hook):
        """Names the step's values before the trace and tracker hooks (registered after it) collect them."""
        done = 0

        def after_step(self, metrics=None, global_step=0):
            rows = seen[Name.done:]                       # this step's samples
            Name.done = len(seen)
            add_to_trace("uid", rows)
            add_to_trace("loss", [float(metrics["loss"])] * len(rows))
            add_to_ml_tracker("loss", metrics["loss"])

    hooks = [Name(), TraceToOdpsHook({"output_dir": str(tmp_path / "trace")}, ["uid", "loss"], ["bigint", "double"]),
             MLTrackerHook("p", "r", {}, id="1", root=str(tmp_path / "track"))]
    trainer, _ = _window_trainer(tmp_path, table, str(tmp_path / "run"), seen, hooks=hooks)
    trainer.train()
    t = pads.dataset(str(tmp_path / "trace"), format="parquet").to_table()
    assert sorted(t["uid"].to_pylist()) == list(range(128))
    lines = [json.loads(l) for l in open(tmp_path / "track" / "p" / "r-1" / "metrics.jsonl")]
    assert len(lines) == 5 and all("loss" in l for l in lines)          # windows of 100 and 28 rows: 4 + 1 batches of up to 32


# ------------------------------------------------------------------------------------------ checkpoints on a remote file system
def test_checkpoints_on_a_remote_file_system_round_trip(tmp_path, monkeypatch):
    import fsspec
    from recis_b200.framework.checkpoint_manager import CheckpointManager, Saver
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.nn.modules.hashtable import HashtableRegister
    from recis_b200.ragged import RaggedTensor
    import recis_b200.framework.checkpoint_manager as cm
    fs = fsspec.filesystem("memory")
    url = "memory://ckpts/run1"

    def build(stage):
        monkeypatch.setattr(cm, "_STAGING", str(tmp_path / stage))
        os.makedirs(tmp_path / stage, exist_ok=True)
        HashtableRegister().clear()
        torch.manual_seed(0)

        class M(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.emb = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu", initializer=NormalInitializer(0, 1))})
                self.head = torch.nn.Linear(4, 1)

        return M()

    ids = RaggedTensor(torch.arange(20, dtype=torch.int64), [torch.arange(21, dtype=torch.int32)])
    m = build("stage_a")
    rows = m.emb({"a": ids})["a"].detach().clone()
    saver = Saver(m, output_dir=url, max_keep=2)
    for step in (1, 2, 3):
        with torch.no_grad():
            m.head.weight.fill_(float(step))
        saver.save(f"ckpt_{step}")
    assert fs.cat("/ckpts/run1/checkpoint").decode().split() == ["ckpt_2", "ckpt_3"]
    assert not fs.exists("/ckpts/run1/ckpt_1") and fs.exists("/ckpts/run1/ckpt_3/model.pt")
    assert any(f.endswith(".safetensors") for f in fs.ls("/ckpts/run1/ckpt_3", detail=False))

    # a fresh process (an empty staging directory) restores from the remote directory
    m2 = build("stage_b")
    mgr = CheckpointManager(Saver(m2, output_dir=url), save_interval=100)
    mgr.restore()
    assert float(m2.head.weight.detach()[0, 0]) == 3.0
    assert torch.equal(m2.emb({"a": ids})["a"].detach(), rows)
    # and an older checkpoint of it serves as a model bank for another model
    m3 = build("stage_c")
    CheckpointManager(Saver(m3, output_dir=str(tmp_path / "local_out")), 100).load_model_bank([{"path": url + "/ckpt_2", "load": ["dense"]}])
    assert float(m3.head.weight.detach()[0, 0]) == 2.0


def _register_shared_fs():
    """A second name for the local file system, so that child processes share a 'remote' directory the checkpoint code treats as
    remote (a URL that is not file://)."""
    import fsspec
    from fsspec.implementations.local import LocalFileSystem

    class SharedFS(LocalFileSystem):
        protocol = "sharedtest"

        @classmethod
        def _strip_protocol(cls, path):
            path = str(path)
            return super()._strip_protocol(path[len("sharedtest://"):] if path.startswith("sharedtest://") else path)

    fsspec.register_implementation("sharedtest", SharedFS, clobber=True)


def _remote_ckpt_ranks_fn(rank, world, remote_dir, stage_dir):
    import torch
    import recis_b200.framework.checkpoint_manager as cm
    from recis_b200.framework.checkpoint_manager import CheckpointManager, Saver
    from recis_b200.nn import EmbeddingEngine, EmbeddingOption
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.nn.modules.hashtable import HashtableRegister
    from recis_b200.ragged import RaggedTensor
    _register_shared_fs()
    url = "sharedtest://" + remote_dir

    def build():
        HashtableRegister().clear()
        torch.manual_seed(3)

        class M(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.emb = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu", initializer=NormalInitializer(0, 1))})
                self.head = torch.nn.Linear(4, 1)

        return M()

    ids = RaggedTensor(torch.arange(40, dtype=torch.int64) * 7 + rank, [torch.arange(41, dtype=torch.int32)])
    cm._STAGING = os.path.join(stage_dir, f"save_rank{rank}")
    os.makedirs(cm._STAGING, exist_ok=True)
    m = build()
    rows = m.emb({"a": ids})["a"].detach().clone()
    with torch.no_grad():
        m.head.weight.fill_(5.0)
    CheckpointManager(Saver(m, output_dir=url), save_interval=100).save()
    cm._STAGING = os.path.join(stage_dir, f"load_rank{rank}")          # as a fresh job: nothing staged locally
    os.makedirs(cm._STAGING, exist_ok=True)
    m2 = build()
    CheckpointManager(Saver(m2, output_dir=url), save_interval=100).restore()
    again = m2.emb({"a": ids})["a"].detach()
    return {"same_rows": bool(torch.equal(rows, again)), "weight": float(m2.head.weight.detach()[0, 0]),
            "remote": sorted(os.listdir(os.path.join(remote_dir, "ckpt_0")))}


def test_two_ranks_checkpoint_through_a_remote_directory(tmp_path):
    import sys
    sys.path.insert(0, os.path.dirname(__file__))
    from multirank import run_ranks
    remote, stage = str(tmp_path / "remote"), str(tmp_path / "stage")
    os.makedirs(remote)
    res = run_ranks(_remote_ckpt_ranks_fn, 2, "gloo", args=(remote, stage), env={"RECIS_COMM": "nccl"})
    assert all(r["same_rows"] and r["weight"] == 5.0 for r in res)
    files = res[0]["remote"]
    assert "model.pt" in files and "index" in files and sum(f.endswith(".safetensors") for f in files) >= 2
    assert open(os.path.join(remote, "checkpoint")).read().split() == ["ckpt_0"]


def test_trace_and_tracker_write_to_object_stores():
    """Stores without rename-in-place or append (here fsspec's in-memory one) get whole parts and a rewritten log."""
    import fsspec
    from recis_b200.hooks import MLTrackerHook, TraceToOdpsHook, add_to_ml_tracker, add_to_trace
    fs = fsspec.filesystem("memory")
    hook = TraceToOdpsHook({"output_dir": "memory://traces/run", "partition": "dt=1"}, ["uid"], ["bigint"], size_threshold=1)
    for s in range(3):
        add_to_trace("uid", [s * 2, s * 2 + 1])
        hook.after_step()
    hook.end()
    parts = [p for p in fs.ls("/traces/run/dt=1", detail=False) if p.endswith(".parquet")]
    rows = []
    for p in parts:
        with fs.open(p, "rb") as f:
            rows += pq.read_table(f)["uid"].to_pylist()
    assert len(parts) == 3 and sorted(rows) == list(range(6))
    tracker = MLTrackerHook("p", "r", {"k": 1}, id="7", root="memory://tracking")
    for step in range(3):
        add_to_ml_tracker("v", step * 1.5)
        tracker.after_step(None, step)
    tracker.end()
    lines = [json.loads(l) for l in fs.cat("/tracking/p/r-7/metrics.jsonl").decode().splitlines()]
    assert [l["v"] for l in lines] == [0.0, 1.5, 3.0] and fs.exists("/tracking/p/r-7/finished")


def test_window_sharding_covers_every_row_exactly_once_property():
    """For random table sizes, worker counts, thread counts and window settings: the sheets of all workers and windows partition
    the table, and the sub-process shares partition each sheet."""
    from hypothesis import given, settings, strategies as st
    import recis_b200.io.window_io as wio
    from recis_b200.io.window_io import _shard_sheets_by_split_num

    @settings(max_examples=150, deadline=None)
    @given(size=st.integers(0, 5000), workers=st.integers(1, 5), threads=st.integers(1, 4), split=st.integers(1, 6),
           row_num=st.integers(1, 700), subs=st.integers(1, 3))
    def check(size, workers, threads, split, row_num, subs):
        orig = wio.get_table_size
        wio.get_table_size = lambda table: size
        try:
            for sheets_of in (lambda w: _shard_sheets_by_split_num("t", w, workers, threads, split, 0)[0],
                              lambda w: _shard_sheets_by_row_num("t", w, workers, threads, row_num, 0)[0]):
                rows = []
                for w in range(workers):
                    sheets = sheets_of(w)
                    for sub in range(subs):
                        for text in _shard_table_by_subprocess(sheets, sub, subs):
                            s = TableSheet.parse(text)
                            assert s.start <= s.end
                            rows += range(s.start, s.end)
                assert sorted(rows) == list(range(size))
        finally:
            wio.get_table_size = orig

    check()


def test_reader_threads_keep_the_row_order(monkeypatch):
    """Several requests in flight, finishing out of order: batches still come in row order."""
    import time
    import recis_b200.io.window_io as wio

    class SlowFirst:
        def size(self, table):
            return 1000

        def read(self, table, start, end, columns):
            time.sleep(0.05 if start == 0 else 0.0)          # the first chunk is the slowest
            return pa.table({"uid": pa.array(np.arange(start, end), pa.int64())})

    register_table_source("slowfirst", SlowFirst())
    monkeypatch.setattr(wio, "_READ_CHUNK_ROWS", 100)
    ds = OdpsDataset(64, read_threads_num=4)
    ds.add_path("slowfirst://t")
    ds.fixedlen_feature("uid")
    rows = torch.cat([b["uid"].flatten() for b in ds]).tolist()
    assert sorted(rows) == list(range(1000))
    # four sheets of 250 rows, each read in order
    assert all(rows[i * 250:(i + 1) * 250] == list(range(i * 250, (i + 1) * 250)) for i in range(4))


def test_native_reader_serves_file_backed_sheets_and_resumes_anywhere(tmp_path):
    """Sheets over files go through the C++ reader (row ranges per file segment); rows, their order and every resume point agree
    with the Python path."""
    from recis_b200._ext_io import load
    if load() is None:
        pytest.skip("native reader not built here")
    table = str(tmp_path / "t")
    _write_table(table, 0, 5, 130)                     # 650 rows in five files: sheets cross file boundaries

    def make(native):
        ds = OdpsDataset(48, worker_idx=1, worker_num=2, read_threads_num=3, native_reader=native)
        ds.add_path(table)
        ds.varlen_feature("items")
        ds.fixedlen_feature("uid")
        return ds

    used = []
    ds = make(True)
    orig = ds._iter_native
    ds._iter_native = lambda sheets: (used.append(1), orig(sheets))[1]
    native_rows, states, native_sizes = [], [], []
    for b in ds:
        assert torch.equal(b["items"].values().view(-1, 2)[:, 0], b["uid"].flatten())
        native_rows += b["uid"].flatten().tolist()
        native_sizes.append(b["uid"].shape[0])
        states.append((len(native_rows), ds.dump_io_state()))
    python_batches = [b["uid"].flatten().tolist() for b in make(False)]
    python_rows = sum(python_batches, [])
    assert used and native_rows == python_rows and len(native_rows) == 325
    assert native_sizes == [len(b) for b in python_batches]          # the same batches, not only the same rows
    dropped = make(True)
    dropped.drop_remainder = True
    assert all(b["uid"].shape[0] == 48 for b in dropped)
    for seen, state in states[:-1][::2]:               # resume after every other batch, on either path (a finished pass starts over)
        for native in (True, False):
            d2 = make(native)
            d2.load_io_state(state)
            rest = [x for b in d2 for x in b["uid"].flatten().tolist()]
            assert native_rows[:seen] + rest == native_rows, (seen, native)


def test_native_reader_row_ranges_decode_only_what_overlaps(tmp_path):
    """Ranges that start and end inside Parquet row groups and ORC stripes give exactly their rows."""
    from recis_b200._ext_io import load
    mod = load()
    if mod is None:
        pytest.skip("native reader not built here")
    n = 20000
    t = pa.table({"uid": pa.array(np.arange(n), pa.int64()), "items": pa.array([[i, i + 1] for i in range(n)], pa.list_(pa.int64()))})
    pq_path, orc_path = str(tmp_path / "a.parquet"), str(tmp_path / "b.orc")
    pq.write_table(t, pq_path, row_group_size=1500)
    orc.write_table(t, orc_path, stripe_size=16 * 1024, batch_size=512)
    assert pq.ParquetFile(pq_path).metadata.num_row_groups > 5 and orc.ORCFile(orc_path).nstripes > 1
    for path in (pq_path, orc_path):
        for lo, hi in ((0, n), (1499, 1501), (1500, 3000), (4321, 17777), (19990, -1), (0, 1), (n, n + 5)):
            reader = mod.ColumnarReader([path, path], 700, [("items", -1, 0, False)], [("uid", 0.0)], 2, 2, False, False,
                                        ranges=[(lo, hi), (10, 12)])
            rows = []
            while True:
                item = reader.next()
                if item is None:
                    break
                count, cols = item
                uid = cols["uid"][1].flatten().long()
                assert count == len(uid) and torch.equal(cols["items"][1].view(-1, 2)[:, 0], uid)
                rows += uid.tolist()
            want = list(range(lo, n if hi < 0 else min(hi, n))) + [10, 11]
            assert rows == want, (path, lo, hi)


def test_ragged_concat_joins_rows_levels_and_weights():
    from recis_b200.ragged import RaggedTensor
    a = RaggedTensor(torch.tensor([1, 2, 3]), [torch.tensor([0, 2, 3], dtype=torch.int32)], weight=torch.tensor([.1, .2, .3]))
    b = RaggedTensor(torch.tensor([4]), [torch.tensor([0, 0, 1], dtype=torch.int32)], weight=torch.tensor([.4]))
    c = RaggedTensor.concat([a, b])
    assert c.values().tolist() == [1, 2, 3, 4] and c.offsets()[0].tolist() == [0, 2, 3, 3, 4] and c.get_shape(0) == 4
    assert torch.allclose(c.weight(), torch.tensor([.1, .2, .3, .4]))
    # two levels (rows -> strings -> bytes)
    s1 = RaggedTensor(torch.arange(5, dtype=torch.int8), [torch.tensor([0, 1, 2], dtype=torch.int32), torch.tensor([0, 2, 5], dtype=torch.int32)])
    s2 = RaggedTensor(torch.arange(3, dtype=torch.int8), [torch.tensor([0, 2], dtype=torch.int32), torch.tensor([0, 1, 3], dtype=torch.int32)])
    j = RaggedTensor.concat([s1, s2])
    assert j.offsets()[0].tolist() == [0, 1, 2, 4] and j.offsets()[1].tolist() == [0, 2, 5, 6, 8] and j.values().numel() == 8
    assert RaggedTensor.concat([a]) is a


def test_proportional_windows_natively_equal_the_python_path(tmp_path):
    from recis_b200._ext_io import load
    if load() is None:
        pytest.skip("native reader not built here")
    t1, t2 = str(tmp_path / "t1"), str(tmp_path / "t2")
    _write_table(t1, 0, 3, 170)                       # sheets cross file boundaries and formats
    _write_table(t2, 100000, 2, 120)

    def run(native):
        ds = make_odps_window_io(split_num=2)(60, read_threads_num=3, native_reader=native)
        ds.add_path(t1, (2, 3))
        ds.add_path(t2, (1, 3))
        ds.varlen_feature("items")
        ds.fixedlen_feature("uid")
        ds.fixedlen_feature("score")
        used = []
        if native:
            orig = ds._iter_native_wide
            ds._iter_native_wide = lambda group, per: (used.append(1), orig(group, per))[1]
        out = []
        while True:
            try:
                if ds.next_window():
                    continue
            except StopIteration:
                break
            for b in ds:
                out.append((b["uid"].flatten().tolist(), b["items"].values().tolist(), b["items"].offsets()[0].tolist(),
                            b["score"].flatten().tolist()))
        return out, used

    nat, used = run(True)
    py, _ = run(False)
    assert used and nat == py and sum(len(b[0]) for b in nat) == 510 + 240


def test_tracker_log_on_object_stores_is_written_in_parts():
    import fsspec
    from recis_b200.hooks.ml_tracker_hook import FileTracker
    fs = fsspec.filesystem("memory")
    tr = FileTracker("pp", "run", id="x", root="memory://parts")
    tr.part_lines, tr.flush_every = 5, 2
    for step in range(12):
        tr.log({"v": step}, step)
    tr.finish()
    names = sorted(n.rsplit("/", 1)[1] for n in fs.ls("/parts/pp/run-x", detail=False) if "metrics" in n)
    assert names == ["metrics-00001.jsonl", "metrics-00002.jsonl", "metrics.jsonl"]
    got = []
    for n in ["metrics.jsonl", "metrics-00001.jsonl", "metrics-00002.jsonl"]:
        got += [json.loads(l)["v"] for l in fs.cat("/parts/pp/run-x/" + n).decode().splitlines()]
    assert got == list(range(12))
