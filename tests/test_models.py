"""Model zoo and benchmark scripts on CPU: the sequence model's ragged attention against a per-sequence reference, and the
benchmark scripts end to end at toy sizes (they print one JSON line)."""
import json
import os
import subprocess
import sys

import pytest
import torch

from recis_b200.models.seq_model import EncoderLayer, SequenceModel, segment_softmax
from recis_b200.nn import filter_out_sparse_param
from recis_b200.nn.modules.hashtable import HashtableRegister
from recis_b200.optim import DenseAdam, SparseAdam
from recis_b200.ragged import RaggedTensor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ragged_batch(B=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(3, 20, (B,), generator=g)
    offs = torch.zeros(B + 1, dtype=torch.int32)
    offs[1:] = lens.cumsum(0)
    return lens, offs, int(offs[-1])


def test_segment_softmax_matches_per_segment():
    lens, offs, T = _ragged_batch()
    s = torch.randn(T)
    seg = torch.repeat_interleave(torch.arange(lens.numel()), lens)
    ref = torch.cat([torch.softmax(s[offs[i]:offs[i + 1]], 0) for i in range(lens.numel())])
    assert torch.allclose(segment_softmax(s, seg, lens.numel()), ref, atol=1e-6)


def test_encoder_layer_on_packed_tokens_matches_per_sequence():
    torch.manual_seed(0)
    lens, offs, T = _ragged_batch(B=5, seed=1)
    layer = EncoderLayer(hidden=32, heads=4, ffn=64, dtype=torch.float32)
    x = torch.randn(T, 32)
    seg = torch.repeat_interleave(torch.arange(lens.numel()), lens)
    pos = torch.arange(T) - offs[:-1].long()[seg]
    got = layer(x, seg, pos, lens.long(), int(lens.max()) + 3)      # extra padding columns must not change anything
    for i in range(lens.numel()):
        xi = x[offs[i]:offs[i + 1]]
        one = layer(xi, torch.zeros(xi.shape[0], dtype=torch.long), torch.arange(xi.shape[0]), lens[i:i + 1].long(), int(lens[i]))
        assert torch.allclose(got[offs[i]:offs[i + 1]], one, atol=1e-5), i


def test_sequence_model_trains_on_cpu():
    HashtableRegister().clear()
    torch.manual_seed(0)
    lens, offs, T = _ragged_batch(B=8, seed=2)
    B = lens.numel()
    pf = ["p0", "p1"]
    batch = {"seq_item": RaggedTensor(torch.randint(0, 500, (T,)), [offs]), "seq_cate": RaggedTensor(torch.randint(0, 20, (T,)), [offs]),
             "tgt_item": torch.randint(0, 500, (B,)), "tgt_cate": torch.randint(0, 20, (B,)),
             "label": (torch.rand(B, 1) < 0.4).float(), "max_len": int(lens.max()), "p0": torch.randint(0, 9, (B,)),
             "p1": torch.randint(0, 9, (B,))}
    m = SequenceModel(pf, emb_dim=8, profile_dim=4, hidden=32, heads=4, layers=2, ffn=64, head_mlp=(16, 1), device="cpu",
                      compute_dtype=torch.float32, max_len=64)
    # sequence and target features of one entity share one child table
    assert len(m.embedding_engine.tables()) == 2
    so = SparseAdam(filter_out_sparse_param(m), lr=1e-2)
    do = DenseAdam([p for p in m.parameters() if p.requires_grad], lr=1e-2)
    losses = []
    for _ in range(25):
        loss, logit = m(batch)
        do.zero_grad(); so.zero_grad(); loss.backward(); so.step(); do.step()
        losses.append(float(loss.detach()))
    assert logit.shape == (B, 1) and losses[-1] < 0.5 * losses[0]


def _run(script, *args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", script), *args], capture_output=True, text=True, timeout=600,
                         env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    return json.loads(lines[-1])


def test_benchmark_scripts_run_on_cpu():
    r = _run("embedding_microbench.py", "--tables", "5", "--batch", "32", "--steps", "2", "--warmup", "1")
    assert r["bench"] == "embedding_microbench" and r["unique_per_rank"] <= r["ids_per_rank"] and r["forward_ms"] > 0
    r = _run("multitable.py", "--fields", "10", "--batch", "32", "--steps", "4", "--warmup", "1", "--ttl", "2", "--filter-interval", "2")
    assert r["physical_tables"] == 5 and r["checkpoint"]["round_trip_identical"] is True and r["evicted_rows_rank0"] > 0
    r = _run("sequence_model.py", "--batch", "8", "--min-len", "4", "--max-len", "20", "--items", "2000", "--cates", "50",
             "--profile-fields", "2", "--hidden", "32", "--steps", "2", "--warmup", "1")
    assert r["bench"] == "sequence_model" and r["ms_per_step"] > 0


def _run_example(path, *args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, os.path.join(ROOT, path), *args], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    return out.stdout + out.stderr


def test_examples_run_on_cpu(tmp_path):
    log = _run_example("examples/deepfm/run.py", "--device", "cpu", "--steps", "6", "--batch", "64", "--output-dir", str(tmp_path / "fm"))
    assert "trained 6 steps" in log and os.path.exists(tmp_path / "fm" / "checkpoint")
    _run_example("examples/deepctr/make_orc_data.py", "--out", str(tmp_path / "orc"), "--shards", "2", "--rows", "256")
    log = _run_example("examples/deepctr/run.py", "--data", str(tmp_path / "orc"), "--device", "cpu", "--batch", "64",
                       "--output-dir", str(tmp_path / "ctr"))
    assert "CoalescedHashtable_" in log
    log = _run_example("examples/deepctr/run.py", "--data", str(tmp_path / "orc"), "--device", "cpu", "--batch", "64", "--windows", "2",
                       "--trace-dir", str(tmp_path / "trace"), "--output-dir", str(tmp_path / "ctr_windows"))
    import pyarrow.dataset as pads
    assert "Window IO Finish" in log and pads.dataset(str(tmp_path / "trace" / "rank=0"), format="parquet").count_rows() == 512
    log = _run_example("examples/seq2seq/run.py", "--device", "cpu", "--steps", "3", "--batch", "4", "--max-len", "16")
    assert "step    2" in log


def test_csv_to_orc_round_trip(tmp_path):
    from recis_b200.io import OrcDataset
    from recis_b200.io.csv_to_orc import convert
    csv = tmp_path / "d.csv"
    csv.write_text("label,uid,seq\n1,10,1|2|3\n0,11,\n1,12,7\n0,13,4|4\n")
    assert convert(str(csv), str(tmp_path / "out"), rows_per_shard=3, list_columns=["seq"]) == 2
    ds = OrcDataset(batch_size=4)
    ds.add_paths([str(tmp_path / "out" / f) for f in sorted(os.listdir(tmp_path / "out"))])
    ds.varlen_feature("uid")
    ds.varlen_feature("seq")
    ds.fixedlen_feature("label")
    batches = list(ds)
    assert sum(b["label"].shape[0] for b in batches) == 4
    assert batches[0]["seq"].values().tolist() == [1, 2, 3, 7] and batches[0]["seq"].offsets()[0].tolist() == [0, 3, 3, 4]
    assert batches[1]["uid"].values().tolist() == [13]


def test_quickstart_document_runs_as_written(tmp_path, monkeypatch):
    """The first python block of docs/quickstart.md, with the data paths and sizes swapped for a generated toy set."""
    import re
    import numpy as np
    pa = pytest.importorskip("pyarrow")
    import pyarrow.orc as orc
    from recis_b200.nn.modules.hashtable import HashtableRegister
    HashtableRegister().clear()
    rng = np.random.default_rng(0)
    paths = []
    for s in range(2):
        n = 200
        t = pa.table({"user": pa.array([rng.integers(0, 1 << 40, rng.integers(1, 4)).astype(np.int64) for _ in range(n)], type=pa.list_(pa.int64())),
                      "city": pa.array([f"c{int(x)}" for x in rng.integers(0, 30, n)]),
                      "price": (rng.random(n) * 100).astype(np.float32), "label": (rng.random(n) < 0.3).astype(np.float32)})
        p = str(tmp_path / f"part-{s:05d}.orc")
        orc.write_table(t, p)
        paths.append(p)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = re.search(r"```python\n(.*?)```", open(os.path.join(root, "docs", "quickstart.md")).read(), re.S).group(1)
    code = code.replace('["/data/part-00000.orc", "/data/part-00001.orc"]', repr(paths)).replace("batch_size=4096", "batch_size=50")
    code = code.replace("train_steps=1000, save_steps=500", "train_steps=4, save_steps=2").replace('output_dir="out"', f'output_dir={str(tmp_path / "out")!r}')
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)          # the document picks the device; keep this test on CPU
    exec(compile(code, "quickstart.md", "exec"), {"__name__": "quickstart"})
    assert sorted(os.listdir(tmp_path / "out")) == ["checkpoint", "ckpt_2", "ckpt_4"]


def test_examples_run_as_two_cpu_ranks(tmp_path):
    """The examples under torch.distributed.run: two CPU ranks, tables sharded over them; DeepFM on the shared-memory fused
    exchange, the ORC example on the collective exchange with the files dealt to the ranks."""
    import socket

    def launch(script, *args, env=None):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
               "--master-port", str(port), os.path.join(ROOT, script), *args]
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=dict(os.environ, CUDA_VISIBLE_DEVICES="", **(env or {})))
        assert out.returncode == 0, out.stderr[-3000:]
        return out.stdout + out.stderr

    log = launch("examples/deepfm/run.py", "--device", "cpu", "--steps", "4", "--batch", "32", "--output-dir", str(tmp_path / "fm"),
                 env={"RECIS_COMM": "fused"})
    assert "x 2 rank(s)" in log
    files = os.listdir(tmp_path / "fm" / "ckpt_4")
    assert sum(f.endswith(".safetensors") for f in files) >= 2 and "index" in files          # both ranks' shards, merged metadata
    _run_example("examples/deepctr/make_orc_data.py", "--out", str(tmp_path / "orc"), "--shards", "2", "--rows", "128")
    log = launch("examples/deepctr/run.py", "--data", str(tmp_path / "orc"), "--device", "cpu", "--batch", "32")
    assert "CoalescedHashtable_" in log
    # windows are walked in step by both ranks, each reading its share of every window and tracing its own samples
    log = launch("examples/deepctr/run.py", "--data", str(tmp_path / "orc"), "--device", "cpu", "--batch", "32", "--windows", "2",
                 "--trace-dir", str(tmp_path / "trace"), "--output-dir", str(tmp_path / "ctr_windows"))
    import pyarrow.dataset as pads
    counts = [pads.dataset(str(tmp_path / "trace" / f"rank={r}"), format="parquet").count_rows() for r in range(2)]
    assert "Window IO Finish" in log and counts == [128, 128]
