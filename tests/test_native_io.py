"""Native columnar reader (C++: reader threads, packer, prefetch queue, iterator state) against the pyarrow-in-Python path."""
import os

import numpy as np
import pytest
import torch

from recis_b200._ext_io import load
from recis_b200.io import OrcDataset

pa = pytest.importorskip("pyarrow")
pytestmark = pytest.mark.skipif(load() is None, reason="Arrow C++ development files are not available")


def _write(tmp_path, shards=3, rows=(70, 33, 50), fmt="orc"):
    import pyarrow.orc as orc
    import pyarrow.parquet as pq
    rng = np.random.default_rng(0)
    paths = []
    for s in range(shards):
        n = rows[s]
        seq = [rng.integers(0, 1000, rng.integers(0, 6)).astype(np.int64) for _ in range(n)]
        words = [[f"w{int(x)}" for x in rng.integers(0, 50, rng.integers(0, 4))] for _ in range(n)]
        t = pa.table({
            "label": rng.random(n).astype(np.float32), "age": rng.integers(0, 90, n).astype(np.int32),
            "uid": rng.integers(-(1 << 40), 1 << 40, n), "seq": pa.array(seq, type=pa.list_(pa.int64())),
            "city": pa.array([f"city_{int(x)}" for x in rng.integers(0, 20, n)]), "words": pa.array(words, type=pa.list_(pa.string())),
        })
        p = str(tmp_path / f"part-{s:05d}.{fmt}")
        if fmt == "orc":
            orc.write_table(t, p)
        else:
            pq.write_table(t, p, row_group_size=16)          # several row groups per file
        paths.append(p)
    return paths


def _dataset(paths, native, **kw):
    ds = OrcDataset(batch_size=32, native_reader=native, read_threads_num=3, prefetch=2, **kw)
    ds.add_paths(paths)
    ds.varlen_feature("uid", hash_bucket=1000003)
    ds.varlen_feature("seq")
    ds.varlen_feature("city", hash_type="farm", hash_bucket=1000)
    ds.varlen_feature("words", hash_type="murmur")
    ds.fixedlen_feature("label")
    ds.fixedlen_feature("age")
    return ds


def _same(a, b):
    assert a.keys() == b.keys()
    for k in a:
        x, y = a[k], b[k]
        if isinstance(x, torch.Tensor):
            assert torch.equal(x, y), k
        else:
            assert torch.equal(x.values(), y.values()), k
            assert len(x.offsets()) == len(y.offsets())
            for ox, oy in zip(x.offsets(), y.offsets()):
                assert torch.equal(ox.to(torch.int64), oy.to(torch.int64)), k


def test_native_reader_matches_python_reader(tmp_path):
    paths = _write(tmp_path)
    nat, ref = list(_dataset(paths, True)), list(_dataset(paths, False))
    assert len(nat) == len(ref) == 3 + 2 + 2
    for a, b in zip(nat, ref):
        _same(a, b)
    assert [b["label"].shape[0] for b in nat] == [32, 32, 6, 32, 1, 32, 18]
    # drop_remainder drops the short tail of every file
    assert [b["label"].shape[0] for b in _dataset(paths, True, drop_remainder=True)] == [32, 32, 32, 32]


def test_native_reader_keeps_bytes_for_the_feature_engine(tmp_path):
    paths = _write(tmp_path, shards=1, rows=(10,))
    ds = OrcDataset(batch_size=10, native_reader=True)
    ds.add_paths(paths)
    ds.varlen_feature("city", trans_int8=True)
    ref = OrcDataset(batch_size=10, native_reader=False)
    ref.add_paths(paths)
    ref.varlen_feature("city", trans_int8=True)
    _same(next(iter(ds)), next(iter(ref)))


def test_native_reader_state_resumes_mid_file(tmp_path):
    paths = _write(tmp_path)
    full = list(_dataset(paths, True))
    ds = _dataset(paths, True)
    it = iter(ds)
    for _ in range(4):
        next(it)
    state = ds.dump_io_state()
    assert state == {"file_idx": 1, "row_in_file": 32}
    ds2 = _dataset(paths, True)
    ds2.load_io_state(state)
    rest = list(ds2)
    assert len(rest) == len(full) - 4
    for a, b in zip(rest, full[4:]):
        _same(a, b)


def test_native_reader_reports_a_missing_file(tmp_path):
    paths = _write(tmp_path, shards=1, rows=(5,)) + [str(tmp_path / "missing.orc")]
    ds = OrcDataset(batch_size=4, native_reader=True)
    ds.add_paths(paths)
    ds.varlen_feature("uid")
    with pytest.raises(RuntimeError, match="missing.orc"):
        list(ds)


def test_repeat_and_worker_sharding(tmp_path):
    paths = _write(tmp_path)
    rows_native = sum(b["label"].shape[0] for b in _dataset(paths, True, repeat=2))
    rows_python = sum(b["label"].shape[0] for b in _dataset(paths, False, repeat=2))
    assert rows_native == rows_python == 2 * (70 + 33 + 50)
    # two workers split the files; together they see every row once
    per_worker = []
    for w in range(2):
        ds = OrcDataset(batch_size=32, worker_idx=w, worker_num=2)
        ds.add_paths(paths)
        ds.varlen_feature("uid")
        per_worker.append(sum(b["uid"].values().numel() for b in ds))
    assert sorted(per_worker) == sorted([70 + 50, 33])


def test_native_reader_reads_parquet_like_the_python_reader(tmp_path):
    """Parquet files (several row groups each) go through the same native packer; a missing column is reported by name."""
    paths = _write(tmp_path, fmt="parquet")
    ds = _dataset(paths, True)
    assert ds._native(ds._my_paths()) is not None                   # the native reader takes Parquet
    nat, ref = list(ds), list(_dataset(paths, False))
    assert len(nat) == len(ref) == 7
    for a, b in zip(nat, ref):
        _same(a, b)
    bad = OrcDataset(batch_size=8, native_reader=True)
    bad.add_paths(paths[:1])
    bad.varlen_feature("no_such_column")
    with pytest.raises(RuntimeError, match="no_such_column"):
        list(bad)


def test_shuffle_is_a_seeded_file_order_shared_by_both_readers(tmp_path):
    paths = _write(tmp_path, shards=3, rows=(40, 41, 42))
    sizes = lambda ds: [b["label"].shape[0] for b in ds]
    plain = sizes(_dataset(paths, True))
    orders = {seed: sizes(_dataset(paths, True, shuffle=True, seed=seed)) for seed in range(6)}
    assert all(sorted(o) == sorted(plain) for o in orders.values())          # same batches, some other file order
    assert any(o != plain for o in orders.values())
    for seed, o in orders.items():
        assert o == sizes(_dataset(paths, True, shuffle=True, seed=seed))    # deterministic
        assert o == sizes(_dataset(paths, False, shuffle=True, seed=seed))   # both readers agree
    # two passes are shuffled independently but cover every file twice
    two = sizes(_dataset(paths, True, shuffle=True, seed=1, repeat=2))
    assert sorted(two) == sorted(plain * 2)


@pytest.mark.parametrize("native_reader", [True, False])
def test_ragged_format_false_gives_sparse_tensors(tmp_path, native_reader):
    paths = _write(tmp_path, shards=1, rows=(20,))

    def make(ragged_format):
        ds = OrcDataset(batch_size=20, native_reader=native_reader, ragged_format=ragged_format)
        ds.add_paths(paths)
        ds.varlen_feature("seq")
        ds.fixedlen_feature("label")
        return next(iter(ds))

    ragged, sparse = make(True), make(False)
    assert sparse["seq"].is_sparse and not sparse["label"].is_sparse
    dense = ragged["seq"].to_dense()
    assert torch.equal(sparse["seq"].to_dense()[:, : dense.shape[1]], dense)
    with pytest.raises(AssertionError):
        OrcDataset(batch_size=4, device="tpu")


def test_registered_maps_run_before_transform_fn_and_filters_skip(tmp_path):
    paths = _write(tmp_path, shards=1, rows=(64,))
    for native_reader in (True, False):
        ds = OrcDataset(batch_size=16, native_reader=native_reader,
                        transform_fn=[lambda b: dict(b, order=b["order"] + ["transform"])])
        ds.add_paths(paths)
        ds.fixedlen_feature("label")
        ds.map(lambda b: dict(b, order=["map"]))
        n = [0]

        def every_other(b):
            n[0] += 1
            return n[0] % 2 == 0                       # True = skip
        ds.filter(every_other)
        got = list(ds)
        assert len(got) == 2 and all(b["order"] == ["map", "transform"] for b in got)


@pytest.mark.parametrize("native_reader", [True, False])
def test_second_iteration_is_a_new_epoch(tmp_path, native_reader):
    paths = _write(tmp_path, shards=2, rows=(20, 12))
    ds = _dataset(paths, native_reader)
    first = [b["label"].clone() for b in ds]
    second = [b["label"].clone() for b in ds]
    assert len(first) == len(second) == 2 and all(torch.equal(a, b) for a, b in zip(first, second))
