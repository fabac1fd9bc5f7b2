"""Sparse checkpoint bundle: layout checked with an independent reader, save -> load -> save byte equality, resharding."""
import json
import os

import pytest
import torch

import recis_b200
from recis_b200.nn import EmbeddingEngine, EmbeddingOption, HashTable, filter_out_sparse_param, gen_slice
from recis_b200.nn.hashtable_hook import FilterHook
from recis_b200.nn.initializers import NormalInitializer
from recis_b200.nn.modules.hashtable import HashtableRegister
from recis_b200.optim import SparseAdamW
from recis_b200.serialize import CheckpointReader, Loader, Saver


def _trained_engine(steps=3, seed=0):
    torch.manual_seed(seed)
    init = NormalInitializer(0, 0.05)
    opts = {"user": EmbeddingOption(embedding_dim=8, shared_name="user", initializer=init, device="cpu"),
            "item": EmbeddingOption(embedding_dim=8, shared_name="item", initializer=init, device="cpu"),
            "wide": EmbeddingOption(embedding_dim=4, shared_name="wide", initializer=init, device="cpu",
                                    filter_hook=FilterHook("GlobalStepFilter", {"filter_step": 100}))}
    eng = EmbeddingEngine(opts)
    opt = SparseAdamW(filter_out_sparse_param(eng), lr=0.01)
    for t in range(steps):
        feats = {k: torch.randint(0, 500, (16, 3)) * 31 for k in opts}
        out = eng(feats)
        loss = sum(v.square().sum() for v in out.values())
        opt.zero_grad(); loss.backward(); opt.step()
    return eng, opt


def _dump(eng):
    out = {}
    for name, ht in eng.tables().items():
        ids, rows = ht.impl.ids_map()
        order = torch.argsort(ids)
        st = ht.impl.store
        out[name] = dict(ids=ids[order], emb=st.emb()[rows[order]],
                         slots={s: st.slot(s)[rows[order]] for s in st.slot_names()}, seen=st.last_seen()[rows[order]])
    return out


def test_layout_and_independent_reader(tmp_path):
    eng, opt = _trained_engine()
    dense = {"w": torch.randn(3, 5), "flag": torch.tensor([True, False]), "sparse_adamw_step": torch.tensor(3.0)}
    Saver(0, 1, 2, str(tmp_path), filter_out_sparse_param(eng), dense).save()
    files = sorted(os.listdir(tmp_path))
    assert files == ["index", "model-000000-of-000002.safetensors", "model-000001-of-000002.safetensors", "tensorkey.json",
                     "torch_rank_weights_embs_table_multi_shard.json"]
    index = json.load(open(tmp_path / "index"))
    assert set(index) == {"file_index", "block_index"}
    tk = json.load(open(tmp_path / "tensorkey.json"))
    assert tk["user.embedding/part_0_1"] == "user@embedding^00000@65536@65536"
    assert "user.sparse_adamw_exp_avg/part_0_1" in tk and "wide.id/part_0_1" in tk and "w^ " in index["block_index"]
    rank = json.load(open(tmp_path / "torch_rank_weights_embs_table_multi_shard.json"))
    e = rank["item.embedding/part_0_1"]
    assert e["is_hashmap"] and e["hashmap_key"] == "item.id/part_0_1" and e["dimension"] == 8 and e["dtype"] == "float32"
    # raw format: u64 header length, JSON padded with at least one space to a multiple of 8
    raw = open(tmp_path / "model-000000-of-000002.safetensors", "rb").read()
    hlen = int.from_bytes(raw[:8], "little")
    assert hlen % 8 == 0 and raw[8 + hlen - 1:8 + hlen] == b" "
    # an independent implementation reads the files
    safetensors = pytest.importorskip("safetensors")
    from safetensors import safe_open
    seen = {}
    for f in files:
        if f.endswith(".safetensors"):
            with safe_open(str(tmp_path / f), framework="pt") as fh:
                for k in fh.keys():
                    seen[k] = fh.get_tensor(k)
    ref = _dump(eng)
    table = next(n for n, t in eng.tables().items() if t.impl.dim == 8)
    ids = seen["user.id/part_0_1"]
    enc = ids | (0 << 52)
    pos = torch.searchsorted(ref[table]["ids"], enc)
    assert torch.equal(ref[table]["ids"][pos], enc)
    assert torch.equal(seen["user.embedding/part_0_1"], ref[table]["emb"][pos])
    assert torch.equal(seen["w^ "], dense["w"]) and torch.equal(seen["flag^ "], dense["flag"])
    rd = CheckpointReader(str(tmp_path))
    assert "user@embedding" in rd.list_tensors() and "w" in rd.list_tensors()
    assert torch.equal(rd.read_tensor("user@embedding"), seen["user.embedding/part_0_1"])
    assert rd.tensor_shape("w") == [3, 5] and rd.tensor_dtype("user@id") == torch.int64


def test_save_load_save_is_byte_identical(tmp_path):
    eng, _ = _trained_engine()
    dense = {"w": torch.randn(4, 4)}
    a, b = tmp_path / "a", tmp_path / "b"
    Saver(0, 1, 1, str(a), filter_out_sparse_param(eng), dense).save()
    ref = _dump(eng)
    HashtableRegister().clear()
    eng2, opt2 = _trained_engine(steps=0, seed=1)          # fresh, empty tables (optimizer slots exist)
    dense2 = {"w": torch.zeros(4, 4)}
    Loader(str(a), filter_out_sparse_param(eng2), dense2).load()
    got = _dump(eng2)
    for name in ref:
        assert torch.equal(got[name]["ids"], ref[name]["ids"]) and torch.equal(got[name]["emb"], ref[name]["emb"])
        assert torch.equal(got[name]["seen"], ref[name]["seen"])
        for s in ref[name]["slots"]:
            assert torch.equal(got[name]["slots"][s], ref[name]["slots"][s])
    assert torch.equal(dense2["w"], dense["w"])
    Saver(0, 1, 1, str(b), filter_out_sparse_param(eng2), dense2).save()
    for f in os.listdir(a):
        assert open(a / f, "rb").read() == open(b / f, "rb").read(), f


@pytest.mark.parametrize("w_save,w_load", [(4, 1), (1, 3), (3, 2)])
def test_resharding(tmp_path, w_save, w_load):
    torch.manual_seed(0)
    all_ids = torch.randint(0, 1 << 40, (3000,)).unique()
    emb_of = {}
    for r in range(w_save):
        HashtableRegister().clear()
        sl = gen_slice(r, w_save)
        ht = HashTable([8], initializer=NormalInitializer(0, 1), name="tbl", device="cpu", slice=sl)
        mine = all_ids[((all_ids & 0xFFFF) >= sl.slice_begin) & ((all_ids & 0xFFFF) < sl.slice_end)]
        e = ht(mine)
        for i, v in zip(mine.tolist(), e.detach()):
            emb_of[i] = v.clone()
        Saver(r, w_save, 2, str(tmp_path), filter_out_sparse_param(ht), {"d": torch.arange(3.0)} if r == 0 else {}).save()
    assert os.path.exists(tmp_path / "index")
    total = 0
    for r in range(w_load):
        HashtableRegister().clear()
        sl = gen_slice(r, w_load)
        ht = HashTable([8], initializer=NormalInitializer(0, 1), name="tbl", device="cpu", slice=sl)
        Loader(str(tmp_path), filter_out_sparse_param(ht), {}).load()
        ids, rows = ht.ids_map()
        assert bool((((ids & 0xFFFF) >= sl.slice_begin) & ((ids & 0xFFFF) < sl.slice_end)).all())
        for i, row in zip(ids.tolist(), rows.tolist()):
            assert torch.equal(ht.embeddings()[row], emb_of[i])
        total += ids.numel()
    assert total == all_ids.numel()


def test_failures_are_clean_errors(tmp_path):
    eng, _ = _trained_engine(steps=1)
    Saver(0, 1, 1, str(tmp_path), filter_out_sparse_param(eng), {"w": torch.ones(2)}).save()
    HashtableRegister().clear()
    eng2, _ = _trained_engine(steps=0)
    with pytest.raises(KeyError):
        Loader(str(tmp_path), filter_out_sparse_param(eng2), {"missing": torch.zeros(1)}).load()
    with pytest.raises(ValueError):
        Loader(str(tmp_path), {}, {"w": torch.zeros(3)}).load()
    # truncated shard: the loader reports it instead of reading garbage
    f = tmp_path / "model-000000-of-000001.safetensors"
    data = open(f, "rb").read()
    open(f, "wb").write(data[: len(data) // 2])
    HashtableRegister().clear()
    eng3, _ = _trained_engine(steps=0)
    with pytest.raises(RuntimeError):
        Loader(str(tmp_path), filter_out_sparse_param(eng3), {}).load()
    os.remove(tmp_path / "index")
    with pytest.raises(FileNotFoundError):
        Loader(str(tmp_path), {}, {})


def test_resharding_chain_8_4_1_8(tmp_path):
    """Save with 8 shards, reload into 4, save, reload into 1, save, reload into 8: every id keeps its embedding and its
    optimizer-free slots, and lands on the shard that owns its low 16 bits."""
    torch.manual_seed(1)
    all_ids = torch.randint(0, 1 << 44, (4000,)).unique()
    truth = {}

    def make(world):
        tables = []
        for r in range(world):
            HashtableRegister().clear()
            tables.append(HashTable([4], initializer=NormalInitializer(0, 1), name="tbl", device="cpu", slice=gen_slice(r, world)))
        return tables

    def owned(ids, sl):
        low = ids & 0xFFFF
        return ids[(low >= sl.slice_begin) & (low < sl.slice_end)]

    def save(tables, world, d):
        os.makedirs(d, exist_ok=True)
        for r, ht in enumerate(tables):
            Saver(r, world, 2, str(d), filter_out_sparse_param(ht), {}).save()

    def load(world, d):
        tables = make(world)
        for ht in tables:
            Loader(str(d), filter_out_sparse_param(ht), {}).load()
        return tables

    tables = make(8)
    for r, ht in enumerate(tables):
        mine = owned(all_ids, gen_slice(r, 8))
        for i, v in zip(mine.tolist(), ht(mine).detach()):
            truth[i] = v.clone()
    prev_world = 8
    for step, world in enumerate([4, 1, 8]):
        d = tmp_path / f"ckpt{step}"
        save(tables, prev_world, d)
        tables = load(world, d)
        seen = 0
        for r, ht in enumerate(tables):
            ids, rows = ht.ids_map()
            assert torch.equal(owned(ids, gen_slice(r, world)).sort().values, ids.sort().values)
            for i, row in zip(ids.tolist(), rows.tolist()):
                assert torch.equal(ht.embeddings()[row], truth[i])
            seen += ids.numel()
        assert seen == all_ids.numel()
        prev_world = world


def test_native_platform_layer(tmp_path):
    C = recis_b200.native()
    assert C.fs_join("a/", "/b") == "a/b" and C.fs_join("a", "b") == "a/b" and C.fs_join("", "b") == "b"
    assert C.fs_dirname("/x/y/z.txt") == "/x/y" and C.fs_basename("/x/y/z.txt") == "z.txt" and C.fs_dirname("z") == ""
    assert C.fs_parse_uri("file:///tmp/a") == ("file", "/tmp/a") and C.fs_parse_uri("/tmp/a") == ("", "/tmp/a")
    assert C.fs_parse_uri("weird path://x") == ("", "weird path://x")
    assert set(C.fs_schemes()) >= {"", "file"}
    d = str(tmp_path / "a" / "b" / "c")
    C.fs_mkdirs(d)
    C.fs_mkdirs(d)                                              # idempotent
    payload = bytes(range(256)) * 1000
    C.fs_write_bytes("file://" + d + "/blob.bin", payload)       # scheme form and plain form name the same file
    assert C.fs_exists(d + "/blob.bin") and C.fs_file_size(d + "/blob.bin") == len(payload)
    assert C.fs_read_bytes(d + "/blob.bin") == payload and C.fs_list(d) == ["blob.bin"]       # no ".tmp" left behind
    C.fs_rename(d + "/blob.bin", d + "/blob2.bin")
    assert C.fs_list(d) == ["blob2.bin"]
    C.fs_delete(d + "/blob2.bin")
    assert not C.fs_exists(d + "/blob2.bin")
    with pytest.raises(RuntimeError, match="no file system registered"):
        C.fs_exists("pangu://cluster/path")
    with pytest.raises(RuntimeError):
        C.fs_write_bytes(str(tmp_path / "missing_dir" / "x.bin"), b"1")
    assert not os.path.exists(tmp_path / "missing_dir")


def test_failed_save_leaves_no_partial_shard(tmp_path):
    """A save whose files cannot be created fails with an error and leaves nothing behind that a later load could mistake for a
    checkpoint (shards are written under a temporary name and renamed when complete)."""
    HashtableRegister().clear()
    eng, _opt = _trained_engine(steps=1)
    good = tmp_path / "good"
    Saver(0, 1, 1, str(good), filter_out_sparse_param(eng), {"w": torch.ones(3)}).save()
    before = sorted(os.listdir(good))
    blocker = tmp_path / "blocker"
    blocker.write_text("a regular file where a directory is expected")
    with pytest.raises((RuntimeError, OSError)):
        Saver(0, 1, 1, str(blocker / "ckpt"), filter_out_sparse_param(eng), {"w": torch.ones(3)}).save()
    assert blocker.read_text().startswith("a regular file")
    assert sorted(os.listdir(good)) == before and not any(f.endswith(".tmp") for f in before)


def test_filter_func_leaves_tensors_out_of_save_and_load(tmp_path):
    """``filter_func`` of Saver (write blocks) and Loader (load plan), the reference's hooks of the same name."""
    from recis_b200.ragged import RaggedTensor

    def engine(name):
        return EmbeddingEngine({"u": EmbeddingOption(embedding_dim=4, shared_name=name, initializer=NormalInitializer(0, 0.05), device="cpu")})
    eng = engine("ff_tab")
    eng({"u": RaggedTensor(torch.arange(10) * 7919, [torch.arange(0, 11, 2, dtype=torch.int32)])})
    dense = {"keep": torch.ones(3), "drop": torch.zeros(2)}
    Saver(0, 1, 1, str(tmp_path), filter_out_sparse_param(eng), dense,
          filter_func=lambda blocks: [b for b in blocks if not b[0].startswith("drop")]).save()
    names = CheckpointReader(str(tmp_path)).list_tensors()
    assert "keep" in names and "drop" not in names
    del eng
    import gc
    gc.collect()
    eng2 = engine("ff_tab")
    target = {"keep": torch.zeros(3)}
    seen = {}

    def plan(p):
        seen.update(p)
        return {"hashtables": [], "tensors": p["tensors"]}              # dense only
    Loader(str(tmp_path), filter_out_sparse_param(eng2), target, filter_func=plan).load()
    assert torch.equal(target["keep"], torch.ones(3)) and seen["tensors"] == ["keep"] and seen["hashtables"] == ["ff_tab"]
    table = next(iter(eng2.tables().values()))
    assert table.impl.store.size() == 0                                   # the table was left out of the plan
    Loader(str(tmp_path), filter_out_sparse_param(eng2), {}).load()
    assert table.impl.store.size() == 10


def test_convert_v1_directory_into_a_loadable_bundle(tmp_path):
    """Per-shard ``torch.save`` files + ``dense.pt`` -> safetensors bundle that the Loader reshards into one table."""
    from recis_b200.serialize.convert_v1_to_v2 import convert_v1_to_v2
    src, dst = tmp_path / "v1", tmp_path / "v2"
    src.mkdir()
    torch.manual_seed(0)
    all_ids = torch.arange(0, 400, dtype=torch.int64) * 7919
    emb = torch.randn(400, 4)
    world = 2
    for r in range(world):
        sl = gen_slice(r, world)
        mine = ((all_ids & 0xFFFF) >= sl.slice_begin) & ((all_ids & 0xFFFF) < sl.slice_end)
        torch.save({"ids": all_ids[mine], "embeddings": emb[mine]}, src / f"conv_tab.shard_{r}_of_{world}.pt")
    torch.save({"w": torch.arange(6.0).view(2, 3)}, src / "dense.pt")
    convert_v1_to_v2(str(src), str(dst))
    reader = CheckpointReader(str(dst))
    assert torch.equal(reader.read_tensor("w"), torch.arange(6.0).view(2, 3))
    ht = HashTable([4], name="conv_tab", initializer=NormalInitializer(0, 0.01), slice=gen_slice(0, 1))
    dense = {"w": torch.zeros(2, 3)}
    Loader(str(dst), filter_out_sparse_param(ht), dense).load()
    assert ht.impl.store.size() == 400 and torch.equal(dense["w"], torch.arange(6.0).view(2, 3))
    ids, rows = ht.impl.ids_map()
    order = torch.argsort(ids)
    assert torch.equal(ids[order], all_ids) and torch.allclose(ht.impl.store.emb()[rows[order]], emb)


def test_write_that_fails_midway_removes_its_temporary_file(tmp_path):
    """The file system refuses data beyond 64 KiB (RLIMIT_FSIZE, standing in for a full disk): the save raises, and neither a
    shard nor a temporary file is left in the directory."""
    import subprocess
    import sys
    code = f"""
import os, resource, signal, sys, torch
sys.path.insert(0, {os.path.dirname(os.path.dirname(os.path.abspath(__file__)))!r})
from recis_b200.serialize import Saver
signal.signal(signal.SIGXFSZ, signal.SIG_IGN)
resource.setrlimit(resource.RLIMIT_FSIZE, (65536, 65536))
try:
    Saver(0, 1, 1, {str(tmp_path)!r}, {{}}, {{"big": torch.zeros(1 << 20)}}).save()
except Exception as e:
    print("raised", type(e).__name__)
print("files", sorted(os.listdir({str(tmp_path)!r})))
"""
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert "raised" in out.stdout, out.stdout + out.stderr
    assert "files []" in out.stdout, out.stdout


def test_missing_index_entry_is_reported_by_name(tmp_path):
    """A block that the tensor-key file lists but the index does not know: the load names it instead of reading another block."""
    HashtableRegister().clear()
    eng, _opt = _trained_engine(steps=1)
    Saver(0, 1, 1, str(tmp_path), filter_out_sparse_param(eng), {}).save()
    index = json.load(open(tmp_path / "index"))
    victim = next(k for k in index["block_index"] if k.startswith("user.embedding/"))
    del index["block_index"][victim]
    json.dump(index, open(tmp_path / "index", "w"))
    HashtableRegister().clear()
    eng2, _ = _trained_engine(steps=0)
    with pytest.raises((KeyError, RuntimeError, ValueError)) as e:
        Loader(str(tmp_path), filter_out_sparse_param(eng2), {}).load()
    assert "user.embedding" in str(e.value)
