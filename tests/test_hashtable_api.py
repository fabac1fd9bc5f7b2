"""HashTable / engine behaviours that the reference tests in tests/hashtable and tests/optim: direct table API, slots, state
dict, gradient accumulation, learning-rate schedulers on the sparse optimizer, mean / weighted pooling, shared and conflicting
table names, non-trainable features."""
import pytest
import torch

from recis_b200.nn import EmbeddingEngine, EmbeddingOption, HashTable, filter_out_sparse_param
from recis_b200.nn.initializers import ConstantInitializer, NormalInitializer
from recis_b200.nn.modules.hashtable import HashtableRegister, split_sparse_dense_state_dict
from recis_b200.optim import SparseAdam, SparseAdamW, SparseSGD
from recis_b200.ragged import RaggedTensor


@pytest.fixture(autouse=True)
def _fresh_registry():
    HashtableRegister().clear()
    yield
    HashtableRegister().clear()


def test_direct_table_api_insert_ids_embeddings_clear():
    ht = HashTable([4], device="cpu", initializer=ConstantInitializer(0.5), name="t")
    ids = torch.tensor([7, 3, 7, 1 << 40])
    out = ht(ids)
    assert out.shape == (4, 4) and torch.all(out == 0.5) and sorted(ht.ids().tolist()) == sorted({7, 3, 1 << 40})
    ht.insert(torch.tensor([3, 99]), torch.tensor([[1.0] * 4, [2.0] * 4]))
    got = ht(torch.tensor([3, 99, 7])).detach()
    assert got.tolist() == [[1.0] * 4, [2.0] * 4, [0.5] * 4]
    keys, rows = ht.ids_map()
    assert keys.numel() == 4 and ht.embeddings().shape[1] == 4 and rows.max() < ht.embeddings().shape[0]
    ht.clear()
    assert ht.ids().numel() == 0
    with pytest.raises(Exception):
        HashTable([4], device="cpu", name="t2", children=["a"] * 2)          # duplicate child names


def test_duplicate_table_name_is_rejected():
    first = HashTable([4], device="cpu", name="dup")
    with pytest.raises(ValueError):
        HashTable([4], device="cpu", name="dup")
    del first                                               # a destroyed table frees its name
    import gc
    gc.collect()
    HashTable([4], device="cpu", name="dup")


def test_slots_follow_the_optimizer_and_state_dict_exposes_the_table():
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu")})
    opt = SparseAdam(filter_out_sparse_param(eng), lr=0.1)
    out = eng({"a": torch.arange(5)})["a"]
    out.sum().backward()
    opt.step()
    (table,) = eng.tables().values()
    names = table.table.slot_group().slot_names() if hasattr(table, "table") else table.impl.slot_group.slot_names()
    assert any("exp_avg_sq" in n for n in names) and any(n.endswith("exp_avg") for n in names)
    sparse, dense = split_sparse_dense_state_dict(eng.state_dict())
    assert len(sparse) == 1 and not dense
    scalars = {k for k in opt.state_dict() if "step" in k}
    assert scalars, "the optimizer's step scalar travels with the checkpoint as a dense tensor"


def test_gradient_accumulation_equals_one_big_step():
    def run(accum):
        HashtableRegister().clear()
        torch.manual_seed(0)
        eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu", initializer=NormalInitializer(0, 0.1))})
        opt = SparseSGD(filter_out_sparse_param(eng), lr=0.5)
        opt.set_grad_accum_steps(accum)
        batches = [torch.tensor([1, 2, 3]), torch.tensor([3, 4])]
        if accum == 1:
            out = torch.cat([eng({"a": b})["a"] for b in batches])
            opt.zero_grad()
            (out.sum() / 2).backward()
            opt.step()
        else:
            for b in batches:
                opt.zero_grad()
                eng({"a": b})["a"].sum().backward()
                opt.step()                                # only the second call applies, with the mean over the two micro-batches
        (t,) = eng.tables().values()
        keys, rows = t.impl.ids_map()
        emb = t.impl.store.emb()[rows]
        return {int(k): emb[i].clone() for i, k in enumerate(keys.tolist())}
    a, b = run(1), run(2)
    assert a.keys() == b.keys()
    for k in a:
        assert torch.allclose(a[k], b[k], atol=1e-6), k


def test_lr_scheduler_drives_the_sparse_optimizer():
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=2, shared_name="a", device="cpu", initializer=ConstantInitializer(1.0))})
    opt = SparseSGD(filter_out_sparse_param(eng), lr=1.0)
    sched = torch.optim.lr_scheduler.StepLR(opt, step_size=1, gamma=0.5)
    for _ in range(3):
        opt.zero_grad()
        eng({"a": torch.tensor([5])})["a"].sum().backward()
        opt.step()
        sched.step()
    # the row loses lr * 1 per step with lr = 1, 0.5, 0.25
    (t,) = eng.tables().values()
    keys, rows = t.impl.ids_map()
    assert abs(float(t.impl.store.emb()[rows[0]][0]) - (1.0 - 1.0 - 0.5 - 0.25)) < 1e-6


def test_mean_weights_and_grad_by_id():
    vals = torch.tensor([1, 2, 2, 3, 3, 3])
    offs = torch.tensor([0, 2, 6], dtype=torch.int32)
    w = torch.tensor([1.0, 3.0, 1.0, 1.0, 1.0, 1.0])
    opts = {
        "m": EmbeddingOption(embedding_dim=2, shared_name="x", device="cpu", combiner="mean", use_weight=True, initializer=NormalInitializer(0, 1)),
        "s": EmbeddingOption(embedding_dim=2, shared_name="x", device="cpu", combiner="sum", use_weight=False, initializer=NormalInitializer(0, 1)),
    }
    eng = EmbeddingEngine(opts)
    out = eng({"m": RaggedTensor(vals, [offs], weight=w), "s": RaggedTensor(vals, [offs])})
    (t,) = eng.tables().values()
    assert len(eng.tables()) == 1                       # same shared_name: one child, shared rows
    rows = {int(k): t.impl.store.emb()[r] for k, r in zip(*t.impl.ids_map())}
    # both features live in child 0 of the merged table; ids keep their low 52 bits
    e = {i: rows[i] for i in (1, 2, 3)}
    want_sum = torch.stack([e[1] + e[2], e[2] + 3 * e[3]])
    want_mean = torch.stack([(1 * e[1] + 3 * e[2]) / 2, (e[2] + 3 * e[3]) / 4])      # weighted sum over the bag length
    assert torch.allclose(out["s"], want_sum, atol=1e-6) and torch.allclose(out["m"], want_mean, atol=1e-6)


def test_conflicting_merge_key_for_one_shared_name_is_an_error():
    with pytest.raises(RuntimeError):
        EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="x", device="cpu"),
                         "b": EmbeddingOption(embedding_dim=8, shared_name="x", device="cpu")})


def test_non_trainable_feature_gets_no_gradient():
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=2, shared_name="a", device="cpu", trainable=False, initializer=ConstantInitializer(1.0)),
                           "b": EmbeddingOption(embedding_dim=2, shared_name="b", device="cpu", initializer=ConstantInitializer(1.0))})
    opt = SparseAdamW(filter_out_sparse_param(eng), lr=0.1, weight_decay=0.0)
    out = eng({"a": torch.tensor([1, 2]), "b": torch.tensor([1, 2])})
    assert not out["a"].requires_grad and out["b"].requires_grad
    (out["a"].sum() + out["b"].sum()).backward()
    opt.step()
    (t,) = eng.tables().values()
    keys, rows = t.impl.ids_map()
    emb = t.impl.store.emb()[rows]
    child = keys >> 52
    assert torch.all(emb[child == 0] == 1.0) and torch.all(emb[child == 1] != 1.0)


def test_half_precision_table_dtype_is_the_output_dtype():
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu", dtype=torch.bfloat16,
                                                initializer=ConstantInitializer(0.25))})
    opt = SparseSGD(filter_out_sparse_param(eng), lr=0.5)
    out = eng({"a": torch.arange(3)})["a"]
    assert out.dtype == torch.bfloat16 and out.requires_grad
    out.float().sum().backward()
    opt.step()
    (t,) = eng.tables().values()
    assert t.impl.store.emb().dtype == torch.bfloat16                     # rows are stored in the table dtype (2 bytes each)
    assert torch.allclose(eng({"a": torch.arange(3)})["a"].float(), torch.full((3, 4), -0.25))
    with pytest.raises(NotImplementedError):
        EmbeddingOption(embedding_dim=4, dtype=torch.float64, device="cpu")


def test_reference_submodule_import_paths_exist():
    """Module paths of the reference that user code imports from (package name aside)."""
    import importlib
    for mod, names in {
        "recis_b200.io.orc_dataset": ["OrcDataset", "get_dir_size"], "recis_b200.io.dataset_base": ["DatasetBase"],
        "recis_b200.io.state_dataset": ["StateDataset"], "recis_b200.io.map_dataset": ["MapDataset"],
        "recis_b200.io.filter_dataset": ["FilterDataset"], "recis_b200.io.wrap_end_dataset": ["WrapEndDataset"],
        "recis_b200.optim.sparse_adam": ["SparseAdam"], "recis_b200.optim.sparse_adamw": ["SparseAdamW"],
        "recis_b200.optim.sparse_adamw_tf": ["SparseAdamWTF"], "recis_b200.optim.adamw_tf": ["AdamWTF"],
        "recis_b200.info": ["is_internal_enabled", "get_build_info"],
        "recis_b200.nn.modules.embedding": ["DynamicEmbedding", "EmbeddingOption"],
        "recis_b200.nn.modules.embedding_engine": ["EmbeddingEngine"], "recis_b200.nn.modules.hashtable": ["HashTable", "gen_slice"],
        "recis_b200.nn.hashtable_hook": ["AdmitHook", "FilterHook"], "recis_b200.ragged.tensor": ["RaggedTensor"],
        "recis_b200.framework.trainer": ["Trainer", "TrainingArguments"], "recis_b200.framework.checkpoint_manager": ["CheckpointManager"],
        "recis_b200.metrics.auroc": ["AUROC"], "recis_b200.metrics.gauc": ["Gauc"],
        "recis_b200.serialize.checkpoint_reader": ["CheckpointReader"], "recis_b200.utils.logger": ["Logger"],
        "recis_b200.utils.data_utils": ["copy_data_to_device"],
    }.items():
        m = importlib.import_module(mod)
        for n in names:
            assert hasattr(m, n), (mod, n)


def test_three_stage_lookup_interface_matches_forward():
    """exchange_ids -> lookup_exchange_emb -> emb_reduce (the reference's staged interface) gives what forward() gives."""
    from recis_b200.nn import DynamicEmbedding, EmbeddingOption
    from recis_b200.nn.initializers import NormalInitializer
    from recis_b200.ragged import RaggedTensor
    emb = DynamicEmbedding(EmbeddingOption(embedding_dim=8, shared_name="staged_api", combiner="mean", initializer=NormalInitializer(0, 0.1)))
    ids = torch.tensor([5, 9, 5, 77, 1 << 40, 9], dtype=torch.int64)
    offsets = torch.tensor([0, 2, 2, 5, 6], dtype=torch.int32)
    want = emb(RaggedTensor(ids, [offsets]))
    r1 = emb.exchange_ids(ids, offsets)
    r2 = emb.wait_exchange_emb(emb.lookup_exchange_emb(r1))
    got = emb.emb_reduce(r2, None, "mean", {})
    assert torch.allclose(got.view_as(want), want)
    assert emb.emb_reduce(emb.lookup_exchange_emb(emb.exchange_ids(ids, offsets)), None, "sum", fp16_enable=True).dtype == torch.float16
