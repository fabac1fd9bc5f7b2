"""Embedding rows stored in float16 / bfloat16 (trainable) and int8 (read-only, served as float16 or float32), as the reference
dispatches its row kernels over these types (``csrc/ops/block_ops_kernel.cu:236-273``, ``recis/nn/modules/embedding.py:610-615``).
Optimizer state and every accumulation stay fp32; the oracle is the same computation on an fp32 table."""
import pytest
import torch

from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param
from recis_b200.nn.initializers import NormalInitializer
from recis_b200.nn.modules.hashtable import HashtableRegister
from recis_b200.optim import SparseAdagrad, SparseAdam

DEVICES = ["cpu"] + (["cuda"] if torch.cuda.is_available() else [])


def _train(dtype, device, opt_cls, steps=4, dim=16):
    HashtableRegister().clear()
    torch.manual_seed(5)
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=dim, shared_name=f"rd_{dtype}_{opt_cls.__name__}", dtype=dtype, device=device,
                                                combiner="sum", initializer=NormalInitializer(0, 0.1)),
                           "b": EmbeddingOption(embedding_dim=dim, shared_name=f"rd_b_{dtype}_{opt_cls.__name__}", dtype=dtype, device=device,
                                                combiner="mean", initializer=NormalInitializer(0, 0.1))})
    opt = opt_cls(filter_out_sparse_param(eng), lr=0.05)
    outs = []
    for step in range(steps):
        g = torch.Generator().manual_seed(step)
        feats = {n: torch.randint(0, 50, (24, 3), generator=g).to(device) for n in ("a", "b")}
        coef = {n: torch.randn(24, dim, generator=g).to(device) for n in ("a", "b")}
        opt.zero_grad()
        out = eng(feats)
        sum((out[n].float() * coef[n]).sum() for n in out).backward()
        opt.step()
        outs.append({n: out[n].detach().float().cpu() for n in out})
    (table,) = eng.tables().values()
    ids, rows = table.impl.ids_map()
    order = torch.argsort(ids)
    emb = table.impl.store.emb()
    return outs, ids[order].cpu(), emb[rows[order]].float().cpu(), emb


@pytest.mark.parametrize("device", [pytest.param(d, marks=pytest.mark.gpu) if d == "cuda" else d for d in DEVICES])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("opt_cls", [SparseAdam, SparseAdagrad])
def test_half_precision_rows_train_like_fp32_rows(device, dtype, opt_cls):
    outs, ids, rows, slab = _train(dtype, device, opt_cls)
    ref_outs, ref_ids, ref_rows, ref_slab = _train(torch.float32, device, opt_cls)
    assert slab.dtype == dtype and slab.element_size() == 2 and ref_slab.dtype == torch.float32      # rows really are 2 bytes wide
    assert torch.equal(ids, ref_ids)
    tol = 4e-2 if dtype == torch.bfloat16 else 6e-3
    assert outs[0]["a"].dtype == torch.float32                       # (cast back by the test) the model saw the table dtype
    for o, r in zip(outs, ref_outs):
        for n in o:
            assert torch.allclose(o[n], r[n], atol=tol, rtol=tol), (n, float((o[n] - r[n]).abs().max()))
    assert float((rows - ref_rows).abs().max()) < tol


@pytest.mark.parametrize("device", [pytest.param(d, marks=pytest.mark.gpu) if d == "cuda" else d for d in DEVICES])
def test_model_sees_the_table_dtype(device):
    HashtableRegister().clear()
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name="rd_see", dtype=torch.bfloat16, device=device)})
    assert eng({"a": torch.arange(10).view(5, 2).to(device)})["a"].dtype == torch.bfloat16


@pytest.mark.parametrize("device", [pytest.param(d, marks=pytest.mark.gpu) if d == "cuda" else d for d in DEVICES])
@pytest.mark.parametrize("fp16", [True, False])
def test_int8_table_is_read_only_and_served_upcast(device, fp16):
    HashtableRegister().clear()
    dim = 16
    eng = EmbeddingEngine({"q": EmbeddingOption(embedding_dim=dim, shared_name=f"rd_q_{fp16}", dtype=torch.int8, device=device, combiner="sum",
                                                fp16_enabled=fp16)})
    (table,) = eng.tables().values()
    ids = torch.arange(40)
    vals = torch.randint(-100, 100, (40, dim), dtype=torch.int8)
    # ids of a merged table carry the child prefix; a single child has index 0, so the raw ids are the table's ids
    table.impl.insert(ids, vals)
    assert table.impl.store.emb().dtype == torch.int8 and not table.impl.trainable
    bags = torch.randint(0, 40, (6, 4))
    out = eng({"q": bags.to(device)})["q"]
    assert out.dtype == (torch.float16 if fp16 else torch.float32)
    ref = vals.float()[bags].sum(1)
    assert torch.allclose(out.float().cpu(), ref, atol=0.51)
    # unknown ids read as zeros, nothing is inserted, and a backward pass stages nothing
    before = table.impl.size()
    eng.train()
    out = eng({"q": torch.tensor([[1000, 1001]]).to(device)})["q"]
    assert float(out.detach().float().abs().sum()) == 0 and table.impl.size() == before
    if out.requires_grad:
        out.float().sum().backward()
    assert not table.impl.records()


def test_bf16_rows_round_trip_through_the_checkpoint_bundle(tmp_path):
    from recis_b200.serialize import CheckpointReader, Loader, Saver
    HashtableRegister().clear()
    torch.manual_seed(0)
    mk = lambda: EmbeddingEngine({"a": EmbeddingOption(embedding_dim=8, shared_name="rd_ckpt", dtype=torch.bfloat16, device="cpu",
                                                       initializer=NormalInitializer(0, 0.1))})
    eng = mk()
    opt = SparseAdam(filter_out_sparse_param(eng), lr=0.01)
    out = eng({"a": torch.arange(64).view(16, 4)})["a"]
    out.float().sum().backward(); opt.step()
    Saver(0, 1, 1, str(tmp_path), filter_out_sparse_param(eng), {}).save()
    reader = CheckpointReader(str(tmp_path))
    emb_names = [n for n in reader.list_tensors() if n.endswith("@embedding")]
    assert emb_names and all(reader.tensor_dtype(n) == torch.bfloat16 for n in emb_names)        # a BF16 slot on disk
    state_names = [n for n in reader.list_tensors() if "exp_avg" in n]
    assert state_names and all(reader.tensor_dtype(n) == torch.float32 for n in state_names)     # optimizer state stays fp32
    HashtableRegister().clear()
    eng2 = mk()
    opt2 = SparseAdam(filter_out_sparse_param(eng2), lr=0.01)
    Loader(str(tmp_path), filter_out_sparse_param(eng2), {}).load()
    t1, t2 = next(iter(eng.tables().values())).impl, next(iter(eng2.tables().values())).impl
    i1, r1 = t1.ids_map(); i2, r2 = t2.ids_map()
    o1, o2 = torch.argsort(i1), torch.argsort(i2)
    assert torch.equal(i1[o1], i2[o2])
    assert torch.equal(t1.store.emb()[r1[o1]], t2.store.emb()[r2[o2]])                           # bit-identical 2-byte rows
    for slot in t1.store.slot_names():
        assert torch.equal(t1.store.slot(slot)[r1[o1]], t2.store.slot(slot)[r2[o2]])
