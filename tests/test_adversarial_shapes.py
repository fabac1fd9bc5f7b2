"""Edge shapes for the sparse path on CPU (the CPU kernels are the oracles of the GPU ones): odd and tiny widths, empty bags,
empty batches, all-duplicate ids, negative ids / ids with high bits set, world sizes that do not divide the slice space."""
import pytest
import torch

import recis_b200
from recis_b200.nn import EmbeddingEngine, EmbeddingOption, filter_out_sparse_param, gen_slice
from recis_b200.nn.initializers import NormalInitializer
from recis_b200.nn.modules.hashtable import HashtableRegister
from recis_b200.optim import SparseAdam
from recis_b200.ragged import RaggedTensor

C = recis_b200.native()


@pytest.fixture(autouse=True)
def _fresh():
    HashtableRegister().clear()
    yield
    HashtableRegister().clear()


@pytest.mark.parametrize("world", [1, 3, 7, 13])
def test_dedup_partition_edge_inputs(world):
    for ids in (torch.zeros(0, dtype=torch.int64), torch.tensor([-1]), torch.full((1000,), 42, dtype=torch.int64),
                torch.tensor([-1, -2, -(1 << 62), (1 << 63) - 1, 0, 65535, 65536, -65536]),
                torch.arange(-3000, 3000, dtype=torch.int64) * 65537):
        uniq, rev, counts, offs = C.dedup_partition(ids, world)
        nu = int(offs[-1])
        assert nu == ids.unique().numel() and int(counts.sum()) == nu
        if ids.numel():
            assert torch.equal(uniq[:nu][rev.long()], ids)
        for r in range(world):
            sl = gen_slice(r, world)
            low = uniq[offs[r]:offs[r + 1]] & 0xFFFF                       # routing by the low 16 bits of the two's-complement id
            assert bool(((low >= sl.slice_begin) & (low < sl.slice_end)).all())
    # the slice ranges of all ranks tile [0, 65536) exactly, with the first 65536 % world ranks one slice larger
    sizes = [gen_slice(r, world).slice_end - gen_slice(r, world).slice_begin for r in range(world)]
    assert sum(sizes) == 65536 and max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


@pytest.mark.parametrize("dim", [1, 3, 8, 16, 64, 128])
@pytest.mark.parametrize("combiner", ["sum", "mean"])
def test_engine_matches_embedding_bag_on_edge_bags(dim, combiner):
    torch.manual_seed(dim)
    eng = EmbeddingEngine({"f": EmbeddingOption(embedding_dim=dim, shared_name="f", device="cpu", combiner=combiner, use_weight=False,
                                                initializer=NormalInitializer(0, 1))})
    opt = SparseAdam(filter_out_sparse_param(eng), lr=0.1)
    # bags: empty, single, all duplicates, negative ids and ids with the top bits set (only the low 52 bits address a row)
    bags = [[], [5], [7, 7, 7, 7], [-1, -2, 1 << 60, (1 << 60) + 1], [], [5, 7, -1]]
    values = torch.tensor([v for b in bags for v in b], dtype=torch.int64)
    offsets = torch.tensor([0] + [sum(len(b) for b in bags[:i + 1]) for i in range(len(bags))], dtype=torch.int32)
    out = eng({"f": RaggedTensor(values, [offsets])})["f"]
    (t,) = eng.tables().values()
    keys, rows = t.impl.ids_map()
    row_of = {int(k): t.impl.store.emb()[r].clone() for k, r in zip(keys.tolist(), rows.tolist())}
    mask52 = (1 << 52) - 1
    want = torch.zeros(len(bags), dim)
    for i, b in enumerate(bags):
        for v in b:
            want[i] += row_of[v & mask52]
        if combiner == "mean" and b:
            want[i] /= len(b)
    assert torch.allclose(out, want, atol=1e-6)
    assert len(row_of) == len({v & mask52 for v in values.tolist()})
    # one optimizer step on these bags keeps the table consistent (duplicates inside a bag are summed, empty bags contribute nothing)
    out.sum().backward()
    opt.step()
    out2 = eng({"f": RaggedTensor(values, [offsets])})["f"]
    assert torch.isfinite(out2).all() and not torch.allclose(out2[1], out[1])
    assert torch.equal(out2[0], torch.zeros(dim)) and torch.equal(out2[4], torch.zeros(dim))


def test_empty_batch_and_empty_feature():
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu", use_weight=False),
                           "b": EmbeddingOption(embedding_dim=4, shared_name="b", device="cpu", use_weight=False)})
    off = torch.zeros(4, dtype=torch.int32)
    out = eng({"a": RaggedTensor(torch.zeros(0, dtype=torch.int64), [off]), "b": RaggedTensor(torch.tensor([1, 2, 3]), [torch.tensor([0, 1, 2, 3], dtype=torch.int32)])})
    assert out["a"].shape == (3, 4) and float(out["a"].detach().abs().sum()) == 0 and out["b"].shape == (3, 4)


def test_debug_bounds_rejects_malformed_ragged_inputs(monkeypatch):
    monkeypatch.setenv("RECIS_DEBUG_BOUNDS", "1")
    eng = EmbeddingEngine({"a": EmbeddingOption(embedding_dim=4, shared_name="a", device="cpu", use_weight=False)})
    vals = torch.arange(6)
    ok = eng({"a": RaggedTensor(vals, [torch.tensor([0, 2, 6], dtype=torch.int32)])})["a"]
    assert ok.shape == (2, 4)
    for bad, msg in (([1, 2, 6], "start at 0"), ([0, 4, 3, 6], "decrease"), ([0, 2, 5], "does not match")):
        with pytest.raises(ValueError, match=msg):
            eng({"a": RaggedTensor(vals, [torch.tensor(bad, dtype=torch.int32)])})
