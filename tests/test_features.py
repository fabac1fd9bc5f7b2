"""Feature engine, fused feature ops and ragged ops against plain PyTorch / Python references (CPU)."""
import pytest
import torch

from recis_b200.features import (Bucketize, Feature, FeatureCross, FeatureEngine, Hash, IDMultiHash, Mod, SelectField, SelectFields,
                                 SequenceTruncate)
from recis_b200.nn.functional import array_ops, embedding_ops, fused_ops, hash_ops, ragged_ops
from recis_b200.ragged import RaggedTensor


def _bytes_ragged(strings):
    data = b"".join(strings)
    offs = [0]
    for s in strings:
        offs.append(offs[-1] + len(s))
    return torch.tensor(list(data), dtype=torch.uint8).view(torch.int8), torch.tensor(offs, dtype=torch.int32)


def test_hash_golden_vectors():
    # vectors of the reference's own unit test (tests/ops/fused_hash_test.py)
    inputs = [torch.tensor([0, 1, 2, 1, 2, 3], dtype=torch.int8), torch.tensor([0, 5, 5, 5, 6, 7], dtype=torch.int8)]
    offs = [torch.tensor([0, 3, 6], dtype=torch.int32)] * 2
    farm = hash_ops.farmhash(inputs, offs)
    assert farm[0].tolist() == [-7736835464683084646, -5546720800891377920]
    assert farm[1].tolist() == [-4442022684725028445, -909183002746659612]
    mur = hash_ops.murmurhash(inputs, offs)
    assert mur[0].tolist() == [-4003751876240412087, -1042754718167355375]
    assert mur[1].tolist() == [-5541886947548579749, 4434088491466393040]


def test_murmur_matches_python_restatement():
    def murmur(data: bytes):
        m, r, mask = 0xc6a4a7935bd1e995, 47, (1 << 64) - 1
        n = len(data)
        h = (n * m) & mask
        i = 0
        while n - i >= 8:
            k = int.from_bytes(data[i:i + 8], "little")
            k = (k * m) & mask; k ^= k >> r; k = (k * m) & mask
            h ^= k; h = (h * m) & mask
            i += 8
        if n - i:
            h ^= int.from_bytes(data[i:], "little"); h = (h * m) & mask
        h ^= h >> r; h = (h * m) & mask; h ^= h >> r
        return h - (1 << 64) if h >= (1 << 63) else h
    strings = [bytes((7 * i + j) % 251 for j in range(i)) for i in range(0, 90, 3)]
    v, o = _bytes_ragged(strings)
    out = hash_ops.murmurhash([v], [o])[0].tolist()
    assert out == [murmur(s) for s in strings]


def test_bucketize_mod_multihash():
    b = torch.tensor([1.0, 2.0, 2.0, 5.0])
    x = torch.tensor([[0.5, 1.0], [2.0, 7.0]])
    assert array_ops.bucketize(x, b).tolist() == [[0, 1], [3, 4]]
    assert torch.equal(array_ops.bucketize(x, b), torch.bucketize(x, b, right=True))
    ids = torch.tensor([-1, 10, 2 ** 62 + 5])
    assert array_ops.bucketize_mod(ids, 7).tolist() == [((1 << 64) - 1) % 7, 3, (2 ** 62 + 5) % 7]
    mh = array_ops.multi_hash(torch.tensor([5, -3, 100]), [1, 3], [29, 47], [10, 10])
    assert mh[0].tolist() == [5 % 29 % 10, ((-3 % 29) + 29) % 29 % 10, 100 % 29 % 10]
    assert mh[1].tolist() == [15 % 47 % 10, ((-9 % 47) + 47) % 47 % 10, 300 % 47 % 10]
    outs = fused_ops.fused_bucketize_gpu([x, x + 1], [b, b])
    assert torch.equal(outs[1], torch.bucketize(x + 1, b, right=True))


def test_ragged_dense_roundtrip_and_sparse():
    v = torch.arange(1, 8)
    off = [torch.tensor([0, 2, 2, 3]), torch.tensor([0, 3, 5, 7])]
    dense = ragged_ops.ragged_to_dense(v, off, 0)
    assert dense.shape == (3, 2, 3)
    assert dense[0].tolist() == [[1, 2, 3], [4, 5, 0]] and dense[2].tolist() == [[6, 7, 0], [0, 0, 0]]
    sp = ragged_ops.ragged_to_sparse(v, off)
    assert torch.equal(sp.to_dense(), dense)
    vals, offs = ragged_ops.dense_to_ragged(torch.tensor([[1, 2, 0], [0, 0, 0], [3, 0, 4]]), True, 0)
    assert vals.tolist() == [1, 2, 3, 0, 4] and offs[0].tolist() == [0, 2, 2, 5]
    r = RaggedTensor(torch.arange(5.0), [torch.tensor([0, 2, 5])])
    assert r.to_dense().tolist() == [[0, 1, 0], [2, 3, 4]]
    assert RaggedTensor.from_dense(r.to_dense()).values().numel() == 6


def test_cutoff_2d_and_3d():
    v, o, d, p, _, _ = ragged_ops.fused_ragged_cutoff_2D(
        [torch.arange(10), torch.arange(10)], [torch.tensor([0, 4, 5, 10])] * 2, torch.tensor([3, 2]),
        torch.tensor([True, False]), torch.tensor([False, False]))
    assert v[0].tolist() == [1, 2, 3, 4, 7, 8, 9] and o[0].tolist() == [0, 3, 4, 7]
    assert v[1].tolist() == [0, 1, 4, 5, 6] and o[1].tolist() == [0, 2, 3, 5]
    assert d[0].tolist() == [1, 0, 2] and p[0].tolist() == [0, 2, 0]
    vals, offs = ragged_ops.fused_ragged_cutoff_3D(
        [torch.arange(1, 8)], [[torch.tensor([0, 3, 4]), torch.tensor([0, 2, 3, 5, 7])]], torch.tensor([2]),
        torch.tensor([True]), torch.tensor([False]))
    # sample 0 has rows [1,2] [3] [4,5] -> keep the last two; sample 1 has one row [6,7] -> one empty row padded on the right
    assert vals[0].tolist() == [3, 4, 5, 6, 7]
    assert offs[0][0].tolist() == [0, 2, 4] and offs[0][1].tolist() == [0, 1, 3, 5, 5]


def test_topk_index_cutoff_and_feature_cross():
    idx, off = ragged_ops.ragged_topk_index_cutoff(
        torch.tensor([5, 0, 0]), torch.tensor([0, 0, 0]), torch.tensor(True), torch.tensor(False),
        torch.tensor([0, 8, 10, 13], dtype=torch.int32), torch.tensor([[1, 2], [0, 2], [0, 1]]), torch.tensor([0, 1, 2]))
    assert idx.tolist() == [6, 7, 8, 10, 11] and off.tolist() == [0, 2, 3, 5]
    vals, offs, w = ragged_ops.feature_cross_ragged(torch.tensor([1, 2, 1, 3]), torch.tensor([0, 3, 4]), torch.tensor([7, 7, 8, 9]),
                                                    torch.tensor([0, 2, 4]), torch.tensor([1.0, 2.0, 5.0, 3.0]), None)
    assert offs.tolist() == [0, 2, 4] and w.tolist() == [1.0, 2.0, 3.0, 3.0]
    assert len(set(vals.tolist())) == 4


def test_segment_reduce_autograd():
    torch.manual_seed(0)
    emb = torch.randn(10, 4, requires_grad=True)
    idx = torch.tensor([1, 3, 3, 7, 0])
    off = torch.tensor([0, 2, 2, 5])
    w = torch.tensor([1.0, 2.0, 0.5, 1.0, 3.0])
    out = embedding_ops.ragged_embedding_segment_reduce(emb, w, idx, off, "mean")
    ref = torch.stack([(emb[[1, 3]] * w[:2, None]).sum(0) / 2, torch.zeros(4), (emb[[3, 7, 0]] * w[2:, None]).sum(0) / 3])
    assert torch.allclose(out, ref, atol=1e-6)
    g = torch.autograd.grad(out.sum(), emb)[0]
    gr = torch.autograd.grad(ref.sum(), emb)[0]
    assert torch.allclose(g, gr, atol=1e-6)
    uniq, counts, rev = embedding_ops.ids_partition(torch.tensor([5, 65536 + 5, 5, 40000]), 65536, 2)
    assert counts.tolist() == [2, 1] and torch.equal(uniq[rev.long()], torch.tensor([5, 65536 + 5, 5, 40000]))
    enc = embedding_ops.ids_encode([torch.tensor([1, 2]), torch.tensor([3])], [0, 2])
    assert enc.tolist() == [1, 2, 3 | (2 << 52)]


def test_feature_engine_fuses_and_dedups():
    strings = [b"user_1", b"user_22", b"u", b"a-much-longer-user-identifier-string-0123456789-0123456789-0123456789-abcdefgh"]
    sv, so = _bytes_ragged(strings)
    batch = {
        "uid": RaggedTensor(sv, [torch.tensor([0, 1, 3, 4]), so]),            # 3 samples, strings per sample 1,2,1
        "price": torch.tensor([[0.5], [3.0], [10.0]]),
        "item": RaggedTensor(torch.arange(12), [torch.tensor([0, 5, 6, 12])]),
        "label": torch.ones(3, 1),
    }
    feats = [
        Feature("uid_h").add_op(SelectField("uid")).add_op(Hash("farm")).add_op(Mod(1000)),
        Feature("uid_m").add_op(SelectField("uid")).add_op(Hash("murmur")).add_op(Mod(1000)),
        Feature("price_b").add_op(SelectField("price")).add_op(Bucketize([1.0, 5.0])),
        Feature("item_t").add_op(SelectField("item")).add_op(Mod(7)).add_op(SequenceTruncate(seq_len=3, truncate_side="right")),
        Feature("item_mh").add_op(SelectField("item")).add_op(IDMultiHash([11, 13])),
        Feature("cross").add_op(SelectFields([SelectField("item"), SelectField("item")])).add_op(FeatureCross()),
    ]
    fe = FeatureEngine(feats)
    assert len(fe.plan) == 3
    # step 1 holds one fused Hash launch (both hash features), one fused Bucketize launch, one fused Mod launch, ...
    kinds = [launch.kind for launch in fe.plan[1]]
    assert {"Hash", "Bucketize", "Mod", "IDMultiHash"} <= set(kinds) and kinds.count("Hash") == 1
    assert next(launch for launch in fe.plan[1] if launch.kind == "Hash").names == ("uid_h", "uid_m")
    out = fe(batch)
    assert out["label"] is batch["label"]
    assert out["price_b"].tolist() == [[0], [1], [2]]
    assert isinstance(out["uid_h"], RaggedTensor) and out["uid_h"].values().shape == (4,)
    assert out["uid_h"].offsets()[0].tolist() == [0, 1, 3, 4]
    direct = hash_ops.farmhash([sv], [so])[0]
    assert torch.equal(out["uid_h"].values(), array_ops.bucketize_mod(direct, 1000))
    assert out["item_t"].values().tolist() == [0, 1, 2, 5, 6, 0, 1] and out["item_t"].offsets()[0].tolist() == [0, 3, 4, 7]
    assert set(out["item_mh"]) == {"multi_hash_0", "multi_hash_1"}
    assert out["cross"].offsets()[-1].tolist() == [0, 25, 26, 62]


def test_duplicate_features_computed_once():
    a = Feature("x").add_op(SelectField("raw")).add_op(Mod(10))
    b = Feature("x").add_op(SelectField("raw")).add_op(Mod(10))
    fe = FeatureEngine([a, b])
    assert len(fe._features) == 1


def test_same_chain_under_two_names_is_computed_once_and_op_order_matters():
    calls = []

    class Probe(Mod):
        def forward(self, x):
            calls.append(1)
            return super().forward(x)

    a = Feature("a").add_op(SelectField("raw")).add_op(Probe(10))
    b = Feature("b").add_op(SelectField("raw")).add_op(Probe(10))
    c = Feature("c").add_op(SelectField("raw")).add_op(Mod(7)).add_op(Mod(5))
    d = Feature("d").add_op(SelectField("raw")).add_op(Mod(5)).add_op(Mod(7))
    assert a.get_hash() == b.get_hash() and c.get_hash() != d.get_hash()
    fe = FeatureEngine([a, b, c, d])
    out = fe({"raw": torch.arange(40).view(-1, 1)})
    assert len(calls) == 1 and out["b"] is out["a"]
    assert torch.equal(out["c"], (torch.arange(40).view(-1, 1) % 7) % 5) and torch.equal(out["d"], (torch.arange(40).view(-1, 1) % 5) % 7)
