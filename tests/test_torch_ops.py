"""``torch.ops.recis.*``: the reference's operator names (``csrc/bind.cc:46-211``) resolve on this framework and compute what the
reference's Python layer expects from them."""
import torch

import recis_b200.torch_ops as T

REFERENCE_NAMES = """ragged_to_dense ragged_to_sparse uint64_mod bucketize_op fused_multi_hash gauc_calc adam_tf_apply segment_mean segment_sum
block_insert block_insert_with_mask block_gather block_filter gather block_apply_adamw generate_ids free_ids mask_key_index
scatter_ids_with_mask ids_encode merge_offsets ids_partition segment_reduce_forward segment_reduce_backward gen_segment_indices_by_offset
dense_to_ragged fused_uint64_mod fused_bucketized fused_hash fused_ragged_cutoff fused_ragged_cutoff_3D feature_cross_ragged ragged_tile
ragged_tile_back calc_ragged_index""".split()


def test_every_reference_operator_name_resolves():
    assert T.register()
    for name in REFERENCE_NAMES:
        assert hasattr(torch.ops.recis, name), name
    assert callable(T.make_hashtable)


def test_embedding_operators():
    o = torch.ops.recis
    ids = torch.tensor([5, 65536 + 5, 5, 40000])
    uniq, counts, rev = o.ids_partition(ids, 2)
    assert counts.tolist() == [2, 1] and torch.equal(uniq[rev], ids)
    assert o.ids_encode([torch.tensor([1, 2]), torch.tensor([3])], torch.tensor([0, 2])).tolist() == [1, 2, 3 | (2 << 52)]
    assert o.merge_offsets([torch.tensor([0, 2, 3]), torch.tensor([0, 1, 4])], torch.tensor(0)).tolist() == [0, 2, 3, 4, 7]
    assert o.gen_segment_indices_by_offset(torch.tensor([0, 2, 2, 5])).tolist() == [0, 0, 2, 2, 2]
    emb = torch.randn(4, 3)
    rev = torch.tensor([0, 1, 1, 3]); offs = torch.tensor([0, 2, 4])
    fwd = o.segment_reduce_forward(emb, None, rev, offs, "mean")
    assert torch.allclose(fwd, torch.stack([(emb[0] + emb[1]) / 2, (emb[1] + emb[3]) / 2]), atol=1e-6)
    x = emb.clone().requires_grad_(True)
    torch.stack([(x[0] + x[1]) / 2, (x[1] + x[3]) / 2]).backward(torch.ones(2, 3))
    assert torch.allclose(o.segment_reduce_backward(torch.ones(2, 3), None, rev, offs, 4, "mean"), x.grad)
    w = torch.tensor([1.0, 3.0, 2.0, 2.0])
    assert torch.allclose(o.segment_mean(emb, w, torch.tensor([0, 0, 1, 1]), 2), torch.tensor([0.25, 0.75, 0.5, 0.5]))
    data = torch.arange(6.0).view(3, 2)
    assert o.segment_sum(data, torch.tensor([1.0, 2.0]), torch.tensor([0, 2]), torch.tensor([0, 0]), 2).tolist() == [[8.0, 11.0], [0.0, 0.0]]


def test_ragged_and_feature_operators():
    o = torch.ops.recis
    v, off = o.dense_to_ragged(torch.tensor([[1, 2, 0], [3, 0, 0]]), True, torch.tensor(0))
    assert v.tolist() == [1, 2, 3] and off.tolist() == [0, 2, 3]
    assert o.ragged_to_dense(v, [off], 0).tolist() == [[1, 2], [3, 0]]
    assert o.bucketize_op(torch.tensor([0.5, 2.5]), torch.tensor([1.0, 2.0])).tolist() == [0, 2]
    assert o.uint64_mod(torch.tensor([10, -1]), 7).tolist() == [3, ((1 << 64) - 1) % 7]
    vals, offs, drops, pads = o.fused_ragged_cutoff([torch.arange(5)], [torch.tensor([0, 3, 5], dtype=torch.int32)],
                                                    torch.tensor([2], dtype=torch.int32), torch.tensor([True]), torch.tensor([False]))
    assert vals[0].tolist() == [1, 2, 3, 4] and offs[0].tolist() == [0, 2, 4] and drops[0].tolist() == [1, 0] and pads[0].tolist() == [0, 0]
    ids, o2, w = o.feature_cross_ragged(torch.tensor([1, 2, 1, 3]), torch.tensor([0, 3, 4]), torch.tensor([1.0, 2.0, 5.0, 3.0]),
                                        torch.tensor([7, 7, 8, 9]), torch.tensor([0, 2, 4]), torch.empty(0))
    assert o2.tolist() == [0, 2, 4] and w.tolist() == [1.0, 2.0, 3.0, 3.0] and len(set(ids.tolist())) == 4
    aucs, counts = o.gauc_calc(torch.tensor([1.0, 0.0, 1.0, 0.0]), torch.tensor([0.9, 0.1, 0.2, 0.8]), torch.tensor([0, 0, 1, 1]))
    assert aucs.tolist() == [1.0, 0.0] and counts.tolist() == [2, 2]


def test_block_storage_and_allocator_shims():
    o = torch.ops.recis
    blocks = [torch.zeros(4, 2), torch.zeros(4, 2)]
    o.block_insert(torch.tensor([1, 6]), torch.ones(2, 2), blocks, 4)
    assert blocks[0][1].tolist() == [1, 1] and blocks[1][2].tolist() == [1, 1]
    assert o.block_gather(torch.tensor([1, 6, -1]), blocks, 4, -1, True).tolist() == [[1, 1], [1, 1], [0, 0]]
    o.block_insert_with_mask(torch.tensor([0, 3]), torch.full((2, 2), 5.0), torch.tensor([False, True]), blocks, 4)
    assert blocks[0][0].tolist() == [0, 0] and blocks[0][3].tolist() == [5, 5]
    steps = [torch.tensor([3, 9, 1, 7])]
    assert o.block_filter(torch.tensor([0, 1, 2]), steps, 4, 5).tolist() == [True, False, True]
    assert o.generate_ids(4, [torch.tensor([7, 8, 9, 0])], 3, 100, 4).tolist() == [100, 7, 8, 9]
    free = [torch.zeros(4, dtype=torch.int64)]
    o.free_ids(torch.tensor([11, 12]), free, 1, 4)
    assert free[0].tolist() == [0, 11, 12, 0]
    assert o.gather(torch.tensor([2, 0]), torch.arange(6.0).view(3, 2)).tolist() == [[4, 5], [0, 1]]
    # one AdamW step on block storage against the formula
    emb = [torch.ones(4, 2)]; m = [torch.zeros(4, 2)]; v = [torch.zeros(4, 2)]
    b1, b2 = torch.tensor(1.0), torch.tensor(1.0)
    o.block_apply_adamw(torch.tensor([2]), torch.full((1, 2), 0.5), emb, b1, b2, torch.tensor(1), m, v, 0.1, 0.9, 0.999, 0.0, 1e-8, 4)
    assert abs(float(emb[0][2, 0]) - (1.0 - 0.1)) < 1e-4 and float(emb[0][1, 0]) == 1.0
    p, g, a, s = torch.ones(3), torch.full((3,), 2.0), torch.zeros(3), torch.zeros(3)
    o.adam_tf_apply(p, g, a, s, 1, 0.1, 0.9, 0.999, 1e-8)
    assert torch.allclose(p, torch.full((3,), 0.9), atol=1e-4)
