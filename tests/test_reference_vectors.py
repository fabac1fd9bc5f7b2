"""Inputs and expected outputs taken from the reference project's own unit tests (read as text), run against this framework on
CPU: tests/metrics/gauc_test.py, tests/ops/ragged_topk_index_cutoff_test.py, tests/ops/dense_to_ragged_test.py,
tests/ops/ragged_to_dense_test.py (docstring example), tests/ops/ids_encode_test.py (re-statement used as its oracle),
tests/ops/fused_ragged_cutoff_2D_test.py (inputs; expected values from the row-wise definition of the op)."""
import torch

from recis_b200.metrics.gauc import Gauc
from recis_b200.nn.functional import fused_ops, ragged_ops


def test_gauc_vector():
    cur, acc = Gauc(dist_sync=False)(torch.tensor([1.0, 0.0, 1, 0, 1]), torch.tensor([0.1, 0.2, 0.3, 0.4, 0.5]), torch.tensor([0, 1, 1, 1, 2]))
    assert cur == 0.5 and acc == 0.5


def test_ragged_topk_index_cutoff_vector():
    vi, off = ragged_ops.ragged_topk_index_cutoff(torch.tensor([5, 0, 0]), torch.tensor([0, 0, 0]), torch.tensor(True), torch.tensor(False),
                                                  torch.tensor([0, 8, 10, 13], dtype=torch.int32), torch.tensor([[1, 2], [0, 2], [0, 1]]),
                                                  torch.tensor([0, 1, 2]))
    assert vi.tolist() == [6, 7, 8, 10, 11] and off.tolist() == [0, 2, 3, 5]


def test_dense_to_ragged_vectors():
    for dtype in (torch.int32, torch.float32, torch.int64):
        for row0, vals in (([1, 0, 3, 0, 0], [1, 0, 3, 6, 7, 8]), ([1, 2, 3, 0, 0], [1, 2, 3, 6, 7, 8])):
            data = torch.tensor([row0, [6, 7, 8, 0, 0]]).to(dtype)
            v, offs = ragged_ops.dense_to_ragged(data, True, 0)
            assert v.tolist() == vals and offs[0].tolist() == [0, 3, 6]
    v, offs = ragged_ops.dense_to_ragged(torch.tensor([[1, 2, 3, 0, 0], [6, 7, 8, 0, 0]], dtype=torch.int32), False, 0)
    assert v.numel() == 10 and offs[0].tolist() == [0, 5, 10]


def test_ragged_to_dense_docstring_example():
    out = ragged_ops.ragged_to_dense(torch.tensor([1, 2, 3, 4, 5, 6, 7, 8, 9, 9, 10, 11, 12]),
                                     [torch.tensor([0, 2, 2, 3, 6]), torch.tensor([0, 2, 4, 6, 9, 11, 13])], default_value=0)
    assert out.tolist() == [[[1, 2, 0], [3, 4, 0], [0, 0, 0]], [[0, 0, 0], [0, 0, 0], [0, 0, 0]], [[5, 6, 0], [0, 0, 0], [0, 0, 0]],
                            [[7, 8, 9], [9, 10, 0], [11, 12, 0]]]


def test_ids_encode_restatement():
    torch.manual_seed(0)
    ids_list = [torch.randint(0, 1000000, (n,), dtype=torch.int64) for n in (10, 100, 1000)]
    ids_list[0][0] = -5                                   # high bits set: only the low 52 bits survive
    table = torch.arange(0, 3, dtype=torch.int64)
    want = torch.cat([torch.bitwise_and(ids, (1 << 52) - 1) + (t << 52) for ids, t in zip(ids_list, table)])
    assert torch.equal(fused_ops.fused_ids_encode_gpu(ids_list, table), want)


def test_fused_ragged_cutoff_2d_inputs_of_the_reference_test():
    vals = [torch.tensor([9155707040084860980, 11, 12, 20, 21, 30, 31, 32, 33]), torch.tensor([7, 1, 2, 3, 4, 5, 6]),
            torch.tensor([-7, -1, -2, -3, -4, -5, -6])]
    offs = [torch.tensor([0, 3, 5, 9], dtype=torch.int32), torch.tensor([0, 1, 7], dtype=torch.int32),
            torch.tensor([0, 1, 2, 4, 7], dtype=torch.int32)]
    keep = torch.tensor([3, 4, 2], dtype=torch.int32)
    drop_left = torch.tensor([False, False, True])
    pad_left = torch.tensor([False, False, True])
    out_v, out_o, drops, pads, _ds, _ps = ragged_ops.fused_ragged_cutoff_2D(vals, offs, keep, drop_left, pad_left)
    for v, o, k, dl, ov, oo in zip(vals, offs, keep.tolist(), drop_left.tolist(), out_v, out_o):
        want_v, want_o = [], [0]
        for r in range(o.numel() - 1):
            row = v[int(o[r]):int(o[r + 1])].tolist()
            row = row[len(row) - k:] if (dl and len(row) > k) else row[:k]      # rows are shortened, never padded, in 2-D
            want_v += row
            want_o.append(len(want_v))
        assert ov.tolist() == want_v and oo.tolist() == want_o
