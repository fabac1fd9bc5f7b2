"""``torch.ops.recis.*``: the reference's operator names on this framework's kernels.

The reference registers its native operators with ``TORCH_LIBRARY(recis, ...)`` (``csrc/bind.cc:46-211``) and its Python layer
calls them as ``torch.ops.recis.<name>``. Code written against those names (user models, the reference's own tests) finds them
here after ``import recis_b200.torch_ops``: every operator is defined with the reference's argument list and dispatched to the
implementation of this package (the sm_100a kernels on CUDA tensors, their CPU twins otherwise).

Registration is explicit, not a side effect of ``import recis_b200``: a process can hold only one definition of the ``recis``
namespace, and a process that also loads the reference's own shared object (the benchmark's reference arm does) must keep it.
``register()`` is idempotent and refuses politely when the namespace is already taken.

Operators that expose the reference's internal storage layout (a table as a Python list of fixed-size blocks, the id
allocator's free blocks) are implemented on exactly that layout, as plain tensor code: they are compatibility shims for code
that manipulates blocks directly, not the path this framework's tables use.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

_LIB = None
_DEFINED = []


def _define(lib, schema, fn):
    lib.define(schema)
    name = schema.split("(", 1)[0]
    lib.impl(name, fn, "CompositeExplicitAutograd")
    _DEFINED.append(name)


# --------------------------------------------------------------------------------------------------- ragged / feature ops
def _ragged_to_dense(values, offsets, default_value):
    from .nn.functional import ragged_ops
    return ragged_ops.ragged_to_dense(values, list(offsets), default_value)


def _ragged_to_sparse(values, offset_splits):
    from .nn.functional import ragged_ops
    return ragged_ops.ragged_to_sparse(values, list(offset_splits))


def _dense_to_ragged(data, check_invalid, invalid_value):
    from .nn.functional import ragged_ops
    v, o = ragged_ops.dense_to_ragged(data, bool(check_invalid), invalid_value.reshape(-1)[0].item() if invalid_value.numel() else 0)[:2]
    return v, (o[0] if isinstance(o, (list, tuple)) else o)


def _uint64_mod(inputs, num):
    from .nn.functional import array_ops
    return array_ops.bucketize_mod(inputs, int(num))


def _bucketize_op(values, boundaries):
    from .nn.functional import array_ops
    return array_ops.bucketize(values, boundaries)


def _fused_multi_hash(inputs, muls, primes, bucket_num):
    from .nn.functional import fused_ops
    return list(fused_ops.fused_multi_hash(list(inputs), list(muls), list(primes), list(bucket_num)))


def _fused_uint64_mod(inputs, mod_vec):
    from .nn.functional import fused_ops
    return list(fused_ops.fused_uint64_mod_gpu(list(inputs), mod_vec))


def _fused_bucketized(inputs, boundaries):
    from .nn.functional import fused_ops
    return list(fused_ops.fused_bucketize_gpu(list(inputs), list(boundaries)))


def _fused_hash(inputs, input_offsets, hash_type):
    from .nn.functional import hash_ops
    fn = hash_ops.farmhash if hash_type == "farm" else hash_ops.murmurhash
    return list(fn(list(inputs), list(input_offsets)))


def _fused_ragged_cutoff(values, offsets, keep_lengths, drop_sides, pad_sides):
    """-> values..., offsets..., drop_nums..., pad_nums... as four lists flattened into one (the reference returns
    ``(values, offsets, drop_nums, pad_nums, drop_sides, pad_sides)``; the two side tensors are its inputs)."""
    from .nn.functional import ragged_ops
    v, o, d, p, _ds, _ps = ragged_ops.fused_ragged_cutoff_2D(list(values), list(offsets), keep_lengths, drop_sides, pad_sides)
    return list(v), list(o), list(d), list(p)


def _fused_ragged_cutoff_3d(values, outer_offsets, inner_offsets, keep_lengths, drop_sides, pad_sides):
    from .nn.functional import ragged_ops
    v, offs = ragged_ops.fused_ragged_cutoff_3D(list(values), [[a, b] for a, b in zip(outer_offsets, inner_offsets)], keep_lengths,
                                                drop_sides, pad_sides)
    return list(v), [o[0] for o in offs], [o[1] for o in offs]


def _feature_cross_ragged(x_value, x_offsets, x_weight, y_value, y_offsets, y_weight):
    from .nn.functional import ragged_ops
    xw = x_weight if x_weight is not None and x_weight.numel() else None
    yw = y_weight if y_weight is not None and y_weight.numel() else None
    return ragged_ops.feature_cross_ragged(x_value, x_offsets, y_value, y_offsets, xw, yw)


def _calc_ragged_index(drop_num, pad_num, drop_side, pad_side, offset, topk_index, indicator):
    from .nn.functional import ragged_ops
    return ragged_ops.ragged_topk_index_cutoff(drop_num, pad_num, drop_side, pad_side, offset, topk_index, indicator)


def _gauc_calc(labels, predictions, indicators):
    from . import native
    return native().gauc_calc(labels, predictions, indicators)


# --------------------------------------------------------------------------------------------------- embedding ops
def _ids_partition(ids, num_parts):
    from .nn.functional import embedding_ops
    u, counts, rev = embedding_ops.ids_partition(ids, 65536, int(num_parts))
    return u, counts, rev.to(torch.int64)


def _ids_encode(inputs, table_ids):
    from .nn.functional import embedding_ops
    return embedding_ops.ids_encode(list(inputs), table_ids)


def _merge_offsets(offsets, max_value):
    from .nn.functional import embedding_ops
    return embedding_ops.merge_offsets(list(offsets))


def _gen_segment_indices_by_offset(offset):
    from .nn.functional import ragged_ops
    return ragged_ops.gen_segment_indices(offset)


def _mode(mode: str) -> int:
    return {"sum": 0, "mean": 1}[mode]


def _segment_reduce_forward(unique_emb, weight, reverse_indices, offsets, mode):
    from . import native
    out, _g, _s = native().pool_forward(unique_emb.contiguous(), None, reverse_indices.to(torch.int32).contiguous(),
                                        offsets.to(torch.int32).contiguous(), weight, _mode(mode), 0, 0, False)
    return out.to(unique_emb.dtype)


def _segment_reduce_backward(grad_output, weight, reverse_indices, offsets, unique_size, mode):
    """Gradient of ``segment_reduce_forward`` with respect to the unique embeddings ``[unique_size, D]``."""
    off = offsets.to(torch.int64)
    lens = off[1:] - off[:-1]
    seg = torch.repeat_interleave(torch.arange(lens.numel(), device=grad_output.device), lens)
    scale = torch.ones(seg.numel(), dtype=torch.float32, device=grad_output.device) if weight is None else weight.float().reshape(-1)
    if mode == "mean":
        scale = scale / lens.clamp_min(1).float()[seg]
    g = torch.zeros(int(unique_size), grad_output.shape[1], dtype=torch.float32, device=grad_output.device)
    g.index_add_(0, reverse_indices.to(torch.int64), grad_output.float()[seg] * scale[:, None])
    return g.to(grad_output.dtype)


def _segment_sum(data, weight, indices, segment_ids, num_segments):
    src = data[indices.to(torch.int64)]
    if weight is not None:
        src = src * weight.unsqueeze(-1)
    out = torch.zeros(int(num_segments), data.shape[-1], dtype=src.dtype, device=data.device)
    return out.index_add_(0, segment_ids.to(torch.int64), src)


def _segment_mean(data, weight, segment_ids, num_segments):
    """Weights divided by the weight sum of their segment (the reference's ``weight_norm_sparse``)."""
    if weight is None:
        weight = torch.ones(segment_ids.numel(), dtype=data.dtype, device=data.device)
    total = torch.zeros(int(num_segments), dtype=weight.dtype, device=weight.device).index_add_(0, segment_ids.to(torch.int64), weight)
    return weight / total[segment_ids.to(torch.int64)]


def _ragged_tile(batch, seq, value, offset, table):
    from .nn.functional import ragged_ops
    out = ragged_ops.ragged_tile(list(batch), list(seq), value, offset, table)
    batch_seq = torch.tensor([b * s for b, s in zip(batch, seq)], dtype=torch.int64)
    return [out, batch_seq]


def _ragged_tile_back(batch_seq, batch_info, value, offset, dy):
    """Gradient of ``ragged_tile`` with respect to the table: ``batch_info = (table rows, n features, max batch, min tile len)``;
    the per-feature batch and tile lengths are recovered from ``batch_seq`` and the offsets."""
    n_rows, n_feat = int(batch_info[0]), int(batch_info[1])
    off = offset.to(torch.int64)
    total_rows = off.numel() - 1
    b = total_rows // max(n_feat, 1)
    g = torch.zeros(n_rows, dy.shape[-1], dtype=dy.dtype, device=dy.device)
    row0, out0 = 0, 0
    for f in range(n_feat):
        s = int(batch_seq[f]) // max(b, 1)
        for r in range(b):
            beg, end = int(off[row0 + r]), int(off[row0 + r + 1])
            k = min(end - beg, s)
            if k:
                g.index_add_(0, value[beg:beg + k].to(torch.int64), dy[out0 + r * s:out0 + r * s + k])
        row0 += b
        out0 += b * s
    return g


def _adam_tf_apply(param, grad, avg, avg_sq, step, lr, beta1, beta2, eps):
    """TensorFlow-style Adam on a dense tensor, in place (``csrc/ops/adam_tf_op_kernel.cu``): epsilon inside the square root's
    companion term as TF does (``lr_t = lr * sqrt(1 - b2^t) / (1 - b1^t)``, ``p -= lr_t * m / (sqrt(v) + eps)``)."""
    step, lr, beta1, beta2, eps = float(step), float(lr), float(beta1), float(beta2), float(eps)
    avg.mul_(beta1).add_(grad, alpha=1 - beta1)
    avg_sq.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
    lr_t = lr * (1 - beta2 ** step) ** 0.5 / (1 - beta1 ** step)
    param.addcdiv_(avg, avg_sq.sqrt().add_(eps), value=-lr_t)


# --------------------------------------------------------------------------------------------------- block / allocator shims
def _block_rows(ids, block_size):
    ids = ids.to(torch.int64)
    return torch.div(ids, block_size, rounding_mode="floor"), ids % block_size


def _gather(ids, emb):
    return emb[ids.to(torch.int64)]


def _block_gather(ids, emb_blocks, block_size, default_key, readonly):
    blk, row = _block_rows(ids, block_size)
    stacked = torch.cat(list(emb_blocks))
    valid = ids != default_key
    safe = torch.where(valid, blk * block_size + row, torch.zeros_like(ids.to(torch.int64)))
    out = stacked[safe]
    out[~valid] = 0
    return out


def _block_insert(ids, embedding, emb_blocks, block_size):
    blk, row = _block_rows(ids, block_size)
    for b in blk.unique().tolist():
        m = blk == b
        emb_blocks[b][row[m]] = embedding[m].to(emb_blocks[b].dtype)


def _block_insert_with_mask(ids, embedding, mask, emb_blocks, block_size):
    m = mask.to(torch.bool)
    _block_insert(ids[m], embedding[m], emb_blocks, block_size)


def _block_filter(ids, emb_blocks, block_size, step):
    blk, row = _block_rows(ids, block_size)
    stacked = torch.cat([b.reshape(-1) for b in emb_blocks])
    return stacked[blk * block_size + row] < step


def _block_apply_adamw(index, grad, emb_blocks, beta1_t, beta2_t, step, exp_avg, exp_avg_sq, lr, beta1, beta2, weight_decay, eps, block_size):
    """Row-wise AdamW on block storage (``csrc/ops/block_apply_adamw_op_kernel.cu:11-22``): beta powers advance once, then every
    indexed row is decayed and updated."""
    beta1_t.mul_(beta1); beta2_t.mul_(beta2)
    alpha = -lr * (1 - float(beta2_t)) ** 0.5 / (1 - float(beta1_t))
    blk, row = _block_rows(index, block_size)
    for b in blk.unique().tolist():
        m = blk == b
        r = row[m]
        g = grad[m].float()
        avg = exp_avg[b][r].mul(beta1).add(g, alpha=1 - beta1)
        sq = exp_avg_sq[b][r].mul(beta2).addcmul(g, g, value=1 - beta2)
        exp_avg[b][r] = avg
        exp_avg_sq[b][r] = sq
        w = emb_blocks[b][r].float() * (1 - lr * weight_decay) + alpha * avg / (sq.sqrt() + eps)
        emb_blocks[b][r] = w.to(emb_blocks[b].dtype)


def _generate_ids(gen_num, free_blocks, free_count, cur_count, free_block_size):
    """``gen_num`` row ids: the last ``min(gen_num, free_count)`` entries of the free list first, then fresh ids counted up from
    ``cur_count`` (``csrc/ops/hashtable_ops_kernel.cu``: ``free_index = free_count - gen_num + i``; negative means fresh)."""
    dev = free_blocks[0].device if len(free_blocks) else torch.device("cpu")
    idx = torch.arange(gen_num, device=dev) + (free_count - gen_num)
    out = cur_count - (idx + 1)
    if len(free_blocks):
        flat = torch.cat([b.reshape(-1) for b in free_blocks])
        from_free = idx >= 0
        out = torch.where(from_free, flat[idx.clamp_min(0)], out)
    return out


def _free_ids(free_ids, free_blocks, free_count, free_block_size):
    pos = torch.arange(free_ids.numel(), device=free_ids.device) + free_count
    blk, row = _block_rows(pos, free_block_size)
    for b in blk.unique().tolist():
        m = blk == b
        free_blocks[b].reshape(-1)[row[m]] = free_ids[m]


def _mask_key_index(in_keys, mask, out_index, out_size):
    m = mask.to(torch.bool)
    return in_keys[m][:out_size], out_index[m][:out_size]


def _scatter_ids_with_mask(out_ids, in_ids, mask_index):
    out_ids[mask_index.to(torch.int64)] = in_ids
    return out_ids


_SCHEMAS = [
    ("ragged_to_dense(Tensor values, Tensor[] offsets, Scalar default_value) -> Tensor", _ragged_to_dense),
    ("ragged_to_sparse(Tensor values, Tensor[] offset_splits) -> Tensor", _ragged_to_sparse),
    ("dense_to_ragged(Tensor data, bool check_invalid, Tensor invalid_value) -> (Tensor, Tensor)", _dense_to_ragged),
    ("uint64_mod(Tensor inputs, Scalar num) -> Tensor", _uint64_mod),
    ("bucketize_op(Tensor values, Tensor boundaries) -> Tensor", _bucketize_op),
    ("fused_multi_hash(Tensor[] inputs, Tensor[] muls, Tensor[] primes, Tensor[] bucket_num) -> Tensor[]", _fused_multi_hash),
    ("fused_uint64_mod(Tensor[] inputs, Tensor mod_vec) -> Tensor[]", _fused_uint64_mod),
    ("fused_bucketized(Tensor[] inputs, Tensor[] boundaries) -> Tensor[]", _fused_bucketized),
    ("fused_hash(Tensor[] inputs, Tensor[] input_offsets, str hash_type) -> Tensor[]", _fused_hash),
    ("fused_ragged_cutoff(Tensor[] values, Tensor[] offsets, Tensor keep_lengths, Tensor drop_sides, Tensor pad_sides)"
     " -> (Tensor[], Tensor[], Tensor[], Tensor[])", _fused_ragged_cutoff),
    ("fused_ragged_cutoff_3D(Tensor[] values, Tensor[] outer_offsets, Tensor[] inner_offsets, Tensor keep_lengths, Tensor drop_sides,"
     " Tensor pad_sides) -> (Tensor[], Tensor[], Tensor[])", _fused_ragged_cutoff_3d),
    ("feature_cross_ragged(Tensor x_value, Tensor x_offsets, Tensor x_weight, Tensor y_value, Tensor y_offsets, Tensor y_weight)"
     " -> (Tensor, Tensor, Tensor)", _feature_cross_ragged),
    ("calc_ragged_index(Tensor drop_num, Tensor pad_num, Tensor drop_side, Tensor pad_side, Tensor offset, Tensor topk_index,"
     " Tensor indicator) -> (Tensor, Tensor)", _calc_ragged_index),
    ("gauc_calc(Tensor labels, Tensor predictions, Tensor indicators) -> (Tensor, Tensor)", _gauc_calc),
    ("ids_partition(Tensor ids, int num_parts) -> (Tensor, Tensor, Tensor)", _ids_partition),
    ("ids_encode(Tensor[] inputs, Tensor table_ids) -> Tensor", _ids_encode),
    ("merge_offsets(Tensor[] offsets, Tensor max_value) -> Tensor", _merge_offsets),
    ("gen_segment_indices_by_offset(Tensor offset) -> Tensor", _gen_segment_indices_by_offset),
    ("segment_reduce_forward(Tensor unique_emb, Tensor? weight, Tensor reverse_indices, Tensor offsets, str mode) -> Tensor",
     _segment_reduce_forward),
    ("segment_reduce_backward(Tensor grad_output, Tensor? weight, Tensor reverse_indices, Tensor offsets, int unique_size, str mode)"
     " -> Tensor", _segment_reduce_backward),
    ("segment_sum(Tensor data, Tensor? weight, Tensor indices, Tensor segment_ids, Scalar num_segments) -> Tensor", _segment_sum),
    ("segment_mean(Tensor data, Tensor? weight, Tensor segment_ids, Scalar num_segments) -> Tensor", _segment_mean),
    ("ragged_tile(int[] batch, int[] seq, Tensor value, Tensor offset, Tensor table) -> Tensor[]", _ragged_tile),
    ("ragged_tile_back(Tensor batch_seq, int[] batch_info, Tensor value, Tensor offset, Tensor dy) -> Tensor", _ragged_tile_back),
    ("adam_tf_apply(Tensor(a!) param, Tensor grad, Tensor(b!) avg, Tensor(c!) avg_sq, Scalar step, Scalar lr, Scalar beta1, Scalar beta2,"
     " Scalar eps) -> ()", _adam_tf_apply),
    ("gather(Tensor ids, Tensor emb) -> Tensor", _gather),
    ("block_gather(Tensor ids, Tensor[] emb_blocks, int block_size, int default_key, bool readonly) -> Tensor", _block_gather),
    ("block_insert(Tensor ids, Tensor embedding, Tensor(a!)[] emb_blocks, int block_size) -> ()", _block_insert),
    ("block_insert_with_mask(Tensor ids, Tensor embedding, Tensor mask, Tensor(a!)[] emb_blocks, int block_size) -> ()",
     _block_insert_with_mask),
    ("block_filter(Tensor ids, Tensor[] emb_blocks, int block_size, int step) -> Tensor", _block_filter),
    ("block_apply_adamw(Tensor index, Tensor grad, Tensor(a!)[] emb_blocks, Tensor(b!) beta1_t, Tensor(c!) beta2_t, Tensor step,"
     " Tensor(d!)[] exp_avg, Tensor(e!)[] exp_avg_sq, float lr, float beta1, float beta2, float weight_decay, float eps, int block_size)"
     " -> ()", _block_apply_adamw),
    ("generate_ids(int gen_num, Tensor[] free_blocks, int free_count, int cur_count, int free_block_size) -> Tensor", _generate_ids),
    ("free_ids(Tensor free_ids, Tensor(a!)[] free_blocks, int free_count, int free_block_size) -> ()", _free_ids),
    ("mask_key_index(Tensor in_keys, Tensor mask, Tensor out_index, int out_size) -> (Tensor, Tensor)", _mask_key_index),
    ("scatter_ids_with_mask(Tensor(a!) out_ids, Tensor in_ids, Tensor mask_index) -> Tensor(a!)", _scatter_ids_with_mask),
]


def registered() -> List[str]:
    return list(_DEFINED)


def register() -> bool:
    """Define ``torch.ops.recis.*`` (once per process). Returns False, and leaves everything alone, when the ``recis`` operator
    namespace already belongs to another library in this process (for example the reference's own shared object)."""
    global _LIB
    if _LIB is not None:
        return True
    try:
        lib = torch.library.Library("recis", "DEF")
    except RuntimeError:
        return False
    for schema, fn in _SCHEMAS:
        _define(lib, schema, fn)
    _LIB = lib
    return True


def make_hashtable(*args, **kwargs):
    """The reference creates its native table object through ``torch.ops.recis.make_hashtable``; a table is a Python-visible class
    here (``recis_b200.nn.HashTable`` over ``EmbeddingStore``), so this is a plain function with the same role."""
    from .nn.modules.hashtable import HashtableImpl
    return HashtableImpl(*args, **kwargs)


register()
