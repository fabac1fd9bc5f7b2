"""HashTable: a dynamic (grow-on-insert) embedding table shard.

Public surface of the reference's ``recis/nn/modules/hashtable.py:152-731`` (``HashTable``, ``gen_slice``,
``filter_out_sparse_param``, ``split_sparse_dense_state_dict``, ``HashtableRegister``) on top of the native
``EmbeddingStore`` (one open-addressing index + contiguous slot slabs, see ``csrc/bind/store.cpp``).

Gradients never become a torch sparse tensor on the hot path: the backward pass *stages* records on the
table and the sparse optimizer consumes them. A record is either ``(rows, grads)`` or a "fused" record that
still holds the pooled output gradient plus the element->unique structure; the optimizer turns a single fused
record into one kernel that reduces duplicate ids and applies the update to each touched row exactly once.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Tuple

import torch

from ... import native
from ..hashtable_hook import AdmitHook, FilterHook
from ..initializers import ConstantInitializer

SLICE_SIZE = 65536
ID_BITS = 52
ID_MASK = (1 << ID_BITS) - 1
MAX_CHILDREN = 4095


class Slice:
    """``[slice_begin, slice_end)`` of ``slice_size`` hash slices owned by a shard."""

    def __init__(self, slice_beg, slice_end, slice_size) -> None:
        self.slice_begin = slice_beg
        self.slice_end = slice_end
        self.slice_size = slice_size

    def __repr__(self):
        return f"Slice({self.slice_begin}, {self.slice_end}, {self.slice_size})"

    def to_string(self):
        """Zero-padded ``beg@end@size`` form used in checkpoint block names."""
        width = len(str(self.slice_size))
        return f"{self.slice_begin:0{width}d}@{self.slice_end:0{width}d}@{self.slice_size}"


def gen_slice(shard_index=0, shard_num=1, slice_size=SLICE_SIZE) -> Slice:
    """Contiguous slice range of shard ``shard_index``; the first ``slice_size % shard_num`` shards own one more."""
    q, r = divmod(slice_size, shard_num)
    beg = shard_index * q + min(shard_index, r)
    end = beg + q + (1 if shard_index < r else 0)
    return Slice(beg, end, slice_size)


_default_slice = Slice(0, SLICE_SIZE, SLICE_SIZE)


class ChildrenInfo:
    """Logical tables merged into one physical table; child ``i`` owns ids with prefix ``i`` in the top 12 bits."""

    def __init__(self, coalesced: bool, children: List[str]):
        if len(children) > MAX_CHILDREN:
            raise ValueError(f"at most {MAX_CHILDREN} tables can be merged, got {len(children)}")
        self._coalesced = coalesced
        self._children = list(children)
        self._index = {c: i for i, c in enumerate(self._children)}

    def is_coalesce(self):
        return self._coalesced

    def children(self):
        return list(self._children)

    def child_index(self, name: str) -> int:
        return self._index[name]

    def has_child(self, name: str) -> bool:
        return name in self._index

    def child_at(self, i: int) -> str:
        return self._children[i]

    @staticmethod
    def encode(ids: torch.Tensor, index: int) -> torch.Tensor:
        return (ids & ID_MASK) | (index << ID_BITS)

    @staticmethod
    def decode_index(ids: torch.Tensor) -> torch.Tensor:
        return (ids >> ID_BITS) & 0xFFF

    @staticmethod
    def decode_id(ids: torch.Tensor) -> torch.Tensor:
        return ids & ID_MASK


class SlotView:
    """One named per-row array of a table."""

    def __init__(self, name: str, tensor_fn):
        self._name = name
        self._tensor_fn = tensor_fn

    def name(self):
        return self._name

    def value(self) -> torch.Tensor:
        return self._tensor_fn()


class SlotGroupView:
    def __init__(self, impl: "HashtableImpl"):
        self._impl = impl

    def slot_names(self):
        return ["embedding"] + self._impl.store.slot_names()

    def slot_by_name(self, name: str) -> SlotView:
        if name == "embedding":
            return SlotView(name, lambda: self._impl.store.emb())
        return SlotView(name, lambda: self._impl.store.slot(name))

    def slots(self):
        return [self.slot_by_name(n) for n in self.slot_names()]


class HashtableImpl:
    """Table state shared between the ``HashTable`` module, the sparse optimizers and the checkpoint code."""

    hashtable_tag = True

    def __init__(self, embedding_shape, dtype, device, coalesced, children, initializer, slice_: Slice,
                 name: str, capacity: int = 0, track_last_seen: bool = True, emb_storage=None, growable: bool = True):
        self.name = name
        self.embedding_shape = list(embedding_shape)
        self.dim = 1
        for s in self.embedding_shape:
            self.dim *= int(s)
        self.dtype = dtype
        self.device = torch.device(device)
        self.slice = slice_
        self._children_info = ChildrenInfo(coalesced, children)
        self.initializer = initializer
        kind, a, b, lo, hi, seed = initializer.spec()
        cap = int(capacity) if capacity and capacity > 0 else 4096
        dev_str = str(self.device) if self.device.index is not None or self.device.type == "cpu" else (
            f"cuda:{torch.cuda.current_device()}")
        # rows are stored in the table's dtype (float32 / float16 / bfloat16, or int8 for read-only tables); optimizer state
        # slots and all accumulation are fp32 (the reference dispatches its row kernels over the same types,
        # csrc/ops/block_ops_kernel.cu:236-273)
        if dtype not in (torch.float32, torch.float16, torch.bfloat16, torch.int8):
            raise NotImplementedError(f"embedding dtype {dtype} is not supported (float32, float16, bfloat16 and read-only int8 are)")
        self.store = native().EmbeddingStore(self.dim, cap, dev_str, kind, a, b, lo, hi, seed, track_last_seen, growable,
                                             emb_storage, dtype)
        self.store.set_name(name)
        self.device = torch.device(dev_str)
        self._records = []
        self.trainable = dtype in (torch.float32, torch.float16, torch.bfloat16)

    # ---- reference-compatible accessors
    def children_info(self):
        return self._children_info

    def slot_group(self):
        return SlotGroupView(self)

    def slice_info(self):
        return self.slice

    def embedding_lookup(self, ids: torch.Tensor, readonly: bool = False, step=None, admit_threshold: int = 1):
        """ids (any order, duplicates allowed) -> (row index int32 [-1 = unknown], embeddings)."""
        ids = ids.detach().reshape(-1).to(self.device).contiguous()
        rows = self.store.find(ids) if readonly else self.store.lookup_or_insert(ids, None, step, admit_threshold)
        emb = native().gather_rows(self.store.emb(), rows)
        return rows, emb

    def insert(self, ids: torch.Tensor, embeddings: torch.Tensor):
        ids = ids.detach().reshape(-1).to(self.device).contiguous()
        rows = self.store.lookup_or_insert(ids, None, None, 1)
        native().scatter_rows(self.store.emb(), rows, embeddings.to(self.device, self.store.emb().dtype).contiguous(), False)
        return rows

    def insert_lookup_index(self, ids: torch.Tensor):
        ids = ids.detach().reshape(-1).to(self.device).contiguous()
        return self.store.lookup_or_insert(ids, None, None, 1)

    def delete(self, ids: torch.Tensor):
        return self.store.erase(ids.detach().reshape(-1).to(self.device).contiguous())

    def ids(self) -> torch.Tensor:
        return self.store.snapshot(False, 0)[0]

    def ids_map(self) -> Tuple[torch.Tensor, torch.Tensor]:
        ids, rows = self.store.snapshot(False, 0)
        return ids, rows.to(torch.int64)

    def clear(self):
        self.store.clear()
        self._records = []

    def size(self) -> int:
        return self.store.size()

    def stats(self) -> dict:
        """Occupancy of this shard (one device-to-host read of the 64-byte counter block): live rows, row capacity and load,
        index slots and load, ids on admission probation, erased-but-unreclaimed index slots, rows on the free stack, rows
        admitted by the last lookup, and the sticky status bits (0 = healthy)."""
        c = self.store.counters()
        bump, free_top, _new, status, live, tomb, prob, last_new = (int(x) for x in c[:8])
        cap = int(self.store.capacity())
        slots = int(self.store.keys().numel())
        return {
            "rows": live, "row_capacity": cap, "row_load": (bump - free_top) / max(cap, 1), "free_rows": free_top,
            "index_slots": slots, "index_load": (live + tomb + prob) / max(slots, 1), "probation": prob, "tombstones": tomb,
            "admitted_last_lookup": last_new, "status": status,
        }

    # ---- gradient staging
    def accept_grad(self, index: torch.Tensor, grad: torch.Tensor):
        self._records.append({"kind": "rows", "rows": index.to(torch.int32), "grad": grad})

    def stage_fused(self, record: dict):
        record["kind"] = "fused"
        self._records.append(record)

    def records(self):
        return self._records

    def clear_grad(self):
        self._records = []

    def materialize(self):
        """All staged records as one ``(unique rows int32, summed grads)`` pair (rows < 0 dropped)."""
        C = native()
        rows_l, grad_l = [], []
        for r in self._records:
            if r["kind"] == "rows":
                rows_l.append(r["rows"].reshape(-1))
                grad_l.append(r["grad"].reshape(-1, self.dim).to(torch.float32))
            elif r["kind"] == "peer":
                rows, grads = r["exchange"].owner_reduce(self, r, apply=False)
                rows_l.append(rows)
                grad_l.append(grads)
            else:
                csr_u, csr_elem, start = C.build_csr(r["rev"])
                gu = C.grad_reduce(r["grad_out"], r["gsrc"], r["gscale"], csr_u, csr_elem, start, self.dim, None, False,
                                   2, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0, None, None, None, r["rows"].numel())
                rows_l.append(r["rows"])
                grad_l.append(gu * r.get("scale", 1.0))
        if not rows_l:
            return None, None
        rows = torch.cat(rows_l)
        grads = torch.cat([g.to(torch.float32) for g in grad_l])
        keep = rows >= 0  # unknown / not admitted ids, and the padding past a record's unique count
        rows, grads = rows[keep], grads[keep]
        uniq, inv = torch.unique(rows, return_inverse=True)
        out = torch.zeros(uniq.numel(), self.dim, dtype=torch.float32, device=grads.device)
        out.index_add_(0, inv, grads)
        return uniq.to(torch.int32), out

    def grad(self, acc_step: int = 1) -> torch.Tensor:
        """Staged gradient as a sparse COO tensor indexed by row (compatibility API)."""
        rows, grads = self.materialize()
        cap = self.store.capacity()
        if rows is None:
            return torch.sparse_coo_tensor(torch.zeros(1, 0, dtype=torch.int64), torch.zeros(0, self.dim), (cap, self.dim))
        return torch.sparse_coo_tensor(rows.to(torch.int64).unsqueeze(0), grads / acc_step, (cap, self.dim))


class HashtableRegister:
    """Process-wide registry that rejects two tables declaring the same shard name."""

    _instance = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
            cls._instance._hashtables = {}
        return cls._instance

    def register(self, name: str, info: str):
        if name in self._hashtables:
            raise ValueError(f"Duplicate hashtable shard name: {name}, before: {self._hashtables[name]}, now: {info}")
        self._hashtables[name] = info

    def unregister(self, name: str):
        self._hashtables.pop(name, None)

    def clear(self):
        self._hashtables.clear()


class _LookupFn(torch.autograd.Function):
    """ids -> embeddings [N, D]; backward stages ``(rows, grad)`` on the table."""

    @staticmethod
    def forward(ctx, holder, impl: HashtableImpl, ids, readonly, step, admit_threshold, scale):
        C = native()
        uniq, rev, _counts, offs = C.dedup_partition(ids, 1)
        n_dev = offs[1:2]
        if readonly:
            rows_u = impl.store.find(uniq, n_dev)
        else:
            rows_u = impl.store.lookup_or_insert(uniq, n_dev, step, admit_threshold, True)      # distinct ids: erased slots may be reused
        rows = rows_u[rev.long()] if rev.numel() else rows_u[:0]
        ctx.impl, ctx.scale = impl, scale
        ctx.save_for_backward(rows)
        return C.gather_rows(impl.store.emb(), rows), rows

    @staticmethod
    def backward(ctx, grad_emb, _grad_rows):
        (rows,) = ctx.saved_tensors
        g = grad_emb.contiguous().to(torch.float32)
        if ctx.scale != 1.0:
            g = g * ctx.scale
        ctx.impl.accept_grad(rows, g)
        return (None,) * 7


class HashTable(torch.nn.Module):
    """One table shard. ``forward(ids)`` returns one embedding per id (duplicates allowed)."""

    def __init__(self, embedding_shape: List, block_size: int = 5, dtype: torch.dtype = torch.float32,
                 device: torch.device = torch.device("cpu"), coalesced: bool = False, children: Optional[List[str]] = None,
                 slice: Slice = _default_slice, initializer=None, name: str = "hashtable", grad_reduce_by: str = "worker",
                 filter_hook: Optional[FilterHook] = None, capacity: int = 0, emb_storage=None, growable: bool = True):
        super().__init__()
        assert grad_reduce_by in ("id", "worker")
        self._initializer = initializer if initializer is not None else ConstantInitializer(init_val=0)
        if children is None:
            children = [name]
        self._grad_reduce_by = grad_reduce_by
        if self._initializer.impl() is None:
            self._initializer.set_shape([block_size] + list(embedding_shape))
            self._initializer.set_dtype(dtype)
            self._initializer.build()
        self._dtype = dtype
        self._name = name
        self._children = list(children)
        for child in children:
            info = json.dumps(dict(shape=list(embedding_shape), dtype=str(dtype), initializer=str(self._initializer)))
            HashtableRegister().register(child, info)
        # block_size only sizes the first allocation here: storage is one growable slab, not a list of blocks.
        self._hashtable_impl = HashtableImpl(embedding_shape, dtype, device, coalesced, children, self._initializer, slice, name,
                                             capacity=capacity or max(int(block_size), 1024), emb_storage=emb_storage,
                                             growable=growable)
        self._device = self._hashtable_impl.device
        self._backward_holder = torch.tensor([0.0], requires_grad=True)
        self._worker_num = int(os.environ.get("WORLD_SIZE", 1))

        def state_dict_hook(module, state_dict, prefix, local_metadata):
            state_dict[module._name] = module._hashtable_impl

        self._register_state_dict_hook(state_dict_hook)
        if filter_hook is not None:
            from .hashtable_hook_impl import HashtableHookFactory
            self._filter_hook_impl = HashtableHookFactory().create_filter_hook(self, filter_hook)
        else:
            self._filter_hook_impl = None

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        state_dict.pop(self._name, None)  # table contents travel through the sparse checkpoint, not torch.load
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def __del__(self):
        try:
            for child in self._children:
                HashtableRegister().unregister(child)
        except Exception:
            pass

    @property
    def impl(self) -> HashtableImpl:
        return self._hashtable_impl

    def step_tensor(self):
        return self._filter_hook_impl.step_tensor() if self._filter_hook_impl is not None else None

    def forward(self, ids: torch.Tensor, admit_hook: AdmitHook = None) -> torch.Tensor:
        from .hashtable_hook_impl import admit_params
        readonly, threshold = admit_params(admit_hook)
        impl = self._hashtable_impl
        shape = ids.shape
        ids = ids.detach().reshape(-1).to(self._device).contiguous()
        train = self.training and impl.trainable
        if not train:
            readonly = True
        scale = 1.0 / self._worker_num if self._grad_reduce_by == "worker" else 1.0
        emb, _rows = _LookupFn.apply(self._backward_holder, impl, ids, readonly, self.step_tensor() if train else None, threshold,
                                     scale)
        return emb.view(*shape, impl.dim) if len(shape) != 1 else emb

    def initializer(self):
        return self._initializer

    @property
    def device(self):
        return self._device

    @property
    def coalesce(self):
        return self._hashtable_impl.children_info().is_coalesce()

    @property
    def children_hashtable(self):
        return self._hashtable_impl.children_info().children()

    def accept_grad(self, grad_index, grad) -> None:
        self._hashtable_impl.accept_grad(grad_index, grad)

    def grad(self, acc_step=1) -> torch.Tensor:
        return self._hashtable_impl.grad(acc_step)

    def clear_grad(self) -> None:
        self._hashtable_impl.clear_grad()

    def insert(self, ids, embeddings) -> None:
        self._hashtable_impl.insert(ids, embeddings)

    def clear(self) -> None:
        self._hashtable_impl.clear()

    def ids(self) -> torch.Tensor:
        return self._hashtable_impl.ids()

    def ids_map(self) -> Tuple[torch.Tensor, torch.Tensor]:
        return self._hashtable_impl.ids_map()

    def embeddings(self) -> torch.Tensor:
        return self._hashtable_impl.store.emb()

    def slot_group(self):
        return self._hashtable_impl.slot_group()

    def children_info(self):
        return self._hashtable_impl.children_info()

    def __str__(self) -> str:
        return f"HashTable_{self._name}"

    __repr__ = __str__


def is_hashtable(obj):
    return hasattr(obj, "hashtable_tag")


def split_sparse_dense_state_dict(state_dict: dict) -> Tuple[dict, dict]:
    """Move every table object out of ``state_dict`` (in place); returns ``(sparse, dense)``."""
    sparse = {k: v for k, v in state_dict.items() if v is not None and is_hashtable(v)}
    for k in sparse:
        del state_dict[k]
    return sparse, state_dict


def filter_out_sparse_param(model: torch.nn.Module) -> dict:
    """``{table name: table}`` for every table inside ``model`` (what the sparse optimizers take)."""
    sparse, _ = split_sparse_dense_state_dict(model.state_dict())
    return sparse
