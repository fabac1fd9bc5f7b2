"""Datasets and dataset wrappers (``recis/io``: ``dataset_base.py``, ``orc_dataset.py``, ``state_dataset.py``,
``map_dataset.py``, ``wrap_end_dataset.py``, ``filter_dataset.py``).

A dataset is an iterable of batches (dict name -> Tensor / RaggedTensor) that can dump and restore its position
(``dump_io_state`` / ``load_io_state``). The training loop consumes ``(stop_flag, batch)`` pairs, produced by
``WrapEndDataset``. Sources:
* ``SyntheticDataset``  native multi-threaded generator (``csrc/bind/bind_io.cpp``), pinned output, state = batch index;
* ``OrcDataset``        columnar files through pyarrow (ORC or Parquet): list columns become RaggedTensors, string columns
                        are hashed at read time (FarmHash / MurmurHash, as column-io does), rows are sharded over workers;
* ``TensorDataset``     in-memory dict of tensors, for tests and small jobs.
The ODPS / Lake / Pangu readers of the reference are services internal to its authors and have no counterpart here.
"""
from __future__ import annotations

import os

import queue
import threading
from typing import Callable, Dict, List, Optional

import torch

from .. import native
from ..ragged.tensor import RaggedTensor
from .synthetic import SyntheticSpec

_LEN_KIND = {"fixed": 0, "poisson": 1, "geometric": 2, "uniform": 3}


def is_string_dtype(arr) -> bool:
    """Whether a numpy array holds strings: unicode, bytes or objects (``recis/io/dataset_base.py:23-31``)."""
    return arr.dtype.kind in ("U", "S", "O")


class DatasetBase:
    """Iterable of batches with a restorable position.

    ``map`` / ``filter`` register functions on the dataset itself, as in the reference (``recis/io/dataset_base.py:273-308``):
    every batch goes through the map functions in registration order; a batch for which ANY filter function returns True is
    skipped. Both return the dataset, so calls can be chained."""

    # True: the class (and, by inheritance, classes built on its batch conversion) applies the registered functions itself,
    # at its own place in __iter__
    _pipeline_inline = False

    def map(self, map_func):
        self.__dict__.setdefault("_map_funcs", []).append(map_func)
        return self

    def filter(self, filter_func):
        self.__dict__.setdefault("_filter_funcs", []).append(filter_func)
        return self

    def _run_maps(self, batch):
        for f in self.__dict__.get("_map_funcs", ()):
            batch = f(batch)
        return batch

    def _filtered_out(self, batch) -> bool:
        return any(f(batch) for f in self.__dict__.get("_filter_funcs", ()))

    def _through_pipeline(self, it):
        for batch in it:
            batch = self._run_maps(batch)
            if not self._filtered_out(batch):
                yield batch

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        raw = cls.__dict__.get("__iter__")
        if raw is not None and not getattr(cls, "_pipeline_inline", False):
            def __iter__(self, _raw=raw):
                if self.__dict__.get("_map_funcs") or self.__dict__.get("_filter_funcs"):
                    return self._through_pipeline(_raw(self))
                return _raw(self)
            cls.__iter__ = __iter__

    def __iter__(self):
        raise NotImplementedError

    def dump_io_state(self):
        return {}

    def load_io_state(self, state):
        pass


class SyntheticDataset(DatasetBase):
    def __init__(self, spec: SyntheticSpec, steps: Optional[int] = None, threads: int = 2, prefetch: int = 4, pin: bool = False):
        self.spec, self.steps = spec, steps
        fields = [(f.zipf_a, f.id_bits, int(f.universe or 0), _LEN_KIND[f.length], float(f.mean_len), f.min_len, f.max_len, f.geo_p)
                  for f in spec.sparse]
        self._src = native().SyntheticSource(spec.batch, spec.dense_dim, fields, spec.label_rate, spec.seed, threads, prefetch, pin)
        self._names = [f.name for f in spec.sparse]

    def __iter__(self):
        if self.steps is not None and self._src.state() >= self.steps:
            self._src.set_state(0)          # a finished pass starts over (a new epoch); a restored position resumes
        while self.steps is None or self._src.state() < self.steps:
            dense, label, fields = self._src.next()
            batch = {"label": label}
            if self.spec.dense_dim:
                batch["dense"] = dense
            for name, (ids, off) in zip(self._names, fields):
                batch[name] = RaggedTensor(ids, [off], dense_shape=(self.spec.batch, -1))
            yield batch

    def dump_io_state(self):
        return {"step": self._src.state()}

    def load_io_state(self, state):
        self._src.set_state(int(state["step"]))


class TensorDataset(DatasetBase):
    """Batches sliced from an in-memory dict of equally long tensors."""

    def __init__(self, data: Dict[str, torch.Tensor], batch_size: int, drop_remainder: bool = False, epochs: int = 1):
        self.data, self.batch_size, self.drop_remainder, self.epochs = data, batch_size, drop_remainder, epochs
        self._n = len(next(iter(data.values())))
        self._pos = 0

    def __iter__(self):
        total = self._n * self.epochs
        if self._pos >= total:
            self._pos = 0                   # a finished pass starts over (a new epoch); a restored position resumes
        while self._pos < total:
            b = self._pos % self._n
            e = min(b + self.batch_size, self._n)
            if self.drop_remainder and e - b < self.batch_size:
                self._pos += e - b
                continue
            self._pos += e - b
            yield {k: v[b:e] for k, v in self.data.items()}

    def dump_io_state(self):
        return {"pos": self._pos}

    def load_io_state(self, state):
        self._pos = int(state["pos"])


def get_dir_size(dir_name: str) -> int:
    """Bytes on disk under ``dir_name`` (a file or a directory walked recursively), ``recis/io/orc_dataset.py:17``."""
    if os.path.isfile(dir_name):
        return os.path.getsize(dir_name)
    total = 0
    for root, _dirs, files in os.walk(dir_name):
        total += sum(os.path.getsize(os.path.join(root, f)) for f in files)
    return total


class OrcDataset(DatasetBase):
    """Columnar files -> batches. ``varlen_feature`` columns (lists of ints, or strings / lists of strings with a hash)
    become RaggedTensors; ``fixedlen_feature`` columns become dense ``[batch, dim]`` tensors."""

    _pipeline_inline = True           # registered map functions run before transform_fn, as in the reference

    def __init__(self, batch_size: int, worker_idx: int = 0, worker_num: int = 1, read_threads_num: int = 4,
                 pack_threads_num: Optional[int] = None, prefetch: int = 1, is_compressed: bool = False, drop_remainder: bool = False,
                 worker_slice_batch_num: Optional[int] = None, shuffle: bool = False, ragged_format: bool = True,
                 transform_fn: Optional[Callable] = None, save_interval: int = 100, dtype: torch.dtype = torch.float32,
                 device: str = "cpu", pin: bool = False, seed: int = 0, native_reader: bool = True, repeat: int = 1):
        # Argument order follows the reference (``recis/io/orc_dataset.py:73-90``). Accepted for compatibility, without effect
        # here: ``pack_threads_num`` (one packer thread keeps batches in file order), ``is_compressed`` (ORC / Parquet carry their
        # own compression), ``worker_slice_batch_num`` (files are dealt round-robin to workers) and ``save_interval`` (the
        # iterator position is a (file, row) pair that is always current, so there is nothing to snapshot periodically).
        self.pack_threads_num, self.is_compressed = pack_threads_num, is_compressed
        self.worker_slice_batch_num, self.save_interval = worker_slice_batch_num, save_interval
        self.batch_size, self.worker_idx, self.worker_num = batch_size, worker_idx, worker_num
        self.read_threads_num, self.native_reader = read_threads_num, native_reader
        self.repeat = max(int(repeat), 1)           # passes over this worker's files (the role of column-io's RepeatDataset)
        self.drop_remainder, self.shuffle, self.transform_fn, self.dtype, self.device, self.pin = drop_remainder, shuffle, transform_fn, dtype, device, pin
        self.prefetch, self.seed = prefetch, seed
        # where batches are placed, as in the reference (``recis/io/dataset_base.py:207-212``): host memory, pinned host memory
        # or the current CUDA device (pinned staging + asynchronous copy)
        assert str(device) in ("cpu", "pin", "cuda"), f"Only support io result placed in `cpu|cuda|pin` but got {device}"
        self.ragged_format = ragged_format
        self.pin = self.pin or (str(device) in ("pin", "cuda") and torch.cuda.is_available())
        self._paths: List[str] = []
        self._varlen, self._fixed = {}, {}
        self._file_idx, self._row_in_file = 0, 0

    def add_path(self, file_path: str):
        self._paths.append(file_path)

    def add_paths(self, file_paths: List[str]):
        self._paths.extend(file_paths)

    def varlen_feature(self, name: str, hash_type: Optional[str] = None, hash_bucket: int = 0, trans_int8: bool = False):
        self._varlen[name] = dict(hash_type=hash_type, hash_bucket=hash_bucket, trans_int8=trans_int8)

    def fixedlen_feature(self, name: str, default_value=0.0):
        self._fixed[name] = default_value

    def _my_paths(self):
        mine = [p for i, p in enumerate(sorted(self._paths)) if i % self.worker_num == self.worker_idx]
        if not self.shuffle:
            return mine * self.repeat
        # file-level shuffle, as the reference's file sharding does (``recis/io/orc_dataset.py:285-293``): a new order for every
        # pass, a pure function of (seed, pass) so that a restored iterator state points at the same file again
        import random
        out = []
        for r in range(self.repeat):
            part = list(mine)
            random.Random(self.seed * 1000003 + r).shuffle(part)
            out += part
        return out

    @staticmethod
    def _read_table(path):
        if path.endswith(".parquet"):
            import pyarrow.parquet as pq
            return pq.read_table(path)
        import pyarrow.orc as orc
        return orc.ORCFile(path).read()

    def _column_to_ragged(self, col, conf):
        import numpy as np
        import pyarrow as pa
        col = col.combine_chunks() if hasattr(col, "combine_chunks") else col
        n = len(col)
        if pa.types.is_list(col.type) or pa.types.is_large_list(col.type):
            offsets = np.asarray(col.offsets.to_numpy(zero_copy_only=False), dtype=np.int64)
            offsets = offsets - offsets[0]
            flat = col.flatten()
        else:
            offsets = np.arange(n + 1, dtype=np.int64)
            flat = col
        if pa.types.is_string(flat.type) or pa.types.is_large_string(flat.type) or pa.types.is_binary(flat.type):
            strings = [s if isinstance(s, bytes) else (s or "").encode() for s in flat.to_pylist()]
            data = torch.frombuffer(bytearray(b"".join(strings)) or bytearray(1), dtype=torch.int8)[: sum(len(s) for s in strings)]
            soff = torch.zeros(len(strings) + 1, dtype=torch.int32)
            soff[1:] = torch.cumsum(torch.tensor([len(s) for s in strings], dtype=torch.int64), 0)
            if conf["trans_int8"] or not conf["hash_type"]:
                return RaggedTensor(data, [torch.from_numpy(offsets.astype(np.int32)), soff])
            values = native().fused_hash([data], [soff], 0 if conf["hash_type"] == "farm" else 1)[0]
        else:
            values = torch.from_numpy(np.array(flat.to_numpy(zero_copy_only=False), copy=True)).to(torch.int64)
        if conf["hash_bucket"]:
            values = native().fused_mod([values], [int(conf["hash_bucket"])])[0]
        return RaggedTensor(values, [torch.from_numpy(offsets.astype(np.int32))], dense_shape=(n, -1))

    def _place(self, batch):
        """Output format and placement of one batch: ``ragged_format=False`` turns variable-length columns into sparse COO
        tensors (``recis/io/dataset_base.py:82-90``); ``device`` pins or moves the tensors. Runs before ``transform_fn``."""
        if not self.ragged_format:
            batch = {k: (v.to_sparse() if isinstance(v, RaggedTensor) else v) for k, v in batch.items()}
        if self.pin and torch.cuda.is_available():
            from ..utils.data_utils import pin_data
            batch = {k: (v if (isinstance(v, torch.Tensor) and (v.is_sparse or v.is_pinned())) else pin_data(v)) for k, v in batch.items()}
        if str(self.device) == "cuda" and torch.cuda.is_available():
            from ..utils.data_utils import copy_data_to_device
            batch = copy_data_to_device(batch, "cuda", non_blocking=True)
        return batch

    def _finish(self, batch):
        """Registered map functions, then ``transform_fn`` (one callable or a list of them), then the filter functions
        (``recis/io/dataset_base.py:453-459``). Returns None for a batch that a filter function rejects."""
        batch = self._run_maps(batch)
        if self.transform_fn is not None:
            for f in (self.transform_fn if isinstance(self.transform_fn, (list, tuple)) else [self.transform_fn]):
                batch = f(batch)
        return None if self._filtered_out(batch) else batch

    def _batches_of(self, table, start_row):
        import numpy as np
        n = table.num_rows
        for b in range(start_row, n, self.batch_size):
            e = min(b + self.batch_size, n)
            if self.drop_remainder and e - b < self.batch_size:
                break
            part = table.slice(b, e - b)
            batch = {}
            for name, conf in self._varlen.items():
                batch[name] = self._column_to_ragged(part.column(name), conf)
            for name, default in self._fixed.items():
                col = part.column(name).combine_chunks()
                arr = np.asarray(col.fill_null(default).to_pylist() if col.null_count else col.to_pylist())
                t = torch.as_tensor(arr)
                batch[name] = (t.to(self.dtype) if t.is_floating_point() else t).reshape(e - b, -1)
            batch = self._place(batch)
            batch = self._finish(batch)
            self._row_in_file = e
            if batch is not None:
                yield batch

    def _native(self, paths):
        """The C++ reader (reader threads + packer + prefetch queue, ``csrc_io/columnar_reader.cpp``) when it applies: ORC
        and Parquet files; it is built against the Arrow C++ libraries inside the pyarrow wheel and may be
        unavailable."""
        if not self.native_reader or not paths or not all(p.endswith((".orc", ".parquet")) for p in paths):
            return None
        from .._ext_io import load
        mod = load()
        if mod is None:
            return None
        var = [(n, -1 if not c["hash_type"] else (0 if c["hash_type"] == "farm" else 1), int(c["hash_bucket"] or 0), bool(c["trans_int8"]))
               for n, c in self._varlen.items()]
        fix = [(n, float(d)) for n, d in self._fixed.items()]
        reader = mod.ColumnarReader(paths, self.batch_size, var, fix, max(self.read_threads_num, 1), max(self.prefetch, 1),
                                    self.drop_remainder, self.pin)
        if self._file_idx or self._row_in_file:
            reader.restore(self._file_idx, self._row_in_file)
        return reader

    def _unpack_native(self, rows, cols):
        """One packed batch of the native reader as the batch dict (before placement and user functions)."""
        batch = {}
        for name in list(self._varlen) + list(self._fixed):
            c = cols[name]
            if c[0] == 0:
                batch[name] = RaggedTensor(c[1], [c[2]], dense_shape=(rows, -1))
            elif c[0] == 1:
                batch[name] = RaggedTensor(c[1], [c[2], c[3]])
            else:
                batch[name] = c[1].to(self.dtype) if c[1].is_floating_point() else c[1]
        return batch

    def _drain_native(self, reader, moved=None):
        """Batches of a native reader until it is exhausted: packed columns become RaggedTensors / dense tensors, then placement,
        map / transform / filter functions. ``moved(state)`` is told the reader's position after every batch handed out."""
        while True:
            item = reader.next()
            if item is None:
                return
            batch = self._finish(self._place(self._unpack_native(*item)))
            if moved is not None:
                moved(reader.state())
            if batch is not None:
                yield batch

    def __iter__(self):
        paths = self._my_paths()
        if self._file_idx >= len(paths):
            # a finished pass starts over, as the reference rebuilds its reader graph on every ``__iter__`` (one epoch per
            # iteration, ``recis/io/dataset_base.py:462-464``); a position restored from a checkpoint resumes mid-stream
            self._file_idx, self._row_in_file = 0, 0
        reader = self._native(paths)
        if reader is not None:
            def moved(state):
                self._file_idx, self._row_in_file = state
            yield from self._drain_native(reader, moved)
            return
        while self._file_idx < len(paths):
            table = self._read_table(paths[self._file_idx])
            yield from self._batches_of(table, self._row_in_file)
            self._file_idx += 1
            self._row_in_file = 0

    def get_dir_size(self):
        """Bytes on disk behind every configured path (files, or directories walked recursively)."""
        return [get_dir_size(p) for p in self._paths]

    def dump_io_state(self):
        return {"file_idx": self._file_idx, "row_in_file": self._row_in_file}

    def load_io_state(self, state):
        self._file_idx, self._row_in_file = int(state["file_idx"]), int(state["row_in_file"])


class MapDataset(DatasetBase):
    """``MapDataset(input_dataset, map_funcs)``: every item goes through the functions in order (``recis/io/map_dataset.py:117``).
    ``map_funcs`` may be one callable or a list."""

    def __init__(self, input_dataset, map_funcs):
        self.dataset = input_dataset
        self.map_funcs = list(map_funcs) if isinstance(map_funcs, (list, tuple)) else [map_funcs]

    def __iter__(self):
        for batch in self.dataset:
            for f in self.map_funcs:
                batch = f(batch)
            yield batch

    def dump_io_state(self):
        return self.dataset.dump_io_state()

    def load_io_state(self, state):
        self.dataset.load_io_state(state)


class FilterDataset(DatasetBase):
    """``FilterDataset(input_dataset, filter_funcs)``: an item is skipped when ANY function returns True
    (``recis/io/filter_dataset.py:165``). ``keys`` (an addition) keeps only the listed entries of every batch."""

    def __init__(self, input_dataset, filter_funcs=None, keys: Optional[List[str]] = None):
        self.dataset = input_dataset
        self.filter_funcs = [] if filter_funcs is None else (list(filter_funcs) if isinstance(filter_funcs, (list, tuple)) else [filter_funcs])
        self.keys = keys

    def __iter__(self):
        for batch in self.dataset:
            if any(f(batch) for f in self.filter_funcs):
                continue
            yield {k: batch[k] for k in self.keys} if self.keys else batch

    def dump_io_state(self):
        return self.dataset.dump_io_state()

    def load_io_state(self, state):
        self.dataset.load_io_state(state)


class PrefetchDataset(DatasetBase):
    """Background thread that keeps ``depth`` batches ready (optionally already copied to a device on a side stream)."""

    def __init__(self, dataset, depth: int = 2, device: Optional[str] = None):
        self.dataset, self.depth, self.device = dataset, depth, device

    def __iter__(self):
        q: queue.Queue = queue.Queue(maxsize=self.depth)
        done = object()
        stop = threading.Event()            # set when the consumer goes away early: the worker then stops instead of blocking

        def put(item):
            while not stop.is_set():
                try:
                    q.put(item, timeout=0.1)
                    return True
                except queue.Full:
                    continue
            return False

        def work():
            stream = torch.cuda.Stream() if self.device and str(self.device).startswith("cuda") else None
            try:
                for batch in self.dataset:
                    if self.device:
                        from ..utils.data_utils import copy_data_to_device
                        if stream is not None:
                            with torch.cuda.stream(stream):
                                batch = copy_data_to_device(batch, self.device)
                            stream.synchronize()
                        else:
                            batch = copy_data_to_device(batch, self.device)
                    if not put(batch):
                        return
                put(done)
            except BaseException as e:          # noqa: BLE001 - handed to the consumer, which re-raises it
                put(e)

        worker = threading.Thread(target=work, daemon=True)
        worker.start()
        try:
            while True:
                item = q.get()
                if item is done:
                    return
                if isinstance(item, BaseException):
                    raise item              # an error in the source must not look like the end of the data
                yield item
        finally:
            stop.set()

    def dump_io_state(self):
        return self.dataset.dump_io_state()

    def load_io_state(self, state):
        self.dataset.load_io_state(state)


class StateDataset(DatasetBase):
    """Remembers the source position every ``save_interval`` batches, so that a checkpoint taken between two snapshots
    resumes from the last snapshot (``recis/io/state_dataset.py:118-137``)."""

    def __init__(self, dataset, save_interval: int = 100):
        self.dataset, self.save_interval = dataset, max(int(save_interval), 1)
        self._snapshot = dataset.dump_io_state()
        self._count = 0

    def __iter__(self):
        for batch in self.dataset:
            self._count += 1
            if self._count % self.save_interval == 0:
                self._snapshot = self.dataset.dump_io_state()
            yield batch

    def dump_io_state(self):
        return {"snapshot": self._snapshot, "count": self._count}

    def load_io_state(self, state):
        self._snapshot, self._count = state["snapshot"], int(state.get("count", 0))
        self.dataset.load_io_state(self._snapshot)


class WrapEndDataset(DatasetBase):
    """Yields ``(stop_flag, batch)``; after the source ends it keeps yielding ``(True, last_batch)`` so that ranks whose data
    ran out can keep taking part in collectives until every rank is done (``recis/io/wrap_end_dataset.py:38-79``)."""

    def __init__(self, dataset):
        self.dataset = dataset

    def __iter__(self):
        last = None
        for batch in self.dataset:
            last = batch
            yield False, batch
        while True:
            yield True, last

    def dump_io_state(self):
        return self.dataset.dump_io_state()

    def load_io_state(self, state):
        self.dataset.load_io_state(state)
