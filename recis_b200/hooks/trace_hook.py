"""Sample-level tracing: tensors named during a step are appended, row by row, to a columnar table.

The reference uploads such traces to a proprietary table service from writer processes
(``recis/hooks/trace_to_odps_hook.py:63-465``: ``add_to_trace`` fills a global map, ``TraceToOdpsHook.after_step`` hands the
map to ``TraceWriter`` processes, which buffer rows up to a size threshold and upload blocks). The same interface here, with
the destination behind a small sink interface:

* ``ParquetSink`` - Parquet parts under a directory or any fsspec URL (``hdfs://``, ``s3://``, ``memory://`` ...), one
  sub-directory per partition spec (``dt=20250101,hh=10`` becomes ``dt=20250101/hh=10``), which every columnar reader
  (this framework's included) reads back; chosen when the config has ``output_dir``.
* ``OdpsSink`` - the table service of the reference through the ``odps`` package, when that package is installed and the
  config carries its credentials.

Differences that come from running next to a GPU that must not be stalled: a CUDA tensor passed to ``add_to_trace`` is
copied to pinned host memory on a side stream and only read once its event has completed (in ``after_step``), so tracing adds
no synchronisation to the step; writers are threads of the training process (Arrow and Parquet encoding release the GIL), so
nothing is pickled across processes and no second CUDA context appears.
"""
from __future__ import annotations

import atexit
import functools
import os
import queue
import threading
import time
from typing import Dict, List, Optional, Union

import numpy as np
import torch

from ..utils.logger import Logger
from .hook import Hook

logger = Logger(__name__)

TRACE_MAP: Dict[str, object] = {}
_copy_stream = None


def retry(retry_count: int, interval: float):
    """Decorator: call again after ``interval`` seconds, at most ``retry_count`` times in all, then re-raise."""
    def decorator(func):
        @functools.wraps(func)
        def wrapper(*args, **kwargs):
            for attempt in range(retry_count):
                try:
                    return func(*args, **kwargs)
                except Exception as e:      # noqa: BLE001 - whatever the sink raised is retried, the last one propagates
                    if attempt + 1 >= retry_count:
                        raise
                    logger.warning(f"{func.__name__} failed ({e!r}), retry {attempt + 1}/{retry_count - 1}")
                    time.sleep(interval)
        return wrapper
    return decorator


class _PendingCopy:
    """A device tensor on its way to pinned host memory."""

    def __init__(self, t: torch.Tensor):
        global _copy_stream
        if _copy_stream is None:
            _copy_stream = torch.cuda.Stream(device=t.device)
        src = t.detach()
        self.host = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
        _copy_stream.wait_stream(torch.cuda.current_stream(t.device))
        with torch.cuda.stream(_copy_stream):
            self.host.copy_(src, non_blocking=True)
            src.record_stream(_copy_stream)
            self.event = torch.cuda.Event()
            self.event.record(_copy_stream)

    def numpy(self) -> np.ndarray:
        self.event.synchronize()
        h = self.host
        return (h.float() if h.dtype in (torch.bfloat16, torch.float16) else h).numpy()


def add_to_trace(name: str, tensor: Union[torch.Tensor, np.ndarray, list] = None):
    """Name one column of this step's trace rows (``recis/hooks/trace_to_odps_hook.py:63-104``). The leading dimension is the
    row (sample) dimension; further dimensions become a list column."""
    if not isinstance(tensor, (torch.Tensor, np.ndarray, list)):
        raise ValueError(f"Trace data must be torch.Tensor or np.ndarray or list, not now {type(tensor)}")
    if name in TRACE_MAP:
        logger.warning(f"Trace data {name} already exists")
    if isinstance(tensor, torch.Tensor):
        if tensor.is_cuda:
            TRACE_MAP[name] = _PendingCopy(tensor)
        else:
            t = tensor.detach()
            TRACE_MAP[name] = (t.float() if t.dtype in (torch.bfloat16, torch.float16) else t).numpy().copy()
    else:
        TRACE_MAP[name] = tensor


def get_trace_map() -> Dict[str, object]:
    """This step's columns; device tensors have arrived on the host when this returns."""
    for k, v in list(TRACE_MAP.items()):
        if isinstance(v, _PendingCopy):
            TRACE_MAP[k] = v.numpy()
    return TRACE_MAP


def clear_trace_map():
    global TRACE_MAP
    TRACE_MAP = {}


# ---------------------------------------------------------------------------------------------------------------- schema
_ARROW_SCALARS = {
    "tinyint": "int8", "smallint": "int16", "int": "int32", "bigint": "int64", "float": "float32", "double": "float64",
    "string": "string", "boolean": "bool_", "binary": "binary",
}


def arrow_type(type_name: str):
    """Arrow type of a column type written the way the table service writes it: ``bigint``, ``double``, ``string``,
    ``array<bigint>``, ``array<array<double>>`` ..."""
    import pyarrow as pa
    t = type_name.strip().lower()
    if t.startswith("array<") and t.endswith(">"):
        return pa.list_(arrow_type(t[6:-1]))
    if t not in _ARROW_SCALARS:
        raise ValueError(f"unsupported trace column type {type_name!r}")
    return getattr(pa, _ARROW_SCALARS[t])()


def _column(values, typ):
    import pyarrow as pa
    if isinstance(values, np.ndarray) and values.ndim > 1:
        values = values.tolist()              # nested lists: list columns of any depth
    elif isinstance(values, np.ndarray) and pa.types.is_string(typ):
        values = [str(v) for v in values.tolist()]
    return pa.array(values, type=typ)


def rows_to_table(data: Dict[str, object], fields: List[str], types: List[str]):
    """One Arrow table of the declared schema from a step's columns; every column must have the same number of rows."""
    import pyarrow as pa
    missing = [f for f in fields if f not in data]
    if missing:
        raise KeyError(f"trace step lacks declared fields {missing}")
    cols, n = [], None
    for f, t in zip(fields, types):
        c = _column(data[f], arrow_type(t))
        if n is not None and len(c) != n:
            raise ValueError(f"trace field {f} has {len(c)} rows, the fields before it {n}")
        n = len(c)
        cols.append(c)
    return pa.Table.from_arrays(cols, names=list(fields))


# ----------------------------------------------------------------------------------------------------------------- sinks
class ParquetSink:
    """Blocks become ``<output_dir>/<partition dirs>/part-w<writer>-<seq>.parquet``. A part is written under a temporary name and
    renamed, so a reader of the directory never sees half a file; ``commit`` has nothing left to do."""

    def __init__(self, output_dir: str, partition: Optional[str] = None, writer_id: int = 0, compression: str = "zstd"):
        import fsspec
        self.fs, root = fsspec.core.url_to_fs(str(output_dir))
        parts = [p.strip() for p in (partition or "").split(",") if p.strip()]
        self.dir = "/".join([root.rstrip("/")] + parts)
        self.fs.makedirs(self.dir, exist_ok=True)
        self.writer_id, self.compression, self.seq = writer_id, compression, 0
        self.run = f"{int(time.time() * 1000):x}-{os.getpid():x}"

    def write_block(self, table):
        import pyarrow.parquet as pq
        name = f"part-w{self.writer_id}-{self.run}-{self.seq:06d}.parquet"
        tmp = f"{self.dir}/.{name}.tmp"
        with self.fs.open(tmp, "wb") as f:
            pq.write_table(table, f, compression=self.compression)
        self.fs.mv(tmp, f"{self.dir}/{name}")
        self.seq += 1

    def commit(self):
        pass


class OdpsSink:
    """The reference's destination (``recis/hooks/trace_to_odps_hook.py:195-330``): an upload session of the table service,
    one Arrow block per flush, committed every two blocks. Needs the ``odps`` package and the config keys ``access_id,
    access_key, project, end_point, table_name`` (``partition`` optional)."""

    def __init__(self, config: Dict, fields: List[str], types: List[str], writer_id: int = 0):
        try:
            from odps import ODPS
            from odps.models import Schema
            from odps.tunnel import TableTunnel
        except ImportError as e:
            raise ImportError("tracing into the table service needs the 'odps' package; give the config an 'output_dir' to "
                              "write Parquet parts instead") from e
        client = ODPS(config["access_id"], config["access_key"], config["project"], config["end_point"])
        self.table_name, self.partition = config["table_name"], config.get("partition")
        pnames = [s.split("=")[0] for s in (self.partition or "").split(",") if s]
        table = client.create_table(self.table_name, schema=Schema.from_lists(fields, types, pnames, ["string"] * len(pnames)),
                                    if_not_exists=True, lifecycle=365, table_properties={"columnar.nested.type": "true"})
        if self.partition:
            table.create_partition(self.partition, if_not_exists=True)
        self._tunnel = TableTunnel(client)
        self._session = self._tunnel.create_upload_session(table.name, partition_spec=self.partition)
        self._block = 0

    def write_block(self, table):
        w = self._session.open_arrow_writer(self._block)
        for batch in table.to_batches():
            w.write(batch)
        w.close()
        self._block += 1
        if self._block == 2:
            self.commit()

    def commit(self):
        if self._block > 0:
            self._session.commit(list(range(self._block)))
            self._session = self._tunnel.create_upload_session(self.table_name, partition_spec=self.partition)
            self._block = 0


def make_sink(config: Dict, fields: List[str], types: List[str], writer_id: int):
    if config.get("sink") is not None:                     # an object with write_block(table) / commit()
        return config["sink"]
    if config.get("output_dir"):
        return ParquetSink(config["output_dir"], config.get("partition"), writer_id, config.get("compression", "zstd"))
    return OdpsSink(config, fields, types, writer_id)


# ---------------------------------------------------------------------------------------------------------------- writer
class TraceWriter(threading.Thread):
    """Takes steps' columns from a queue, buffers them as Arrow tables until ``size_threshold`` bytes are held, then writes one
    block (``recis/hooks/trace_to_odps_hook.py:152-340``). ``None`` on the queue flushes what is left and ends the thread; an
    exception ends it too and is kept in ``error`` for the hook to raise in the training thread."""

    def __init__(self, config: Dict, fields: List[str], types: List[str], writer_id: int, q: "queue.Queue",
                 size_threshold: int = 50 * 1024 * 1024):
        super().__init__(daemon=True, name=f"trace-writer-{writer_id}")
        self.fields, self.types, self.queue, self.size_threshold = list(fields), list(types), q, size_threshold
        self.sink = make_sink(config, self.fields, self.types, writer_id)
        self.buffer, self.buffered_size, self.write_count, self.error = [], 0, 0, None

    def run(self):
        try:
            while True:
                data = self.queue.get()
                if data is None:
                    self.flush(force=True)
                    return
                self.write(data)
        except BaseException as e:      # noqa: BLE001 - reported by the hook
            self.error = e
            logger.error(f"{self.name} stopped: {e!r}")

    def write(self, data: Dict[str, object]):
        table = rows_to_table(data, self.fields, self.types)
        self.buffer.append(table)
        self.buffered_size += table.nbytes
        if self.buffered_size >= self.size_threshold:
            self._flush_buffer()

    @retry(retry_count=3, interval=10)
    def _write_block(self, table):
        self.sink.write_block(table)

    def _flush_buffer(self):
        if not self.buffer:
            return
        import pyarrow as pa
        table = pa.concat_tables(self.buffer)
        self._write_block(table)
        self.write_count += table.num_rows
        self.buffer, self.buffered_size = [], 0

    @retry(retry_count=3, interval=10)
    def _commit(self):
        self.sink.commit()

    def flush(self, force: bool = False):
        if force:
            self._flush_buffer()
        self._commit()


class TraceToOdpsHook(Hook):
    """After every step, hand the columns named with ``add_to_trace`` to the writers
    (``recis/hooks/trace_to_odps_hook.py:343-465``).

    ``config``: ``{"output_dir": <dir or URL>, "partition": "dt=...,hh=..."}`` for Parquet parts, or the table service's keys
    (see ``OdpsSink``). ``fields`` / ``types``: the table's columns, types spelled ``bigint, double, string, array<...>``."""

    def __init__(self, config: Dict, fields: List[str], types: List[str], worker_num: int = 1, size_threshold: int = 50 * 1024 * 1024):
        if len(fields) != len(types):
            raise ValueError("fields and types must have the same length")
        self.queue = queue.Queue(maxsize=max(1, worker_num))
        self.writers = [TraceWriter(config, fields, types, i, self.queue, size_threshold) for i in range(worker_num)]
        for w in self.writers:
            w.start()
        # a run that ends without calling end() (an exception in the loop) still flushes what the writers hold
        self._ended = False
        atexit.register(self._end_at_exit)

    def _end_at_exit(self):
        # writers that already failed were reported in after_step; there is nothing left to flush for them
        if self._ended or any(w.error is not None for w in self.writers):
            return
        try:
            self.end()
        except Exception:       # noqa: BLE001 - the interpreter is going down and its log streams may be closed already
            pass

    def check_alive(self) -> bool:
        return all(w.is_alive() and w.error is None for w in self.writers)

    def _raise_writer_error(self):
        for w in self.writers:
            if w.error is not None:
                raise ValueError("TraceToOdpsHook writer raised an error") from w.error
        raise ValueError("TraceToOdpsHook writer stopped unexpectedly")

    def _put(self, item):
        """Queue an item without ever blocking on writers that are gone (the queue is short on purpose: a slow sink holds
        the training loop back instead of piling steps up in memory)."""
        while True:
            try:
                self.queue.put(item, timeout=1.0)
                return
            except queue.Full:
                if not any(w.is_alive() for w in self.writers):
                    self._raise_writer_error()

    def after_step(self, *args, **kw):
        if not self.check_alive():
            self._raise_writer_error()
        data = get_trace_map()
        if data:
            self._put(dict(data))
        clear_trace_map()

    def end(self):
        if self._ended:
            return
        self._ended = True
        for w in self.writers:
            if w.is_alive():
                self._put(None)
        for w in self.writers:
            w.join()
        for w in self.writers:
            if w.error is not None:
                self._raise_writer_error()

    @property
    def rows_written(self) -> int:
        return sum(w.write_count for w in self.writers)


TraceHook = TraceToOdpsHook
