"""Row-addressable tables and time-addressable streams behind one small interface.

The reference's internal build reads two more kinds of input than files: tables of a table service, addressed as
``project.table?start=<row>&end=<row>`` (``recis/io/odps_dataset.py:55-379``), and streams of a data lake, addressed by a
time range (``recis/io/lake_dataset.py:8-204``); the readers live in its closed column-io build. Here both are *sources*
registered by name, and the datasets (``io/window_io.py``) only talk to this interface:

``TableSource``   ``size(table) -> rows``, ``read(table, start, end, columns) -> pyarrow.Table``
``StreamSource``  ``read_range(path, begin_us, end_us, columns) -> pyarrow.Table`` (timestamps in microseconds)

Built in:

* ``FileTableSource`` - a "table" is a columnar file, a directory of them or a glob; rows are numbered across the files in
  name order. Row counts come from the files' metadata (no data is read to count), a slice reads only the files it touches.
* ``FileStreamSource`` - a "stream" is a directory whose files (or sub-directories) start with a time stamp
  ``YYYYmmdd[HH[MM[SS]]]``; a range reads the entries whose stamp lies in ``[begin, end)``.
* ``OdpsTableSource`` - the table service through the ``odps`` package (Arrow readers); registered under ``odps`` when the
  package is installed and credentials are given. Not exercised in this repository's tests (no service to talk to).

``resolve_table_source(name)`` picks by prefix: ``odps://project.table`` or a registered scheme, else files.
"""
from __future__ import annotations

import bisect
import datetime as _dt
import glob
import os
import re
from typing import Dict, List, Optional, Sequence, Tuple

US = 1_000_000                                   # stream time stamps are microseconds since the epoch


def _columnar_files(path: str) -> List[str]:
    if os.path.isdir(path):
        out = []
        for root, _dirs, files in os.walk(path):
            out += [os.path.join(root, f) for f in files if f.endswith((".orc", ".parquet")) and not f.startswith(".")]
        return sorted(out)
    if any(ch in path for ch in "*?["):
        return sorted(p for p in glob.glob(path) if p.endswith((".orc", ".parquet")))
    return [path]


def _file_rows(path: str) -> int:
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        return pq.ParquetFile(path).metadata.num_rows
    import pyarrow.orc as orc
    return orc.ORCFile(path).nrows


def _plain_type(t):
    """List types with the default child field name, at any depth: Parquet names a list's child ``element``, ORC ``item``,
    and tables that differ only in that do not concatenate."""
    import pyarrow as pa
    if pa.types.is_list(t) or pa.types.is_large_list(t):
        return pa.list_(_plain_type(t.value_type))
    return t


def _read_file(path: str, columns: Optional[Sequence[str]]):
    """The file's columns as a table: the requested columns in the requested order (readers differ: ORC returns file order), list
    types normalised, so that pieces of a table that come from files of both formats concatenate."""
    import pyarrow as pa
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        table = pq.read_table(path, columns=list(columns) if columns else None)
    else:
        import pyarrow.orc as orc
        table = orc.ORCFile(path).read(columns=list(columns) if columns else None)
    if columns:
        table = table.select(list(columns))
    want = pa.schema([pa.field(f.name, _plain_type(f.type)) for f in table.schema])
    return table if want.equals(table.schema) else table.cast(want)


class FileTableSource:
    """Columnar files as one row-numbered table."""

    _CACHED_FILES = 4                # decoded files kept: consecutive slices of one file decode it once

    def __init__(self):
        import collections
        import threading
        self._index: Dict[str, Tuple[List[str], List[int]]] = {}     # table -> (files, cumulative row counts)
        self._decoded = collections.OrderedDict()                     # (file, columns) -> pyarrow.Table, most recent last
        self._lock = threading.Lock()

    def _file_table(self, path: str, columns: Optional[Sequence[str]]):
        key = (path, tuple(columns) if columns else None)
        with self._lock:
            if key in self._decoded:
                self._decoded.move_to_end(key)
                return self._decoded[key]
        table = _read_file(path, columns)
        with self._lock:
            self._decoded[key] = table
            while len(self._decoded) > self._CACHED_FILES:
                self._decoded.popitem(last=False)
        return table

    def _files(self, table: str):
        if table not in self._index:
            files = _columnar_files(table)
            if not files or not all(os.path.exists(f) for f in files):
                raise FileNotFoundError(f"table {table!r}: no columnar files")
            cum, total = [], 0
            for f in files:
                total += _file_rows(f)
                cum.append(total)
            self._index[table] = (files, cum)
        return self._index[table]

    def size(self, table: str) -> int:
        _files, cum = self._files(table)
        return cum[-1] if cum else 0

    def read(self, table: str, start: int, end: int, columns: Optional[Sequence[str]] = None):
        import pyarrow as pa
        files, cum = self._files(table)
        end = min(end, cum[-1])
        parts = []
        i = bisect.bisect_right(cum, start)
        while i < len(files) and start < end:
            base = cum[i - 1] if i else 0
            take = min(end, cum[i]) - start
            parts.append(self._file_table(files[i], columns).slice(start - base, take))
            start += take
            i += 1
        if not parts:
            return self._file_table(files[0], columns).slice(0, 0)
        return pa.concat_tables(parts) if len(parts) > 1 else parts[0]


_STAMP = re.compile(r"^(\d{8})(\d{2})?(\d{2})?(\d{2})?")


def stamp_to_us(text: str) -> Optional[int]:
    """Leading ``YYYYmmdd[HH[MM[SS]]]`` of a name as microseconds since the epoch (UTC); None when the name has no stamp."""
    m = _STAMP.match(text)
    if not m:
        return None
    d, hh, mm, ss = m.groups()
    try:
        t = _dt.datetime(int(d[:4]), int(d[4:6]), int(d[6:8]), int(hh or 0), int(mm or 0), int(ss or 0), tzinfo=_dt.timezone.utc)
    except ValueError:
        return None
    return int(t.timestamp()) * US


def us_to_stamp(ts_us: int, fmt: str = "%Y%m%d%H%M%S") -> str:
    return _dt.datetime.fromtimestamp(ts_us / US, tz=_dt.timezone.utc).strftime(fmt)


class FileStreamSource:
    """A directory of time-stamped files or sub-directories as a stream."""

    def entries(self, path: str) -> List[Tuple[int, str]]:
        if not os.path.isdir(path):
            return []
        out = []
        for name in os.listdir(path):
            ts = stamp_to_us(name)
            if ts is not None and not name.startswith("."):
                out.append((ts, os.path.join(path, name)))
        return sorted(out)

    def read_entry(self, entry: str, columns: Optional[Sequence[str]] = None):
        """One listed entry (a file, or a directory of files) as a table; None when it holds nothing."""
        import pyarrow as pa
        parts = [_read_file(f, columns) for f in _columnar_files(entry)]
        if not parts:
            return None
        return pa.concat_tables(parts) if len(parts) > 1 else parts[0]

    def read_range(self, path: str, begin_us: int, end_us: int, columns: Optional[Sequence[str]] = None):
        import pyarrow as pa
        parts = [self.read_entry(entry, columns) for ts, entry in self.entries(path) if begin_us <= ts < end_us]
        parts = [p for p in parts if p is not None]
        if not parts:
            return None
        return pa.concat_tables(parts) if len(parts) > 1 else parts[0]


class OdpsTableSource:
    """The table service through the ``odps`` package: ``table`` is ``project.table[/partition_spec]``. Row ranges are read as
    Arrow record batches from a download session."""

    def __init__(self, access_id: str, access_key: str, end_point: str, project: Optional[str] = None):
        try:
            from odps import ODPS
        except ImportError as e:
            raise ImportError("reading from the table service needs the 'odps' package") from e
        self._client = ODPS(access_id, access_key, project, end_point)

    def _open(self, table: str):
        name, _, partition = table.partition("/")
        project, _, tname = name.rpartition(".")
        t = self._client.get_table(tname, project=project or None)
        return t.open_reader(partition=partition or None, arrow=True)

    def size(self, table: str) -> int:
        with self._open(table) as reader:
            return int(reader.count)

    def read(self, table: str, start: int, end: int, columns: Optional[Sequence[str]] = None):
        import pyarrow as pa
        with self._open(table) as reader:
            batches = list(reader.read(start=start, count=end - start, columns=list(columns) if columns else None))
        return pa.Table.from_batches(batches)


_TABLE_SOURCES: Dict[str, object] = {"file": FileTableSource()}
_STREAM_SOURCES: Dict[str, object] = {"file": FileStreamSource()}


def register_table_source(scheme: str, source) -> None:
    """Make ``<scheme>://...`` table names read through ``source`` (an object with ``size`` and ``read``)."""
    _TABLE_SOURCES[scheme] = source


def register_stream_source(scheme: str, source) -> None:
    _STREAM_SOURCES[scheme] = source


def _split_scheme(name: str):
    m = re.match(r"^([A-Za-z][A-Za-z0-9+.-]*)://(.*)$", name)
    return (m.group(1), m.group(2)) if m else (None, name)


def resolve_table_source(name: str):
    """``(source, name without scheme)``; names without a registered scheme are files."""
    scheme, rest = _split_scheme(name)
    if scheme in _TABLE_SOURCES and scheme != "file":
        return _TABLE_SOURCES[scheme], rest
    if scheme == "odps":
        raise RuntimeError("no table source registered for odps://; call register_table_source('odps', OdpsTableSource(...))")
    return _TABLE_SOURCES["file"], (rest if scheme == "file" else name)


def resolve_stream_source(name: str):
    scheme, rest = _split_scheme(name)
    if scheme in _STREAM_SOURCES and scheme != "file":
        return _STREAM_SOURCES[scheme], rest
    return _STREAM_SOURCES["file"], (rest if scheme == "file" else name)


def get_table_size(table_name: str) -> int:
    """Rows of a table (``recis/io/odps_dataset.py:36-52``)."""
    src, name = resolve_table_source(table_name)
    return int(src.size(name))
