"""Datasets over row-addressable tables and time-addressable streams, and their windowed forms.

What the reference's internal build offers (``recis/io/odps_dataset.py``, ``lake_dataset.py``, ``window_io.py``), on the
sources of ``io/table_source.py`` (columnar files out of the box; a table service or a data lake by registering a source):

``OdpsDataset``           reads tables by row range: each table's rows are cut into ``worker_num * read_threads_num`` slices,
                          worker ``w`` reads slices ``w, w + worker_num, ...`` (``recis/io/odps_dataset.py:286-320``)
``LakeStreamDataset``     reads ``[begin, end)`` time ranges of streams (``recis/io/lake_dataset.py:150-204``)
``make_odps_window_io``   a table is consumed window by window (``next_window()`` until ``StopIteration``), a window being
                          ``read_threads_num`` slices; tables can be mixed in fixed proportions: with proportions (2, 3) and
                          (1, 3) two thirds of every batch come from the first table (``recis/io/window_io.py:268-556``)
``make_odps_sample_io``   one window of ``row_num`` rows at a seeded random offset (``:557-668``)
``make_lake_stream_window_io``  a time window of fixed length that moves forward by ``step_mins`` per ``next_window()``,
                          optionally read in ``repeat_mins`` pieces (``:680-815``)

A window's state is one integer (slices consumed, or the window's start time), so ``state_dict()`` / ``load_state_dict()`` resume
exactly. Batches are built by the same column conversion as ``OrcDataset`` (``varlen_feature`` / ``fixedlen_feature``, placement,
``transform_fn``, map and filter functions).
"""
from __future__ import annotations

import math
import random
from typing import List, Optional, Sequence, Tuple

import torch

from ..ragged import RaggedTensor
from ..utils.logger import Logger
from .dataset import OrcDataset
from .table_source import US, get_table_size, resolve_stream_source, resolve_table_source, us_to_stamp

logger = Logger(__name__)

_READ_CHUNK_ROWS = 1 << 16          # rows fetched from a source per request


class TableSheet:
    """Rows ``[start, end)`` of one table."""

    __slots__ = ("table", "start", "end")

    def __init__(self, table: str, start: int, end: int):
        self.table, self.start, self.end = table, int(start), int(end)

    def __repr__(self):
        return f"{self.table}?start={self.start}&end={self.end}"

    @classmethod
    def parse(cls, text: str) -> "TableSheet":
        table, _, query = text.partition("?")
        kv = dict(p.split("=") for p in query.split("&") if p)
        return cls(table, int(kv["start"]), int(kv["end"]))


def _parse_proportion(thread_num: int, proportions: Sequence[Tuple[int, int]]):
    """Threads per table for proportions ``(parts, total)``: every part gets ``ceil(thread_num / total)`` threads.
    Returns ``(threads per table of one full group, threads in a group)``; ``[(2, 3), (1, 3)]`` with 6 threads gives
    ``([4, 2], 6)``."""
    totals = {t for _, t in proportions}
    if len(totals) != 1:
        raise ValueError(f"total split num should consistency, but get {totals}")
    total = totals.pop()
    per_part = int(math.ceil(float(thread_num) / total))
    acc, threads = 0, []
    for parts, _ in proportions:
        acc += parts
        threads.append(per_part * parts)
        if acc > total:
            raise ValueError(f"invalid proportions: {proportions}")
        if acc == total:
            break
    return threads, total * per_part


def _build_shard(begin: int, length: int, num: int, extra_offset: int = 0):
    """``num`` consecutive ranges covering ``length`` rows from ``begin``; the ``length % num`` longer ones start at
    ``extra_offset`` so that repeated calls spread the surplus. Returns ``(ranges, next extra_offset)``."""
    sizes = [length // num] * num
    for i in range(length % num):
        sizes[(extra_offset + i) % num] += 1
    out = []
    for s in sizes:
        out.append((begin, begin + s))
        begin += s
    return out, (extra_offset + length) % num


def _shard_sheets_by_split_num(table, task_id, task_num, thread_num, split_num, extra_offset):
    shards, extra_offset = _build_shard(0, get_table_size(table), task_num * thread_num * split_num, extra_offset)
    return [TableSheet(table, s, e) for s, e in shards][task_id::task_num], extra_offset


def _shard_sheets_by_row_num(table, task_id, task_num, thread_num, row_num, extra_offset):
    size, sheets = get_table_size(table), []
    for off in range(0, size, row_num * task_num):
        shards, extra_offset = _build_shard(off, min(row_num * task_num, size - off), task_num * thread_num, extra_offset)
        sheets += [TableSheet(table, s, e) for s, e in shards]
    return sheets[task_id::task_num], extra_offset


def _shard_table_by_subprocess(sheets: Sequence[TableSheet], sub_id: int, sub_num: int) -> List[str]:
    """Sub-process ``sub_id`` of ``sub_num`` takes its consecutive share of every sheet."""
    out = []
    for sh in sheets:
        size = sh.end - sh.start
        each, extra = size // sub_num, size % sub_num
        start = sh.start + sub_id * each + min(sub_id, extra)
        end = sh.start + (sub_id + 1) * each + min(sub_id + 1, extra)
        out.append(repr(TableSheet(sh.table, start, end)))
    return out


class OdpsDataset(OrcDataset):
    """Tables read by row range. ``add_path("project.table")`` (or a file, directory or glob of columnar files; or
    ``scheme://name`` of a registered source). Constructor as ``OrcDataset``."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._shard_paths: Optional[List[str]] = None
        self._sheet_idx, self._row_in_sheet = 0, 0
        self._stream_width = 1            # sheets read side by side into one batch (proportional windows)

    # ---- configuration
    def add_path(self, odps_table: str):
        self._paths.append(odps_table)

    def add_paths(self, odps_tables: List[str]):
        for t in odps_tables:
            self.add_path(t)

    def get_table_size(self):
        return [get_table_size(t) for t in self._paths]

    def _columns(self):
        return list(self._varlen) + list(self._fixed)

    # ---- sharding
    def _shard_path(self, sub_id: int = 0, sub_num: int = 1):
        sheets = []
        for table in self._paths:
            shards, _ = _build_shard(0, get_table_size(table), self.worker_num * self.read_threads_num)
            sheets += [TableSheet(table, s, e) for s, e in shards][self.worker_idx::self.worker_num]
        self._shard_paths = _shard_table_by_subprocess(sheets, sub_id, sub_num)

    # ---- reading
    def _sheet_tables(self, sheet: TableSheet, from_row: int):
        """The sheet's rows as Arrow tables of up to ``_READ_CHUNK_ROWS`` rows, in order. Up to ``read_threads_num`` requests are
        in flight on reader threads (sources release the interpreter lock while they read and decode), so the consumer finds the
        next chunk ready; the order of the results, and with it the batch sequence and the resumable position, does not depend
        on which request finishes first."""
        src, name = resolve_table_source(sheet.table)
        columns = self._columns()
        chunks = [(row, min(row + _READ_CHUNK_ROWS, sheet.end)) for row in range(sheet.start + from_row, sheet.end, _READ_CHUNK_ROWS)]
        depth = max(int(self.read_threads_num), 1)
        if depth == 1 or len(chunks) <= 1:
            for lo, hi in chunks:
                yield src.read(name, lo, hi, columns)
            return
        from collections import deque
        from concurrent.futures import ThreadPoolExecutor
        pool = ThreadPoolExecutor(max_workers=depth, thread_name_prefix="table-read")
        try:
            pending, nxt = deque(), 0
            while pending or nxt < len(chunks):
                while nxt < len(chunks) and len(pending) < depth:
                    pending.append(pool.submit(src.read, name, chunks[nxt][0], chunks[nxt][1], columns))
                    nxt += 1
                yield pending.popleft().result()
        finally:
            pool.shutdown(wait=False, cancel_futures=True)

    def _sheet_batches(self, sheet: TableSheet, from_row: int, rows_per_batch: int):
        """Arrow tables of up to ``rows_per_batch`` rows from one sheet, in order."""
        import pyarrow as pa
        held, held_rows = [], 0
        for t in self._sheet_tables(sheet, from_row):
            held.append(t)
            held_rows += t.num_rows
            while held_rows >= rows_per_batch:
                whole = pa.concat_tables(held) if len(held) > 1 else held[0]
                yield whole.slice(0, rows_per_batch)
                rest = whole.slice(rows_per_batch)
                held, held_rows = ([rest] if rest.num_rows else []), rest.num_rows
        if held_rows:
            yield pa.concat_tables(held) if len(held) > 1 else held[0]

    def _to_batch(self, table):
        old = self.batch_size
        self.batch_size = max(table.num_rows, 1)          # one batch out of exactly these rows
        try:
            for b in self._batches_of(table, 0):
                return b
        finally:
            self.batch_size = old
        return None

    # ---- the native reader, when every sheet is a slice of columnar files
    def _file_segments(self, sheets):
        """``[(sheet index, rows of the sheet before the segment, file, first row, end row)]`` covering the sheets in order, or
        None when a sheet is not backed by files."""
        from .table_source import FileTableSource
        import bisect
        segs = []
        for si, sh in enumerate(sheets):
            src, name = resolve_table_source(sh.table)
            if not isinstance(src, FileTableSource):
                return None
            files, cum = src._files(name)
            row, end = sh.start, min(sh.end, cum[-1] if cum else 0)
            i = bisect.bisect_right(cum, row)
            while i < len(files) and row < end:
                base = cum[i - 1] if i else 0
                take = min(end, cum[i]) - row
                segs.append((si, row - sh.start, files[i], row - base, row - base + take))
                row += take
                i += 1
        return segs

    def _segment_reader(self, mod, segs, batch_size, threads, drop_remainder):
        var = [(n, -1 if not c["hash_type"] else (0 if c["hash_type"] == "farm" else 1), int(c["hash_bucket"] or 0), bool(c["trans_int8"]))
               for n, c in self._varlen.items()]
        fix = [(n, float(d)) for n, d in self._fixed.items()]
        try:
            return mod.ColumnarReader([seg[2] for seg in segs], batch_size, var, fix, threads, max(self.prefetch, 1), drop_remainder, self.pin,
                                      ranges=[(seg[3], seg[4]) for seg in segs])
        except TypeError:                      # a reader built before row ranges existed
            return None

    def _joined_pieces(self, reader, per, segs=None):
        """``(sheet, unpacked piece)`` of exactly ``per`` rows each (the last one of a sheet shorter). The reader cuts a piece at
        every file boundary; short pieces are joined up, as the Python path does. With ``segs`` the pieces of different sheets
        are never joined (``sheet`` is the index of the sheet a piece comes from, else None)."""
        held, held_rows, cur = [], 0, None
        pos = reader.state()                      # (entry, row) of the piece that comes next
        while True:
            entry = pos[0]
            item = reader.next()
            if item is None:
                break
            sheet = segs[entry][0] if segs is not None and entry < len(segs) else None
            if held_rows and sheet != cur:
                yield cur, self._merge_pieces(held)
                held, held_rows = [], 0
            cur = sheet
            held.append(self._unpack_native(*item))
            held_rows += item[0]
            if held_rows == per and len(held) == 1:        # the common case: a full piece, nothing to join or cut
                yield cur, held[0]
                held, held_rows = [], 0
            while held_rows >= per:
                whole = self._merge_pieces(held)
                yield cur, self._slice_rows(whole, 0, per)
                rest = self._slice_rows(whole, per, held_rows)
                held_rows -= per
                held = [rest] if held_rows else []
            pos = reader.state()
        if held_rows:
            yield cur, self._merge_pieces(held)

    @staticmethod
    def _piece_rows(piece) -> int:
        first = next(iter(piece.values()))
        return first.offsets()[0].numel() - 1 if isinstance(first, RaggedTensor) else first.shape[0]

    def _iter_native_wide(self, group, per):
        """A window's sheets read side by side by one native reader each: a batch is one packed piece of ``per`` rows from every
        sheet that still has rows, concatenated in sheet order. None when the native reader does not apply."""
        if not self.native_reader:
            return None
        from .._ext_io import load
        mod = load()
        if mod is None:
            return None
        readers = []
        for sh in group:
            segs = self._file_segments([sh])
            if segs is None or not all(seg[2].endswith((".orc", ".parquet")) for seg in segs):
                return None
            if segs:
                r = self._segment_reader(mod, segs, per, 1, False)
                if r is None:
                    return None
                readers.append(r)

        def run():
            streams = [self._joined_pieces(r, per) for r in readers]
            while streams:
                parts, alive = [], []
                for s in streams:
                    got = next(s, None)
                    if got is not None:
                        parts.append(got[1])
                        alive.append(s)
                streams = alive
                if not parts:
                    return
                merged = self._merge_pieces(parts)
                if self.drop_remainder and self._piece_rows(merged) < self.batch_size:
                    continue
                batch = self._finish(self._place(merged))
                if batch is not None:
                    yield batch

        return run()

    @staticmethod
    def _merge_pieces(parts):
        if len(parts) == 1:
            return parts[0]
        return {k: (RaggedTensor.concat([p[k] for p in parts]) if isinstance(parts[0][k], RaggedTensor) else torch.cat([p[k] for p in parts]))
                for k in parts[0]}

    @staticmethod
    def _slice_rows(batch, lo, hi):
        """Rows ``[lo, hi)`` of an unpacked batch."""
        out = {}
        for k, v in batch.items():
            if not isinstance(v, RaggedTensor):
                out[k] = v[lo:hi]
                continue
            offs = v.offsets()
            a, b = lo, hi
            new_offs = []
            for o in offs:                         # outer to inner: the row range becomes a range of the next level
                piece = o[a:b + 1]
                a2, b2 = int(piece[0]), int(piece[-1])
                new_offs.append(piece - piece[0])
                a, b = a2, b2
            w = v.weight()
            out[k] = RaggedTensor(v.values()[a:b], new_offs, weight=None if w is None else w[a:b],
                                  dense_shape=(hi - lo,) + tuple(v._dense_shape[1:]))
        return out

    def _iter_native(self, sheets):
        """Batches of the sheets through the C++ reader (reader threads, packer, prefetch queue), or None when it does not apply.
        The reader cuts at file boundaries; its pieces are joined into the same batches as on the Python path (full batches
        within a sheet, a shorter one at a sheet's end), and the position kept for ``dump_io_state`` is the same (sheet, row in
        sheet) pair."""
        if not self.native_reader or not sheets:
            return None
        segs = self._file_segments(sheets)
        if not segs or not all(seg[2].endswith((".orc", ".parquet")) for seg in segs):
            return None
        from .._ext_io import load
        mod = load()
        if mod is None:
            return None
        # (remainders are dropped below, after joining: the reader would drop one at every file boundary)
        reader = self._segment_reader(mod, segs, self.batch_size, max(self.read_threads_num, 1), False)
        if reader is None:
            return None
        # resume: the segment that holds (sheet, row in sheet)
        start = next((k for k, seg in enumerate(segs) if seg[0] == self._sheet_idx and seg[1] + (seg[4] - seg[3]) > self._row_in_sheet),
                     next((k for k, seg in enumerate(segs) if seg[0] > self._sheet_idx), len(segs)))
        if start >= len(segs):
            return iter(())
        if start or self._row_in_sheet:
            seg = segs[start]
            reader.restore(start, seg[3] + max(self._row_in_sheet - seg[1], 0) if seg[0] == self._sheet_idx else seg[3])

        first_sheet, first_row = self._sheet_idx, self._row_in_sheet

        def run():
            done = {}                                  # rows handed out per sheet in this pass
            for sheet, piece in self._joined_pieces(reader, self.batch_size, segs):
                n = self._piece_rows(piece)
                done[sheet] = done.get(sheet, first_row if sheet == first_sheet else 0) + n
                size = sheets[sheet].end - sheets[sheet].start
                self._sheet_idx, self._row_in_sheet = (sheet + 1, 0) if done[sheet] >= size else (sheet, done[sheet])
                if self.drop_remainder and n < self.batch_size:
                    continue
                batch = self._finish(self._place(piece))
                if batch is not None:
                    yield batch
            self._sheet_idx, self._row_in_sheet = len(sheets), 0

        return run()

    def __iter__(self):
        import pyarrow as pa
        if self._shard_paths is None:
            self._shard_path()
        sheets = [TableSheet.parse(p) for p in self._shard_paths]
        width = max(self._stream_width, 1)
        if self._sheet_idx >= len(sheets):
            self._sheet_idx, self._row_in_sheet = 0, 0
        if width == 1:
            native = self._iter_native(sheets)
            if native is not None:
                yield from native
                return
        while self._sheet_idx < len(sheets):
            group = sheets[self._sheet_idx:self._sheet_idx + width]
            per = int(math.ceil(self.batch_size / len(group))) if width > 1 else self.batch_size
            if width > 1:
                native = self._iter_native_wide(group, per)
                if native is not None:
                    yield from native
                    self._sheet_idx += len(group)
                    self._row_in_sheet = 0
                    continue
            streams = [self._sheet_batches(sh, self._row_in_sheet if width == 1 else 0, per) for sh in group]
            while streams:
                parts, alive = [], []
                for s in streams:
                    t = next(s, None)
                    if t is not None:
                        parts.append(t)
                        alive.append(s)
                streams = alive
                if not parts:
                    break
                table = pa.concat_tables(parts) if len(parts) > 1 else parts[0]
                if self.drop_remainder and table.num_rows < self.batch_size:
                    continue
                if width == 1:
                    self._row_in_sheet += table.num_rows
                batch = self._to_batch(table)
                if batch is not None:
                    yield batch
            self._sheet_idx += len(group)
            self._row_in_sheet = 0

    def dump_io_state(self):
        return {"sheet_idx": self._sheet_idx, "row_in_sheet": self._row_in_sheet}

    def load_io_state(self, state):
        self._sheet_idx, self._row_in_sheet = int(state["sheet_idx"]), int(state["row_in_sheet"])


class _WindowMixin:
    """``next_window()`` protocol shared by the windowed datasets: returns True for an empty window (skip it), False when the
    window has data; raises StopIteration when there is no further window."""

    def _probe(self) -> bool:
        it = iter(self)
        try:
            first = next(it)
        except StopIteration:
            return True
        self._pending = (first, it)          # the batch read to find out is the window's first batch, not a lost one
        return False

    def _window_iter(self, fresh_iter):
        pending, self._pending = getattr(self, "_pending", None), None
        if pending is not None:
            first, it = pending
            yield first
            yield from it
        else:
            yield from fresh_iter()

    def state_dict(self):
        return {"read_offset": self._read_offset}

    def load_state_dict(self, state_dict):
        self._read_offset = state_dict["read_offset"].clone()


def make_odps_window_io(split_num: Optional[int] = None, row_num: Optional[int] = None):
    """A dataset class that consumes its tables window by window. Exactly one of ``split_num`` (every table is cut into that
    many windows) and ``row_num`` (a window is about ``row_num`` rows per worker) is given."""
    if not ((split_num is None) ^ (row_num is None)):
        raise ValueError("only one of split num and row num should be set!")

    class _OdpsWindowDataset(_WindowMixin, OdpsDataset):
        _split_num, _total_row_num = split_num, row_num

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            self._path_proportion: List[Tuple[int, int]] = []
            self._window_paths: List[TableSheet] = []
            self._read_offset = torch.zeros(1, dtype=torch.int64)
            self._shard_sheets: List[TableSheet] = []
            self._window_threads = self.read_threads_num
            self._pending = None

        def add_path(self, odps_table: str, proportion: tuple = (1, 1)):
            if len(proportion) != 2:
                raise ValueError("porportion size must be 2")
            if not all(isinstance(v, int) for v in proportion):
                raise ValueError("element in proportion should be int")
            self._paths.append(odps_table)
            self._path_proportion.append(tuple(proportion))

        def _shard_window_paths(self):
            if not self._paths:
                raise RuntimeError("No paths are added to this dataset.")
            thread_nums, self._window_threads = _parse_proportion(self.read_threads_num, self._path_proportion)
            paths: List[TableSheet] = []
            splits = [[] for _ in range(self._split_num or 0)]
            for index, table in enumerate(self._paths):
                if self._split_num:
                    threads = thread_nums[index % len(thread_nums)]
                    sheets, _ = _shard_sheets_by_split_num(table, self.worker_idx, self.worker_num, threads, self._split_num, 0)
                    for i in range(self._split_num):
                        splits[i] += sheets[i * threads:(i + 1) * threads]
                    if index % len(thread_nums) == len(thread_nums) - 1:       # a full group of tables: emit its windows
                        for i in range(self._split_num):
                            paths += splits[i]
                            splits[i] = []
                else:
                    sheets, _ = _shard_sheets_by_row_num(table, self.worker_idx, self.worker_num, self._window_threads, self._total_row_num, 0)
                    paths += sheets
            self._window_paths = paths

        def _shard_path(self, sub_id: int = 0, sub_num: int = 1):
            self._shard_paths = _shard_table_by_subprocess(self._shard_sheets, sub_id, sub_num)

        def next_window(self) -> bool:
            if not self._window_paths:
                self._shard_window_paths()
            off = int(self._read_offset[0])
            if off >= len(self._window_paths):
                raise StopIteration("Finish IO")
            self._shard_sheets = self._window_paths[off:off + self._window_threads]
            self._read_offset = self._read_offset + self._window_threads
            # the sheets of a window are read side by side: a batch takes its share from each, which is what mixes tables in
            # their proportions (threads per table follow the proportions)
            self._stream_width = len(self._shard_sheets)
            self._shard_path()
            self._sheet_idx, self._row_in_sheet = 0, 0
            return self._probe()

        def __iter__(self):
            return self._window_iter(lambda: OdpsDataset.__iter__(self))

        def reset(self):
            self._window_paths, self._pending = [], None
            self._read_offset = torch.zeros(1, dtype=torch.int64)

    return _OdpsWindowDataset


def _sample_sheets(table: str, task_id: int, thread_num: int, row_num: int, seed: int = 0) -> List[TableSheet]:
    """``thread_num`` sheets covering ``row_num`` consecutive rows at an offset drawn from ``(seed, task_id)``."""
    size = get_table_size(table)
    row_num = min(row_num, size)
    begin = random.Random(seed * 1000003 + task_id).randint(0, size - row_num) if size > row_num else 0
    shards, _ = _build_shard(begin, row_num, thread_num)
    return [TableSheet(table, s, e) for s, e in shards]


def make_odps_sample_io(row_num: int = 500000, seed: int = 0):
    """A dataset class with one window: a random contiguous sample of ``row_num`` rows of every table (evaluation on a
    sample of a large table)."""
    base = make_odps_window_io(row_num=row_num)

    class _OdpsSampleDataset(base):
        def _shard_window_paths(self):
            if not self._paths:
                raise RuntimeError("No paths are added to this dataset.")
            self._window_threads = self.read_threads_num
            self._window_paths = []
            for table in self._paths:
                self._window_paths += _sample_sheets(table, self.worker_idx, self.read_threads_num, row_num, seed)

    return _OdpsSampleDataset


class LakeStreamDataset(OrcDataset):
    """Streams read by time range: ``add_path(path, begin, end)`` with times in microseconds since the epoch. The entries of a
    range are dealt round-robin to workers."""

    def __init__(self, *args, shuffle_seed: int = 0, **kwargs):
        super().__init__(*args, **kwargs)
        self._begins: List[int] = []
        self._ends: List[int] = []
        self._shuffle_seed = shuffle_seed
        self._ranges: Optional[List[Tuple[str, int, int]]] = None
        self._range_idx = 0

    def add_path(self, path: str, begin: int, end: int):
        self._paths.append(path)
        self._begins.append(int(begin))
        self._ends.append(int(end))

    def _shard_path(self, sub_id: int = 0, sub_num: int = 1):
        self._ranges = list(zip(self._paths, self._begins, self._ends))

    def _my_entries(self, src, name: str, begin: int, end: int):
        entries = [e for e in src.entries(name) if begin <= e[0] < end]
        if self.shuffle:
            random.Random(self._shuffle_seed * 1000003 + begin // US).shuffle(entries)
        return entries[self.worker_idx::self.worker_num]

    def _range_files(self, path: str, begin: int, end: int) -> List[str]:
        """The columnar files behind this worker's entries of a time range, in reading order; empty when the source is not one
        of files (the range is then read through the source)."""
        from .table_source import FileStreamSource, _columnar_files
        src, name = resolve_stream_source(path)
        if not isinstance(src, FileStreamSource):
            return []
        return [f for _ts, entry in self._my_entries(src, name, begin, end) for f in _columnar_files(entry)]

    def _native(self, paths):
        # a range is read as a whole: the position inside it is not part of this dataset's state
        self._file_idx, self._row_in_file = 0, 0
        return super()._native(paths)

    def _range_table(self, path: str, begin: int, end: int):
        """This worker's rows of one time range: its share of the range's entries when the source lists entries, else every
        ``worker_num``-th block of rows."""
        import pyarrow as pa
        src, name = resolve_stream_source(path)
        if hasattr(src, "entries") and hasattr(src, "read_entry"):
            mine = self._my_entries(src, name, begin, end)
            parts = [src.read_entry(entry, self._columns()) for _ts, entry in mine]
            parts = [p for p in parts if p is not None and p.num_rows]
            return pa.concat_tables(parts) if parts else None
        table = src.read_range(name, begin, end, self._columns())
        if table is None or self.worker_num == 1:
            return table
        each = int(math.ceil(table.num_rows / self.worker_num))
        return table.slice(self.worker_idx * each, each)

    def _columns(self):
        return list(self._varlen) + list(self._fixed)

    def __iter__(self):
        if self._ranges is None:
            self._shard_path()
        if self._range_idx >= len(self._ranges):
            self._range_idx = 0
        while self._range_idx < len(self._ranges):
            path, begin, end = self._ranges[self._range_idx]
            self._range_idx += 1
            reader = self._native(self._range_files(path, begin, end))
            if reader is not None:                 # this worker's entries are columnar files: the C++ reader serves them
                yield from self._drain_native(reader)
                continue
            table = self._range_table(path, begin, end)
            if table is not None and table.num_rows:
                yield from self._batches_of(table, 0)

    def dump_io_state(self):
        return {"range_idx": self._range_idx}

    def load_io_state(self, state):
        self._range_idx = int(state["range_idx"])


def _str_to_timestamp(s: str, format: str = "%Y%m%d%H%M%S") -> int:
    import datetime as dt
    return int(dt.datetime.strptime(s, format).replace(tzinfo=dt.timezone.utc).timestamp()) * US


def _ts_to_string(ts: int, format: str = "%Y%m%d%H%M%S") -> str:
    return us_to_stamp(ts, format)


def make_lake_stream_window_io(step_mins: int = 60, repeat_mins: Optional[int] = None):
    """A dataset class whose window is a time range of fixed length (set by ``add_path(path, start_time, interval_mins)``)
    that moves forward by ``step_mins`` per ``next_window()``; with ``repeat_mins`` the window is read in pieces of that
    length, in time order. The stream has no end: a window that holds no data yet reports empty."""
    if not isinstance(step_mins, int):
        raise ValueError("The step mins must be int")
    if repeat_mins is not None and not isinstance(repeat_mins, int):
        raise ValueError("the repeat_mins should be None or int")

    class _LakeStreamWindowIO(_WindowMixin, LakeStreamDataset):
        _step = step_mins * 60 * US
        _repeat = None if repeat_mins is None else repeat_mins * 60 * US

        def __init__(self, *args, epochs: int = 1, name: str = "stream", **kwargs):
            super().__init__(*args, **kwargs)
            self._read_offset = torch.zeros(1, dtype=torch.int64)
            self._interval = None
            self._epochs, self._name = epochs, name
            self._pending = None

        def add_path(self, lake_path: str, start_time: int, interval_mins: int):
            self.add_paths([(lake_path, start_time, interval_mins)])

        def add_paths(self, lake_configs, proportions=None):
            for lake_path, start_time, interval_min in lake_configs:
                LakeStreamDataset.add_path(self, lake_path, start_time, start_time + interval_min * 60 * US)

        def _shard_window_data(self):
            start = self._begins[0]
            if int(self._read_offset[0]) == 0:
                self._read_offset = torch.tensor([start], dtype=torch.int64)
            self._interval = self._ends[0] - start
            if self._interval <= 0:
                raise ValueError("interval should be greater than 0")
            if self._repeat is not None and self._interval % self._repeat != 0:
                raise ValueError("the interval should be an integer multiple of repeat_min")

        def next_window(self) -> bool:
            if self._interval is None:
                self._shard_window_data()
            start = int(self._read_offset[0])
            self._read_offset = self._read_offset + self._step
            piece = self._repeat or self._interval
            ranges = []
            for k in range(self._interval // piece):
                ranges += [(p, start + k * piece, start + (k + 1) * piece) for p in self._paths] * self._epochs
            self._ranges, self._range_idx = ranges, 0
            logger.info(f"Initialize IO[{self._name}] to: start[{_ts_to_string(start)}] end[{_ts_to_string(start + self._interval)}].")
            return self._probe()

        def _shard_path(self, sub_id: int = 0, sub_num: int = 1):
            if self._ranges is None:
                self._ranges = []

        def __iter__(self):
            return self._window_iter(lambda: LakeStreamDataset.__iter__(self))

    return _LakeStreamWindowIO
