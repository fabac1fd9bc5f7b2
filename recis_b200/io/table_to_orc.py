"""Export a table to ORC shards readable by ``OrcDataset`` (role of the reference's ``tools/odps_to_orc.py``).

    python -m recis_b200.io.table_to_orc --table <name> --output out_dir [--nfiles 8] [--partitions dt=20250101 ...]
        [--project P --access-id ID --access-key KEY --endpoint URL]

``--table`` is anything ``io/table_source.py`` resolves: columnar files (a file, a directory, a glob), ``scheme://name`` of a
registered source, or, with the four credentials, a table of the table service (``project.table``; each ``--partitions`` entry
is exported as ``table/partition``). Rows are cut into ``--nfiles`` consecutive shards (default: one per 1 M rows) that are
read and written by a pool of threads, shard by shard, so memory stays at a few chunks per thread.
"""
from __future__ import annotations

import argparse
import os
from concurrent.futures import ThreadPoolExecutor

from .table_source import OdpsTableSource, get_table_size, register_table_source, resolve_table_source
from .window_io import _build_shard

_CHUNK_ROWS = 1 << 18


def export_shard(table: str, start: int, end: int, path: str, columns=None) -> int:
    """Rows ``[start, end)`` of ``table`` into one ORC file; returns the rows written."""
    import pyarrow as pa
    import pyarrow.orc as orc
    src, name = resolve_table_source(table)
    tmp = path + ".tmp"
    rows, writer = 0, None
    try:
        for lo in range(start, end, _CHUNK_ROWS):
            part = src.read(name, lo, min(lo + _CHUNK_ROWS, end), columns)
            if writer is None:
                writer = orc.ORCWriter(tmp)
            writer.write(part if isinstance(part, pa.Table) else pa.Table.from_batches([part]))
            rows += part.num_rows
    finally:
        if writer is not None:
            writer.close()
    if writer is not None:
        os.replace(tmp, path)
    return rows


def convert(table: str, output_dir: str, nfiles: int = 0, columns=None, threads: int = 4, prefix: str = "part") -> int:
    """Export ``table`` into ``output_dir/<prefix>-NNNNN.orc``; returns the number of files."""
    os.makedirs(output_dir, exist_ok=True)
    size = get_table_size(table)
    if size == 0:
        return 0
    nfiles = nfiles or max(1, (size + 999_999) // 1_000_000)
    shards, _ = _build_shard(0, size, min(nfiles, size))
    with ThreadPoolExecutor(max_workers=max(1, threads)) as pool:
        jobs = [pool.submit(export_shard, table, s, e, os.path.join(output_dir, f"{prefix}-{i:05d}.orc"), columns)
                for i, (s, e) in enumerate(shards)]
        written = sum(j.result() for j in jobs)
    assert written == size, f"exported {written} of {size} rows"
    return len(shards)


def main(argv=None):
    ap = argparse.ArgumentParser(description="Table to ORC file converter")
    ap.add_argument("--table", "-t", required=True)
    ap.add_argument("--nfiles", type=int, default=0, help="number of output shards (default: one per million rows)")
    ap.add_argument("--partitions", type=str, nargs="*", default=[])
    ap.add_argument("--output", "-o", required=True)
    ap.add_argument("--columns", type=str, nargs="*", default=None)
    ap.add_argument("--threads", type=int, default=4)
    ap.add_argument("--project")
    ap.add_argument("--access-id")
    ap.add_argument("--access-key")
    ap.add_argument("--endpoint")
    args = ap.parse_args(argv)
    table = args.table
    if args.access_id and args.access_key and args.endpoint:
        register_table_source("odps", OdpsTableSource(args.access_id, args.access_key, args.endpoint, args.project))
        if "://" not in table:
            table = "odps://" + (table if "." in table or not args.project else f"{args.project}.{table}")
    targets = [f"{table}/{p}" for p in args.partitions] or [table]
    total = 0
    for k, t in enumerate(targets):
        total += convert(t, args.output, args.nfiles, args.columns, args.threads, prefix=f"part{k}" if len(targets) > 1 else "part")
    print(f"wrote {total} files to {args.output}")


if __name__ == "__main__":
    main()
