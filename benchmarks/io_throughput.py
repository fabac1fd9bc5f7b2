"""Host-side reader throughput: rows per second of the file, table and window datasets, native reader against the Python path.

    python benchmarks/io_throughput.py [--rows 400000] [--files 4] [--batch 8192] [--threads 4]

Writes ``--files`` columnar files (half ORC, half Parquet) of ``--rows / --files`` rows with eight id-list columns (lengths
1..9), one string column that is hashed at read time, and four numeric columns into a temporary directory, then reads them back
once per configuration and prints one JSON line each. No GPU is involved; the numbers are those of the host it runs on.
"""
import argparse
import json
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np
import pyarrow as pa
import pyarrow.orc as orc
import pyarrow.parquet as pq

from recis_b200.io import OdpsDataset, OrcDataset, make_odps_window_io

VAR = [f"ids{i}" for i in range(8)]
FIX = [f"x{i}" for i in range(4)]


def write_files(root, rows, files, seed=0):
    rng = np.random.default_rng(seed)
    per = rows // files
    paths = []
    for f in range(files):
        cols = {}
        for name in VAR:
            lens = rng.integers(1, 10, per)
            offsets = np.zeros(per + 1, dtype=np.int32)
            np.cumsum(lens, out=offsets[1:])
            cols[name] = pa.ListArray.from_arrays(pa.array(offsets), pa.array(rng.integers(0, 1 << 40, int(offsets[-1]))))
        cols["city"] = pa.array([f"city_{v}" for v in rng.integers(0, 5000, per)])
        for name in FIX:
            cols[name] = pa.array(rng.random(per))
        table = pa.table(cols)
        path = os.path.join(root, f"part-{f:03d}." + ("orc" if f % 2 == 0 else "parquet"))
        orc.write_table(table, path) if f % 2 == 0 else pq.write_table(table, path, row_group_size=50_000)
        paths.append(path)
    return paths


def declare(ds):
    for name in VAR:
        ds.varlen_feature(name)
    ds.varlen_feature("city", hash_type="farm", hash_bucket=100_000)
    for name in FIX:
        ds.fixedlen_feature(name)
    return ds


def drain(make):
    t0 = time.perf_counter()
    rows = 0
    ds = make()
    if hasattr(ds, "next_window"):
        while True:
            try:
                if ds.next_window():
                    continue
            except StopIteration:
                break
            for b in ds:
                rows += b["x0"].shape[0]
    else:
        for b in ds:
            rows += b["x0"].shape[0]
    return rows, time.perf_counter() - t0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=400_000)
    ap.add_argument("--files", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--threads", type=int, default=4)
    args = ap.parse_args()
    with tempfile.TemporaryDirectory(prefix="rb_io_bench_") as root:
        paths = write_files(root, args.rows, args.files)

        def files(native):
            ds = OrcDataset(args.batch, read_threads_num=args.threads, prefetch=4, native_reader=native)
            ds.add_paths(paths)
            return declare(ds)

        def table(native):
            ds = OdpsDataset(args.batch, read_threads_num=args.threads, prefetch=4, native_reader=native)
            ds.add_path(root)
            return declare(ds)

        def windows(native):
            ds = make_odps_window_io(split_num=4)(args.batch, read_threads_num=args.threads, prefetch=4, native_reader=native)
            ds.add_path(root, (1, 1))
            return declare(ds)

        for name, make in (("files (OrcDataset)", files), ("table by row range (OdpsDataset)", table), ("windows (make_odps_window_io)", windows)):
            for native in (True, False):
                rows, sec = drain(lambda: make(native))
                print(json.dumps({"dataset": name, "reader": "native" if native else "python", "rows": rows, "seconds": round(sec, 3),
                                  "rows_per_s": round(rows / sec), "batch": args.batch, "threads": args.threads}), flush=True)


if __name__ == "__main__":
    main()
