"""Convert CSV files to ORC shards readable by ``OrcDataset`` (role of the reference's ``tools/csv_to_orc.py``).

    python -m recis_b200.io.csv_to_orc --input data.csv --output out_dir [--rows-per-shard 1000000] [--list-columns seq --list-sep '|']

Columns named in ``--list-columns`` hold ``sep``-separated integer lists and are written as ``list<int64>``.
"""
from __future__ import annotations

import argparse
import os


def convert(input_path: str, output_dir: str, rows_per_shard: int = 1_000_000, list_columns=(), list_sep: str = "|") -> int:
    import pyarrow as pa
    import pyarrow.csv as pacsv
    import pyarrow.orc as orc
    os.makedirs(output_dir, exist_ok=True)
    table = pacsv.read_csv(input_path)
    for name in list_columns:
        col = table.column(name).to_pylist()
        lists = [[int(x) for x in str(v).split(list_sep) if x != ""] if v is not None else [] for v in col]
        table = table.set_column(table.schema.get_field_index(name), name, pa.array(lists, type=pa.list_(pa.int64())))
    n_shards = 0
    for start in range(0, max(table.num_rows, 1), rows_per_shard):
        orc.write_table(table.slice(start, rows_per_shard), os.path.join(output_dir, f"part-{n_shards:05d}.orc"))
        n_shards += 1
    return n_shards


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--rows-per-shard", type=int, default=1_000_000)
    ap.add_argument("--list-columns", nargs="*", default=[])
    ap.add_argument("--list-sep", default="|")
    a = ap.parse_args()
    n = convert(a.input, a.output, a.rows_per_shard, a.list_columns, a.list_sep)
    print(f"wrote {n} shard(s) to {a.output}")


if __name__ == "__main__":
    main()
