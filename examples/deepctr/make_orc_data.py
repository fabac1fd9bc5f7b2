"""Write a few ORC shards of synthetic click logs for ``examples/deepctr/run.py``.

Columns: ``label`` (float), ``dense1``/``dense2`` (float), ``sparse1``/``sparse2`` (int64 id), ``seq`` (list<int64>, variable
length), ``city`` (string). Same role as the reference's ``examples/deepctr/make_orc_data.py``.
"""
import argparse
import os

import numpy as np
import pyarrow as pa
import pyarrow.orc as orc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="/tmp/deepctr_data")
    ap.add_argument("--shards", type=int, default=4)
    ap.add_argument("--rows", type=int, default=4096)
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    rng = np.random.default_rng(0)
    cities = [f"city_{i}" for i in range(200)]
    for s in range(args.shards):
        n = args.rows
        lens = rng.integers(1, 40, n)
        seq = [rng.zipf(1.2, l).astype(np.int64) % 100_000 for l in lens]
        table = pa.table({
            "label": (rng.random(n) < 0.2).astype(np.float32),
            "dense1": rng.standard_normal(n).astype(np.float32),
            "dense2": rng.lognormal(0, 1, n).astype(np.float32),
            "sparse1": rng.integers(0, 1 << 40, n),
            "sparse2": rng.zipf(1.1, n).astype(np.int64),
            "seq": pa.array(seq, type=pa.list_(pa.int64())),
            "city": pa.array([cities[i] for i in rng.integers(0, len(cities), n)]),
        })
        orc.write_table(table, os.path.join(args.out, f"part-{s:05d}.orc"))
    print(f"wrote {args.shards} shards of {args.rows} rows to {args.out}")


if __name__ == "__main__":
    main()
