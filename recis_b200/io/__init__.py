from .dataset import (DatasetBase, FilterDataset, MapDataset, OrcDataset, PrefetchDataset, StateDataset, SyntheticDataset, TensorDataset,
                      WrapEndDataset)
from .prefetch import DevicePrefetcher, PackedBatch
from .table_source import (FileStreamSource, FileTableSource, OdpsTableSource, get_table_size, register_stream_source,
                           register_table_source)
from .window_io import (LakeStreamDataset, OdpsDataset, TableSheet, make_lake_stream_window_io, make_odps_sample_io,
                        make_odps_window_io)
from .synthetic import SparseFieldSpec, SyntheticSpec, make_batch, make_batch_arrays, to_device

__all__ = ["DatasetBase", "OrcDataset", "SyntheticDataset", "TensorDataset", "MapDataset", "FilterDataset", "PrefetchDataset",
           "StateDataset", "WrapEndDataset", "SyntheticSpec", "SparseFieldSpec", "make_batch", "make_batch_arrays", "to_device", "DevicePrefetcher", "PackedBatch",
           "OdpsDataset", "LakeStreamDataset", "make_odps_window_io", "make_odps_sample_io", "make_lake_stream_window_io", "TableSheet",
           "FileTableSource", "FileStreamSource", "OdpsTableSource", "register_table_source", "register_stream_source", "get_table_size"]

# The reference keeps each dataset class in a module of its own (recis/io/orc_dataset.py, dataset_base.py, state_dataset.py,
# map_dataset.py, wrap_end_dataset.py, filter_dataset.py); here they share io/dataset.py. The old import paths resolve to it, so
# `from recis_b200.io.orc_dataset import OrcDataset` works with only the package name changed.
import sys as _sys
from . import dataset as _dataset
for _alias in ("orc_dataset", "dataset_base", "state_dataset", "map_dataset", "wrap_end_dataset", "filter_dataset"):
    _sys.modules.setdefault(__name__ + "." + _alias, _dataset)
# likewise the table and stream datasets (recis/io/odps_dataset.py, lake_dataset.py) live in io/window_io.py
from . import window_io as _window_io
for _alias in ("odps_dataset", "lake_dataset"):
    _sys.modules.setdefault(__name__ + "." + _alias, _window_io)
