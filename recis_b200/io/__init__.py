from .dataset import (DatasetBase, FilterDataset, MapDataset, OrcDataset, PrefetchDataset, StateDataset, SyntheticDataset, TensorDataset,
                      WrapEndDataset)
from .prefetch import DevicePrefetcher, PackedBatch
from .synthetic import SparseFieldSpec, SyntheticSpec, make_batch, make_batch_arrays, to_device

__all__ = ["DatasetBase", "OrcDataset", "SyntheticDataset", "TensorDataset", "MapDataset", "FilterDataset", "PrefetchDataset",
           "StateDataset", "WrapEndDataset", "SyntheticSpec", "SparseFieldSpec", "make_batch", "make_batch_arrays", "to_device", "DevicePrefetcher", "PackedBatch"]
