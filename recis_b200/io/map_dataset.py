"""Import path of the reference (``recis/io/map_dataset.py``): the implementation lives in ``recis_b200.io.dataset``."""
from .dataset import MapDataset

__all__ = ["MapDataset"]
