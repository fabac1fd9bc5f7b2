"""Import path of the reference (``recis/io/filter_dataset.py``): the implementation lives in ``recis_b200.io.dataset``."""
from .dataset import FilterDataset

__all__ = ["FilterDataset"]
