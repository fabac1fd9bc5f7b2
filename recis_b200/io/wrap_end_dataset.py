"""Import path of the reference (``recis/io/wrap_end_dataset.py``): the implementation lives in ``recis_b200.io.dataset``."""
from .dataset import WrapEndDataset

__all__ = ["WrapEndDataset"]
