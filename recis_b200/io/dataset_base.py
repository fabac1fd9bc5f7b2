"""Import path of the reference (``recis/io/dataset_base.py``): the implementation lives in ``recis_b200.io.dataset``."""
from .dataset import DatasetBase

__all__ = ["DatasetBase"]
