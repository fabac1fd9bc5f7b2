"""Import path of the reference (``recis/io/state_dataset.py``): the implementation lives in ``recis_b200.io.dataset``."""
from .dataset import StateDataset

__all__ = ["StateDataset"]
