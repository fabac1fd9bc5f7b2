"""Import path of the reference (``recis/io/orc_dataset.py``): the implementation lives in ``recis_b200.io.dataset``."""
from .dataset import OrcDataset, get_dir_size

__all__ = ["OrcDataset", "get_dir_size"]
