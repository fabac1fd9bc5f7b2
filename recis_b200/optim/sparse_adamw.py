"""Import path of the reference (``recis/optim/sparse_adamw.py``): the implementation lives in ``recis_b200.optim.sparse_optim``."""
from .sparse_optim import SparseAdamW

__all__ = ["SparseAdamW"]
