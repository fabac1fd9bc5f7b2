"""Import path of the reference (``recis/optim/sparse_adam.py``): the implementation lives in ``recis_b200.optim.sparse_optim``."""
from .sparse_optim import SparseAdam

__all__ = ["SparseAdam"]
