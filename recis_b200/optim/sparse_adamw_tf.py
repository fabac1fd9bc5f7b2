"""Import path of the reference (``recis/optim/sparse_adamw_tf.py``): the implementation lives in ``recis_b200.optim.sparse_optim``."""
from .sparse_optim import SparseAdamWTF

__all__ = ["SparseAdamWTF"]
