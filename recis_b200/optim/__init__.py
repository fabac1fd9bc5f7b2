from .adamw_tf import AdamWTF
from .sparse_optim import SparseAdagrad, SparseAdam, SparseAdamW, SparseAdamWTF, SparseOptimizer, SparseSGD

__all__ = ["AdamWTF", "SparseAdam", "SparseAdamW", "SparseAdamWTF", "SparseAdagrad", "SparseSGD", "SparseOptimizer"]
