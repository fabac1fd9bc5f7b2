from .adamw_tf import AdamWTF
from .dense_adam import DenseAdam, DenseAdamW
from .sparse_optim import SparseAdagrad, SparseAdam, SparseAdamW, SparseAdamWTF, SparseOptimizer, SparseSGD

__all__ = ["AdamWTF", "DenseAdam", "DenseAdamW", "SparseAdam", "SparseAdamW", "SparseAdamWTF", "SparseAdagrad", "SparseSGD",
           "SparseOptimizer"]
