"""Optimizers: row-wise sparse optimizers for dynamic tables, and dense Adam variants on one multi-tensor kernel."""
from . import adamw_tf as _tf
from . import dense_adam as _dense
from . import sparse_optim as _sparse

_EXPORTS = {
    _sparse: ("SparseOptimizer", "SparseAdam", "SparseAdamW", "SparseAdamWTF", "SparseAdagrad", "SparseSGD"),
    _dense: ("DenseAdam", "DenseAdamW"),
    _tf: ("AdamWTF",),
}
__all__ = []
for _mod, _names in _EXPORTS.items():
    for _n in _names:
        globals()[_n] = getattr(_mod, _n)
        __all__.append(_n)
