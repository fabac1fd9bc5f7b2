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

# recis/optim/sparse_adam.py, sparse_adamw.py and sparse_adamw_tf.py of the reference are one module here (optim/sparse_optim.py);
# the old import paths resolve to it.
import sys as _sys
for _alias in ("sparse_adam", "sparse_adamw", "sparse_adamw_tf"):
    _sys.modules.setdefault(__name__ + "." + _alias, _sparse)
