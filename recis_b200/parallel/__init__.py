"""Multi-GPU plumbing: symmetric peer-mapped heaps, the fused embedding exchange, the dense gradient reducer.

Sub-modules are imported lazily by their users (they need the native extension and, for the CUDA paths, a device); the two
classes a training script touches directly are re-exported here on first access."""


def __getattr__(name):
    if name == "DenseGradReducer":
        from .dense_reducer import DenseGradReducer
        return DenseGradReducer
    if name == "FusedExchange":
        from .fused_exchange import FusedExchange
        return FusedExchange
    raise AttributeError(name)
