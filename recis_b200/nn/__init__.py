"""Dynamic embedding layer: tables, sharded embeddings, the merging engine and their admission / eviction descriptors."""
from .modules import embedding as _emb
from .modules import embedding_engine as _eng
from .modules import hashtable as _ht
from . import hashtable_hook as _hooks

_EXPORTS = {
    _ht: ("HashTable", "gen_slice", "filter_out_sparse_param", "split_sparse_dense_state_dict"),
    _emb: ("DynamicEmbedding", "EmbeddingOption"),
    _eng: ("EmbeddingEngine",),
    _hooks: ("AdmitHook", "FilterHook"),
}
__all__ = []
for _mod, _names in _EXPORTS.items():
    for _n in _names:
        globals()[_n] = getattr(_mod, _n)
        __all__.append(_n)
