from .hashtable_hook import AdmitHook, FilterHook
from .modules.embedding import DynamicEmbedding, EmbeddingOption
from .modules.embedding_engine import EmbeddingEngine
from .modules.hashtable import HashTable, filter_out_sparse_param, gen_slice, split_sparse_dense_state_dict

__all__ = ["HashTable", "DynamicEmbedding", "EmbeddingOption", "EmbeddingEngine", "AdmitHook", "FilterHook",
           "filter_out_sparse_param", "split_sparse_dense_state_dict", "gen_slice"]
