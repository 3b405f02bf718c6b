from .mha import MHAInterface
from .mha_indexer_level1 import MHAIndexerLevel1Interface
from .mha_indexer_level2 import MHAIndexerLevel2Interface
from .mha_store_k_index import MHAStoreKIndexInterface
from .mha_store_kv import MHAStoreKVInterface
from .sparse_mha import SparseMHAInterface

__all__ = ["MHAInterface", "SparseMHAInterface", "MHAIndexerLevel1Interface", "MHAIndexerLevel2Interface",
           "MHAStoreKVInterface", "MHAStoreKIndexInterface"]
