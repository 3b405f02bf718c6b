"""Operator classes of the `tls_attn` surface that this package serves, under the reference's import paths
(tls_attn/ops/__init__.py): dense and sparse attention over a paged cache, the two indexer levels, and the
stores of K/V rows and of the key index.  Every class is a thin `torch.autograd`-free callable over the C ABI
(`loda_tls_*`); the host-offload (`KVO_*`) twins of the reference are not part of the decode path and are
not provided.
"""
from .mha import MHAInterface
from .mha_indexer_level1 import MHAIndexerLevel1Interface
from .mha_indexer_level2 import MHAIndexerLevel2Interface
from .mha_store_k_index import MHAStoreKIndexInterface
from .mha_store_kv import MHAStoreKVInterface
from .sparse_mha import SparseMHAInterface

__all__ = ["MHAInterface", "SparseMHAInterface", "MHAIndexerLevel1Interface", "MHAIndexerLevel2Interface",
           "MHAStoreKVInterface", "MHAStoreKIndexInterface"]
