from .mha import MHAInterface
from .sparse_mha import SparseMHAInterface

__all__ = ["MHAInterface", "SparseMHAInterface"]
