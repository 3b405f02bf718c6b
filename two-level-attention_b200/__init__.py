"""loda_b200: the decode hot path of LoDA-SA / NFA two-level sparse attention
as hand-written sm_100a CUDA kernels behind the reference's Python operator
surface (sparse_attn.indexer / sparse_attn.ops / sparse_attn.cache).

The directory name is not a Python identifier; import it with
``importlib.import_module("two-level-attention_b200")``.
"""
from ._capi import FallbackRequired, lib  # noqa: F401

__all__ = ["FallbackRequired", "lib"]
