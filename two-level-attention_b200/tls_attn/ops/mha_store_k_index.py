"""Build the two index levels of the keys: per-block min / max and per-token tail sub-dimensions.

Mirrors MHAStoreKIndexInterface (reference: tls_attn/ops/mha_store_k_index.py:139-185; PyTorch
statement ``MHAStoreKIndexReference`` :188-308).  level1 caches are
[max_batch, max_seqlen / block, Hkv, D], the level2 cache is [max_batch, max_seqlen, Hkv, D / cmp_ratio].
"""
from __future__ import annotations

from ... import _capi
from . import _checks


class MHAStoreKIndexInterface:
    def __init__(self, max_batch: int, max_seqlen: int, num_kv_heads: int, dim_k: int, sfa_block_size: int,
                 sfa_cmp_ratio: int) -> None:
        if dim_k % 2 or (dim_k // 2) % sfa_cmp_ratio:
            raise ValueError("dim_k / 2 must be a multiple of sfa_cmp_ratio")
        self.max_batch, self.max_seqlen = max_batch, max_seqlen
        self.num_kv_heads, self.dim_k = num_kv_heads, dim_k
        self.block, self.cmp = sfa_block_size, sfa_cmp_ratio
        self.l1_len = max_seqlen // sfa_block_size
        self.cmp_dim_k = 2 * (dim_k // 2 // sfa_cmp_ratio)

    def _check_caches(self, l1_min, l1_max, l2_k, batch):
        _checks.need_bf16_cuda(level1_k_min_cache=l1_min, level1_k_max_cache=l1_max, level2_k_cache=l2_k)
        if tuple(l1_min.shape[1:]) != (self.l1_len, self.num_kv_heads, self.dim_k) or l1_min.shape != l1_max.shape:
            raise ValueError("level1 caches must be [max_batch, max_seqlen / block, Hkv, dim_k]")
        if tuple(l2_k.shape[1:]) != (self.max_seqlen, self.num_kv_heads, self.cmp_dim_k):
            raise ValueError("level2 cache must be [max_batch, max_seqlen, Hkv, dim_k / cmp_ratio]")
        if min(l1_min.shape[0], l2_k.shape[0]) < batch:
            raise ValueError("caches hold fewer rows than the batch")

    def prefill_forward(self, k, offsets, level1_k_min_cache, level1_k_max_cache, level2_k_cache):
        _checks.need_bf16_cuda(k=k)
        _checks.need_i32("offsets", offsets)
        b, s = k.shape[0], k.shape[1]
        if tuple(k.shape[2:]) != (self.num_kv_heads, self.dim_k):
            raise ValueError("k must be [B, S, Hkv, dim_k]")
        self._check_caches(level1_k_min_cache, level1_k_max_cache, level2_k_cache, b)
        _capi.check(_capi.lib().loda_tls_store_k_index(
            _capi.ptr(k), _capi.ptr(offsets), _capi.ptr(level1_k_min_cache), _capi.ptr(level1_k_max_cache),
            _capi.ptr(level2_k_cache), b, s, self.num_kv_heads, self.dim_k, self.block, self.cmp, self.l1_len,
            self.max_seqlen, 0, _capi.current_stream()))

    def decode_forward(self, k_cache, lengths, level1_k_min_cache, level1_k_max_cache, level2_k_cache):
        _checks.need_bf16_cuda(k_cache=k_cache)
        _checks.need_i32("lengths", lengths)
        b = lengths.shape[0]
        if tuple(k_cache.shape[1:]) != (self.max_seqlen, self.num_kv_heads, self.dim_k) or k_cache.shape[0] < b:
            raise ValueError("k_cache must be [max_batch, max_seqlen, Hkv, dim_k]")
        self._check_caches(level1_k_min_cache, level1_k_max_cache, level2_k_cache, b)
        _capi.check(_capi.lib().loda_tls_store_k_index(
            _capi.ptr(k_cache), _capi.ptr(lengths), _capi.ptr(level1_k_min_cache), _capi.ptr(level1_k_max_cache),
            _capi.ptr(level2_k_cache), b, self.max_seqlen, self.num_kv_heads, self.dim_k, self.block, self.cmp,
            self.l1_len, self.max_seqlen, 1, _capi.current_stream()))
