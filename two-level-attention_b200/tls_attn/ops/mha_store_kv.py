"""Write keys and values into the contiguous caches.

Mirrors MHAStoreKVInterface (reference: tls_attn/ops/mha_store_kv.py:98-141; PyTorch
statement ``MHAStoreKVReference`` :144-199): prefill copies k / v [B, S, Hkv, D] from
``offsets[b]`` on to the start of cache row b; decode writes k / v [B, 1, Hkv, D] at
``lengths[b] - 1``.
"""
from __future__ import annotations

from ... import _capi
from . import _checks


class MHAStoreKVInterface:
    def __init__(self, max_batch: int, max_seqlen: int, num_kv_heads: int, dim_k: int, dim_v: int) -> None:
        self.max_batch, self.max_seqlen = max_batch, max_seqlen
        self.num_kv_heads, self.dim_k, self.dim_v = num_kv_heads, dim_k, dim_v

    def _check(self, k, v, k_cache, v_cache, seqlen):
        _checks.need_bf16_cuda(k=k, v=v, k_cache=k_cache, v_cache=v_cache)
        b = k.shape[0]
        if tuple(k.shape) != (b, seqlen, self.num_kv_heads, self.dim_k) or \
                tuple(v.shape) != (b, seqlen, self.num_kv_heads, self.dim_v):
            raise ValueError("k / v must be [B, S, Hkv, D]")
        if tuple(k_cache.shape[1:]) != (self.max_seqlen, self.num_kv_heads, self.dim_k) or \
                tuple(v_cache.shape[1:]) != (self.max_seqlen, self.num_kv_heads, self.dim_v) or k_cache.shape[0] < b:
            raise ValueError("caches must be [max_batch, max_seqlen, Hkv, D] with max_batch >= B")
        return b

    def prefill_forward(self, k, v, offsets, k_cache, v_cache):
        b = self._check(k, v, k_cache, v_cache, k.shape[1])
        _checks.need_i32("offsets", offsets)
        _capi.check(_capi.lib().loda_tls_store_kv(
            _capi.ptr(k), _capi.ptr(v), _capi.ptr(offsets), _capi.ptr(k_cache), _capi.ptr(v_cache), b, k.shape[1],
            self.max_seqlen, self.num_kv_heads, self.dim_k, self.dim_v, 0, _capi.current_stream()))

    def decode_forward(self, k, v, lengths, k_cache, v_cache):
        b = self._check(k, v, k_cache, v_cache, 1)
        _checks.need_i32("lengths", lengths)
        _capi.check(_capi.lib().loda_tls_store_kv(
            _capi.ptr(k), _capi.ptr(v), _capi.ptr(lengths), _capi.ptr(k_cache), _capi.ptr(v_cache), b, 1,
            self.max_seqlen, self.num_kv_heads, self.dim_k, self.dim_v, 1, _capi.current_stream()))
