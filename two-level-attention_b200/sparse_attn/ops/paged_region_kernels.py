"""Paged KV write and sparse gather attention over a layer arena.

Mirrors paged_write_prefill / paged_write_decode / sparse_paged_attention_gather
(reference: sparse_attn/ops/paged_region_kernels.py:610-724, 800-1041): same
argument meaning, same ValueError conditions; the work is done by the CUDA
library through its C ABI and there is no CPU branch.
"""
from __future__ import annotations

import ctypes as C

import torch

from ... import _capi


def _layer_runtime(cache_layer, *, n_rows, n_query, max_visible, num_q_heads):
    """Geometry / scratch for calls that only know a layer arena (no selector)."""
    store = cache_layer.__dict__.setdefault("_loda_layer_runtime", {})
    key = (n_rows, n_query, max_visible, num_q_heads)
    rt = store.get(key)
    if rt is not None:
        return rt
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("warm this shape up once before CUDA graph capture")
    if cache_layer.dtype != torch.bfloat16:
        raise _capi.FallbackRequired("only bf16 KV pools are implemented")
    page = cache_layer.geometry.page
    g = _capi.Geometry(
        dtype=_capi.LODA_DTYPE_BF16, num_q_heads=num_q_heads, num_kv_heads=cache_layer.num_kv_heads,
        head_dim=cache_layer.head_dim_k, head_dim_v=cache_layer.head_dim_v, sub_dims=32, sub_lo0=0,
        sub_lo1=16, page=page, num_pages=cache_layer.max_physical_pages + 1, max_blocks=16384,
        max_requests=max(n_rows, 1), max_query_tokens=max(n_query, 1), max_visible=max(max_visible, page),
        k_far=0, k_near=0, level2_topk=max(max_visible, page), sink=0, swa=page, near_len=page,
        pool_near_len=page)
    nbytes = _capi.lib().loda_workspace_bytes(C.byref(g))
    if nbytes == 0:
        raise _capi.FallbackRequired(_capi.lib().loda_last_error().decode())
    dev = cache_layer.kv_pool_k.device
    rt = {
        "geometry": g,
        "workspace": torch.zeros(nbytes, dtype=torch.uint8, device=dev),
        "neg_ids": torch.full((max(n_query, 1),), -1, dtype=torch.int64, device=dev),
        "layer": _capi.Layer(pool_k=cache_layer.kv_pool_k.data_ptr(), pool_v=cache_layer.kv_pool_v.data_ptr()),
    }
    store[key] = rt
    return rt


def paged_write_prefill(cache_layer, key_states, value_states, block_table, *, workspace=None):
    """key_states / value_states [1, HK, N, D]; block_table is the request's
    logical -> physical row on the same device."""
    if key_states.ndim != 4 or key_states.shape[0] != 1 or key_states.shape[2] < 1:
        raise ValueError("paged write prefill expects [1,HK,N,D] keys")
    if value_states.ndim != 4 or value_states.shape[:3] != key_states.shape[:3]:
        raise ValueError("paged write prefill expects [1,HK,N,DV] values")
    if key_states.shape[1] != cache_layer.num_kv_heads:
        raise ValueError("KV head count does not match arena")
    if key_states.shape[-1] != cache_layer.head_dim_k:
        raise ValueError("key head dimension does not match arena")
    if value_states.shape[-1] != cache_layer.head_dim_v:
        raise ValueError("value head dimension does not match arena")
    if block_table.ndim != 1 or block_table.device != key_states.device:
        raise ValueError("prefill block table must be a device-matched 1D row")
    n = key_states.shape[2]
    if n > block_table.numel() * cache_layer.geometry.page:
        raise ValueError("prefill length exceeds block-table capacity")
    if not key_states.is_cuda:
        raise RuntimeError("paged write prefill needs CUDA tensors (no CPU path in this package)")
    rt = _layer_runtime(cache_layer, n_rows=1, n_query=1, max_visible=0,
                        num_q_heads=cache_layer.num_query_heads)
    k = key_states.to(cache_layer.dtype).contiguous()
    v = value_states.to(cache_layer.dtype).contiguous()
    table = block_table.to(torch.int32).contiguous()
    _capi.check(_capi.lib().loda_write_prefill(
        C.byref(rt["geometry"]), C.byref(rt["layer"]), _capi.ptr(k), _capi.ptr(v), _capi.ptr(table),
        n, _capi.current_stream()))
    return key_states, value_states


def paged_write_decode(cache_layer, key_states, value_states, slot_mapping, *, workspace=None):
    """key_states / value_states [B, HK, 1, D]; slot_mapping [B] int32, -1 rows
    go to the PAD page.  Writes K/V only; the selector index of the new token is
    refreshed by the selector call that follows."""
    if key_states.ndim != 4 or key_states.shape[-2] != 1:
        raise ValueError("paged write decode expects [B,HK,1,D] keys")
    if value_states.ndim != 4 or value_states.shape[-2] != 1:
        raise ValueError("paged write decode expects [B,HK,1,DV] values")
    if key_states.shape[0] != slot_mapping.shape[0]:
        raise ValueError("slot mapping batch must match KV batch")
    if key_states.shape[1] != cache_layer.num_kv_heads:
        raise ValueError("KV head count does not match arena")
    if not key_states.is_cuda:
        raise RuntimeError("paged write decode needs CUDA tensors (no CPU path in this package)")
    b = key_states.shape[0]
    rt = _layer_runtime(cache_layer, n_rows=b, n_query=b, max_visible=0,
                        num_q_heads=cache_layer.num_query_heads)
    k = key_states.to(cache_layer.dtype).contiguous()
    v = value_states.to(cache_layer.dtype).contiguous()
    slots = slot_mapping.to(device=k.device, dtype=torch.int32).contiguous()
    neg = rt["neg_ids"]
    batch = _capi.Batch(batch=b, lengths=neg.data_ptr(), valid_req_ids=neg.data_ptr(),
                        active_req_ids=neg.data_ptr())
    _capi.check(_capi.lib().loda_append_decode(
        C.byref(rt["geometry"]), C.byref(rt["layer"]), C.byref(batch), _capi.ptr(k), _capi.ptr(v),
        _capi.ptr(slots), None, _capi.current_stream()))
    return key_states, value_states


def sparse_paged_attention_gather(cache_layer, q, gather_indices, visible_lens, query_to_req, *,
                                  scale, workspace=None, split_kv=False, return_lse=False):
    """q [T, HQ, D]; gather_indices [B, HK, K] absolute physical slots
    (page * PAGE + offset) in ascending logical order; visible_lens [B, HK];
    query_to_req [T] maps a query row to its row of the gather list (< 0: the
    output row is zero).  Returns [T, HQ, DV] in q's dtype.  The list is always
    processed split-K with a deterministic merge; ``split_kv`` is accepted for
    signature compatibility.  ``return_lse=True`` also returns [T, HQ, 2] fp32
    (row maximum in the exp2 domain, softmax sum) for merging partial attentions
    over disjoint token sets (``sharding.lse_merge``)."""
    if q.ndim != 3 or q.shape[-1] != cache_layer.head_dim_k:
        raise ValueError("sparse gather attention expects flat [T,HQ,D] query")
    hq, hk = q.shape[1], cache_layer.num_kv_heads
    if hq % hk != 0:
        raise ValueError("GQA requires HQ % HK == 0")
    if (gather_indices.ndim != 3 or gather_indices.shape[1] != hk
            or visible_lens.shape != gather_indices.shape[:2]):
        raise ValueError("gather attention expects indices [B,HK,K] and lens [B,HK]")
    page = cache_layer.geometry.page
    if page & (page - 1):
        raise ValueError("sparse gather attention requires power-of-two page size")
    if not q.is_cuda:
        raise RuntimeError("sparse gather attention needs CUDA tensors (no CPU path in this package)")
    if q.dtype != cache_layer.dtype:
        raise ValueError("query dtype must match the KV pool dtype")
    total_q = q.shape[0]
    rt = _layer_runtime(cache_layer, n_rows=gather_indices.shape[0], n_query=total_q,
                        max_visible=gather_indices.shape[-1], num_q_heads=hq)
    g = rt["geometry"]
    if g.max_visible != gather_indices.shape[-1]:
        raise ValueError("gather list narrower than one page")
    out = q.new_empty((total_q, hq, cache_layer.head_dim_v))
    qc = q.contiguous()
    gi = gather_indices if gather_indices.is_contiguous() else gather_indices.contiguous()
    vl = visible_lens if visible_lens.is_contiguous() else visible_lens.contiguous()
    q2r = query_to_req[:total_q].to(torch.int32).contiguous()
    lse = torch.empty((total_q, hq, 2), dtype=torch.float32, device=q.device) if return_lse else None
    _capi.check(_capi.lib().loda_gather_attend_lse(
        C.byref(g), C.byref(rt["layer"]), _capi.ptr(qc), _capi.ptr(gi), _capi.ptr(vl), _capi.ptr(q2r),
        total_q, gather_indices.shape[0], float(scale), _capi.ptr(out), _capi.ptr(lse),
        _capi.ptr(rt["workspace"]), _capi.current_stream()))
    return (out, lse) if return_lse else out


def sparse_paged_attention_gather_partial(cache_layer, q, gather_indices, visible_lens, query_to_req, *,
                                          scale, workspace=None, name="", nsplit=1):
    """Attention over one region's token list as a partial state that can be merged with
    another region's (reference: sparse_attn/ops/paged_region_kernels.py:727-780).  Returns
    (acc [1, T, HQ, DV] fp32, m [1, T, HQ], z [1, T, HQ]): the partial output normalised by its own
    sum, the row maximum (exp2 domain) and the sum.  `nsplit` and `name` are accepted for signature
    compatibility: the kernel chooses its own split and merges it inside the launch."""
    out, lse = sparse_paged_attention_gather(cache_layer, q, gather_indices, visible_lens, query_to_req,
                                             scale=scale, workspace=workspace, return_lse=True)
    return out.float()[None], lse[None, ..., 0], lse[None, ..., 1]


def sparse_paged_attention_regions_combine(q, protected_parts, middle_parts, *, workspace=None):
    """Fixed-order log-sum-exp merge of the protected and the middle partial attentions
    (reference: sparse_attn/ops/paged_region_kernels.py:783-797); [T, HQ, DV] in q's dtype."""
    from ...sharding import lse_merge
    acc = torch.cat((protected_parts[0], middle_parts[0]))
    m = torch.cat((protected_parts[1], middle_parts[1]))
    z = torch.cat((protected_parts[2], middle_parts[2]))
    return lse_merge(acc, m, z).to(q.dtype)
