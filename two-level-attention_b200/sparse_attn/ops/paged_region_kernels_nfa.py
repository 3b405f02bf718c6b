"""Decode glue: canonical arguments and the gather-attention entry
(reference: sparse_attn/ops/paged_region_kernels_nfa.py:10-20, 122-162)."""
from __future__ import annotations

from types import SimpleNamespace

INVALID_GATHER_IDX = -1


def nfa_args(subspace="tail", **overrides):
    """Production selector settings (the values of the reference's ``nfa_args``)."""
    ns = SimpleNamespace(
        method="nfa", nfa_far_method="minmax", nfa_near_method="avg", nfa_near_pages=32,
        nfa_near_tokens="off", nfa_near_len=4096, nfa_subspace=subspace, nfa_l2_subspace="same",
        nfa_enable_subspace=True, tia_level2_cmp_ratio=4, nfa_sink_tokens=4, nfa_swa_size=128,
        tia_level1_topk=128, tia_level2_topk=1024, tia_block_size=64, nfa_l2_quant=True,
        nfa_enable_layer_skip=False)
    for key, value in overrides.items():
        if not hasattr(ns, key) and key != "head_dim":
            raise ValueError(f"unknown selector argument {key}")
        setattr(ns, key, value)
    return ns


def decode_graph_ready(module, q, cache, *, gather_indices=None, visible_lens=None,
                       query_to_req=None, scale=None):
    """Sparse gather attention over the slots the selector wrote for
    ``module.layer_idx``.  ``q`` is [T, HQ, D] or [B, 1, HQ, D] / [B, HQ, 1, D]."""
    from .paged_region_kernels import sparse_paged_attention_gather

    layer_idx = module.layer_idx
    layer = cache.layers[layer_idx]
    scale = module.scaling if scale is None else scale
    if q.ndim == 4:
        if q.shape[2] == 1 and q.shape[1] != 1:
            q = q[:, :, 0].contiguous()
        elif q.shape[1] == 1:
            q = q[:, 0].contiguous()
        else:
            raise ValueError("graph-ready decode expects one query per row")
    if q.ndim != 3:
        raise ValueError("graph-ready decode expects [T,HQ,D] query")
    gather_indices = cache.gather_indices_buf[layer_idx] if gather_indices is None else gather_indices
    visible_lens = cache.visible_lens_buf[layer_idx] if visible_lens is None else visible_lens
    query_to_req = cache.query_to_req_buf if query_to_req is None else query_to_req
    return sparse_paged_attention_gather(
        layer, q, gather_indices, visible_lens, query_to_req, scale=scale,
        workspace=cache.selector_workspace())


def split_gather_buffers(cache, layer_idx, batch):
    """Fixed-address (protected gather, protected lens, middle gather, middle lens) buffers of one
    layer for the disjoint protected / middle operator mode
    (reference: sparse_attn/ops/paged_region_kernels_nfa.py:60-81)."""
    import torch
    store = cache.__dict__.setdefault("_split_gather_buffers", {})
    key = (layer_idx, batch)
    buffers = store.get(key)
    if buffers is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("split gather buffers must be warmed before capture")
        shape = (batch, cache.num_kv_heads, cache.max_visible_len)
        buffers = (torch.full((2,) + shape, -1, dtype=torch.int32, device=cache.device),
                   torch.zeros((2, batch, cache.num_kv_heads), dtype=torch.int32, device=cache.device))
        store[key] = buffers
    return buffers[0][0], buffers[1][0], buffers[0][1], buffers[1][1]


def build_protected_gather(cache, layer_idx, indexer, gather_out, vis_out):
    """sink ++ sliding window of every planned request row as physical slots into
    (gather_out [B, Hkv, max_visible], vis_out [B, Hkv])
    (reference: sparse_attn/ops/paged_region_kernels_nfa.py:84-119)."""
    import ctypes as C

    from ... import _capi
    rt = cache.ensure_index(indexer)
    batch = gather_out.shape[0]
    if tuple(gather_out.shape[1:]) != (cache.num_kv_heads, cache.max_visible_len) or tuple(vis_out.shape) != (
            batch, cache.num_kv_heads):
        raise ValueError("protected gather buffers must be [B, Hkv, max_visible] and [B, Hkv]")
    _capi.check(_capi.lib().loda_protected_gather(
        C.byref(rt.geometry), C.byref(rt.layer_structs[layer_idx]), C.byref(rt.batch_struct(batch)),
        _capi.ptr(gather_out), _capi.ptr(vis_out), C.c_void_p(cache.status_buf.data_ptr()), _capi.current_stream()))
