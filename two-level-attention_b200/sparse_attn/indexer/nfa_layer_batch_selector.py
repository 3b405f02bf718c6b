"""Per-layer, request-batched two-level selection for the current query.

Mirrors select_topk_for_layer_batched (reference: sparse_attn/indexer/
nfa_layer_batch_selector.py:2649-2720, implementation :2723-3091): same
arguments, results written in place into ``cache.gather_indices_for_layer`` /
``cache.visible_lens_for_layer``, ValueError on contract violations and
FallbackRequired for configurations the CUDA path does not cover.  Two
launches replace the reference's eleven: fused L1 score + select (which also
carries the append / index refresh in extra CTAs) and fused L2 score + select
+ union.
"""
from __future__ import annotations

import ctypes as C

import torch

from ... import _capi
from ..._capi import FallbackRequired  # noqa: F401  (re-exported like the reference)
from .selection.selector import TokenSelection


def _ensure_index_built(cache, rt, layer_idx, req_ids, has_current_token_in_pool):
    """Host-side: requests whose index does not cover their tokens yet (fresh
    prefill) get a bulk build of the missing pages before the step."""
    page = cache.geometry.page
    for request_id in req_ids:
        if request_id is None or request_id < 0 or request_id not in cache.states:
            continue
        state = cache.states[request_id]
        planned = cache.pending_lengths.get(request_id, state.logical_length)
        have = planned if has_current_token_in_pool else planned - 1   # tokens already in the pool
        if state.index_len[layer_idx] >= have and state.index_live[layer_idx]:
            continue
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("selector index must be built (one eager step) before graph capture")
        first = state.index_len[layer_idx] // page
        n_blocks = (have + page - 1) // page - first
        if n_blocks > 0:
            _capi.check(_capi.lib().loda_build_index(
                C.byref(rt.geometry), C.byref(rt.layer_structs[layer_idx]), int(request_id), int(have),
                int(first), int(n_blocks), _capi.current_stream()))
        state.index_len[layer_idx] = have
        state.index_live[layer_idx] = True


def select_topk_for_layer_batched(cache, layer_idx, req_ids, query_states, attention=None,
                                  decode_write=None, middle_only=False, selection_output=None):
    """Select the visible tokens of every request row for one layer.

    query_states: [B, HQ, D] post-RoPE query of the token being decoded.
    attention: object with ``.indexer`` (NFAIndexer) and ``.scaling``.
    decode_write: None (K/V of the current token already written with
    ``cache.write_decode``) or ``(k [B,HK,1,D], v [B,HK,1,DV], slots [B])`` to
    fuse the write into the step.
    """
    if query_states is None:
        raise ValueError("production selection requires current post-RoPE query")
    if middle_only:
        if selection_output is None or len(selection_output) != 2:
            raise ValueError("middle-only selection requires gather/lens output")
    elif selection_output is not None:
        raise ValueError("custom selection output requires middle_only=True")
    b = len(req_ids)
    if b == 0:
        return
    if b > cache.planned_lengths_buf.numel():
        raise ValueError("selector batch exceeds fixed query metadata capacity")
    indexer = attention.indexer
    hq, d = cache.num_query_heads, cache.layers[0].head_dim_k
    if query_states.shape != (b, hq, d):
        raise ValueError(f"current query must be [{b},{hq},{d}] for one layer, got {tuple(query_states.shape)}")
    if not query_states.is_cuda:
        raise FallbackRequired("CUDA required")
    if query_states.dtype != cache.dtype:
        raise ValueError("query dtype must match the KV pool dtype")
    rt = cache.ensure_index(indexer)
    lib = _capi.lib()
    stream = _capi.current_stream()
    g, layer, batch = C.byref(rt.geometry), C.byref(rt.layer_structs[layer_idx]), rt.batch_struct(b)
    q = query_states if query_states.is_contiguous() else query_states.contiguous()
    status = C.c_void_p(cache.status_buf.data_ptr())
    scale = float(attention.scaling)

    _ensure_index_built(cache, rt, layer_idx, req_ids, has_current_token_in_pool=False)
    if decode_write is not None:
        keys, values, slots = decode_write
        if keys.ndim != 4 or keys.shape[-2] != 1:
            raise ValueError("graph-ready decode KV must be one token per row")
        if values.ndim != 4 or values.shape[-2] != 1:
            raise ValueError("paged write decode expects [B,HK,1,DV] values")
        if keys.shape[0] != b or keys.shape[0] != slots.shape[0]:
            raise ValueError("request batch must match KV batch")
        if keys.shape[1] != cache.num_kv_heads:
            raise ValueError("KV head count does not match arena")
        k = keys.to(cache.dtype).contiguous()
        v = values.to(cache.dtype).contiguous()
        slots = slots.to(device=k.device, dtype=torch.int32).contiguous()
        kp, vp, sp = _capi.ptr(k), _capi.ptr(v), _capi.ptr(slots)
    else:
        kp = vp = sp = None      # K/V already in the pool: refresh the index of the newest token
    if middle_only:
        # the L2 survivors alone (no sink, no window) into the caller's buffers: the middle arm of
        # the disjoint protected / middle operator mode (nfa_layer_batch_selector.py:2649-2671)
        gather, lens = selection_output
        if gather.dtype != torch.int32 or lens.dtype != torch.int32 or not gather.is_contiguous():
            raise ValueError("selection_output must be contiguous int32 (gather, lens)")
        if gather.shape[-1] != cache.max_visible_len or tuple(gather.shape[:2]) != (b, cache.num_kv_heads):
            raise ValueError("selection_output gather must be [B, Hkv, max_visible]")
    else:
        gather = cache.gather_indices_for_layer(layer_idx)
        lens = cache.visible_lens_for_layer(layer_idx)
    diag = bool(getattr(cache, "selector_diagnostics", False))
    sel = rt.selection_struct(gather, lens, with_middle=diag, with_page_lists=diag)
    sel.middle_only = 1 if middle_only else 0
    _capi.check(lib.loda_select_step(g, layer, C.byref(batch), _capi.ptr(q), kp, vp, sp, scale, C.byref(sel),
                                     status, _capi.ptr(rt.workspace), stream))


def last_middle_selection(cache, batch):
    """The L2 survivors of the most recent call as a TokenSelection
    (logical ids ascending, before the union with sink and window).  Only
    written when ``cache.selector_diagnostics`` is True."""
    rt = cache._runtime
    return TokenSelection(rt.middle[:batch], rt.middle_counts[:batch])


def decode_step_fused(cache, layer_idx, req_ids, query_states, attention, decode_write, out=None, chained=False):
    """append + L1 + L2 + gather attention of one layer through the single
    C entry point ``loda_decode_step``; returns the attention output [B, HQ, DV].
    chained=True promises that this call directly follows the same call for another layer of the
    same step on the same stream (LODA_SEL_CHAINED in include/loda_b200.h)."""
    b = len(req_ids)
    indexer = attention.indexer
    rt = cache.ensure_index(indexer)
    _ensure_index_built(cache, rt, layer_idx, req_ids, has_current_token_in_pool=False)
    keys, values, slots = decode_write
    k = keys.to(cache.dtype).contiguous()
    v = values.to(cache.dtype).contiguous()
    slots = slots.to(device=k.device, dtype=torch.int32).contiguous()
    q = query_states if query_states.is_contiguous() else query_states.contiguous()
    if out is None:
        out = q.new_empty((b, cache.num_query_heads, cache.layers[layer_idx].head_dim_v))
    batch = rt.batch_struct(b)
    diag = bool(getattr(cache, "selector_diagnostics", False))
    sel = rt.selection_struct(cache.gather_indices_for_layer(layer_idx), cache.visible_lens_for_layer(layer_idx),
                              with_middle=diag, with_page_lists=diag, chained=chained)
    _capi.check(_capi.lib().loda_decode_step(
        C.byref(rt.geometry), C.byref(rt.layer_structs[layer_idx]), C.byref(batch), _capi.ptr(q),
        _capi.ptr(k), _capi.ptr(v), _capi.ptr(slots), float(attention.scaling), C.byref(sel),
        _capi.ptr(cache.query_to_req_buf), _capi.ptr(out), C.c_void_p(cache.status_buf.data_ptr()),
        _capi.ptr(rt.workspace), _capi.current_stream()))
    return out
