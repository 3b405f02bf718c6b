"""A contiguous KV cache [maxB, S, Hkv, D] seen as a paged pool with one-token
pages: token (b, s) is physical slot b * S + s, and the pool layout
[pages, Hkv, 1, D] is exactly the cache's memory.  The gather-attention kernel
of the paged path then serves the prototype operators unchanged."""
from __future__ import annotations

import ctypes as C

import torch

from ... import _capi

_cache = {}


def runtime(q, k, v, num_heads, num_kv_heads, max_visible):
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise _capi.FallbackRequired("tls_attn operators of this package take bf16 tensors")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("tls_attn operators need CUDA tensors (no CPU path in this package)")
    if not (k.is_contiguous() and v.is_contiguous()):
        raise ValueError("k and v caches must be contiguous [maxB, S, Hkv, D]")
    batch = q.shape[0]
    key = (k.data_ptr(), v.data_ptr(), tuple(k.shape), v.shape[-1], num_heads, batch, max_visible, q.device.index)
    rt = _cache.get(key)
    if rt is not None:
        return rt
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("warm this shape up once before CUDA graph capture")
    max_b, s, hkv, d = k.shape
    g = _capi.Geometry(
        dtype=_capi.LODA_DTYPE_BF16, num_q_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=d,
        head_dim_v=v.shape[-1], sub_dims=32, sub_lo0=0, sub_lo1=16, page=1, num_pages=max_b * s + 1,
        max_blocks=16, max_requests=batch, max_query_tokens=batch, max_visible=max_visible, k_far=0, k_near=0,
        level2_topk=1, sink=0, swa=1, near_len=1, pool_near_len=1)      # the selector is not used: smallest legal budgets
    nbytes = _capi.lib().loda_workspace_bytes(C.byref(g))
    if nbytes == 0:
        raise _capi.FallbackRequired(_capi.lib().loda_last_error().decode())
    rt = {
        "geometry": g,
        "layer": _capi.Layer(pool_k=k.data_ptr(), pool_v=v.data_ptr()),
        "workspace": torch.zeros(nbytes, dtype=torch.uint8, device=q.device),
        "q2r": torch.arange(batch, dtype=torch.int32, device=q.device),
        "row_base": (torch.arange(batch, dtype=torch.int32, device=q.device) * s).view(batch, 1, 1),
        "seq": s,
    }
    if len(_cache) > 16:
        _cache.clear()
    _cache[key] = rt
    return rt


def attend(rt, q, gather, lens, scaling, out):
    batch = q.shape[0]
    qc = q.reshape(batch, q.shape[-2], q.shape[-1]).contiguous()
    _capi.check(_capi.lib().loda_gather_attend(
        C.byref(rt["geometry"]), C.byref(rt["layer"]), _capi.ptr(qc), _capi.ptr(gather), _capi.ptr(lens),
        _capi.ptr(rt["q2r"]), batch, batch, float(scaling), _capi.ptr(out), _capi.ptr(rt["workspace"]),
        _capi.current_stream()))
    return out
