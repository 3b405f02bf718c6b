"""Builders for self-checks and tests: a populated paged cache on the device
filled with seeded synthetic requests (no oracle dependency)."""
from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import torch

from . import synth
from .sparse_attn.cache import paged_region_cache as cache_mod
from .sparse_attn.indexer import nfa_indexer as idx_mod
from .sparse_attn.ops import paged_region_kernels_nfa as nfa
from .sparse_attn.policies import region_geometry as geo_mod


def make_setup(lengths, *, seed=0, page=16, hq=32, hkv=8, d=128, n_layers=1, max_visible=1024,
               shuffle_pages=True, extra_blocks=4, selector_overrides=None, max_requests=None,
               device="cuda:0", skip_states=None, dv=None, shared_latent=False):
    """Create a cache, prefill every request with `length - 1` synthetic tokens
    (seeded, generated on the CPU), and return the decode inputs of the last
    token of each request."""
    dev = torch.device(device)
    b = len(lengths)
    max_len = max(lengths)
    max_blocks = (max_len + page - 1) // page + extra_blocks
    total_pages = sum((l + page - 1) // page for l in lengths) + 2 * b + 8
    dv = d if dv is None else dv
    extra = {} if d == 128 else {"head_dim": d}
    args = nfa.nfa_args("tail", tia_block_size=page, **extra, **(selector_overrides or {}))
    indexer = idx_mod.NFAIndexer(args)
    geometry = geo_mod.RegionGeometry(sink=indexer.sink_tokens, near=int(args.nfa_near_len),
                                      window=indexer.sliding_window_size, page=page, max_new_tokens=64)
    cache = cache_mod.GraphReadyPagedRegionCache(
        n_layers, geometry, max_requests=max_requests or b, max_physical_pages=total_pages,
        max_blocks=max_blocks, max_visible_len=max_visible, max_query_tokens=b, num_kv_heads=hkv,
        num_query_heads=hq, head_dim_k=d, head_dim_v=dv, dtype=torch.bfloat16, device=dev,
        shared_latent=shared_latent)
    cache.selector_diagnostics = True
    rng = np.random.default_rng(seed)
    free = [int(p) for p in rng.permutation(total_pages)] if shuffle_pages else list(range(total_pages))
    cases, req_ids = [], []
    for i, length in enumerate(lengths):
        case = synth.make_decode_case(length, num_q_heads=hq, num_kv_heads=hkv, head_dim=d,
                                      seed=seed * 1000 + i, dtype=torch.bfloat16, device="cpu")
        case.v = case.k[..., :dv].clone() if shared_latent else case.v[..., :dv].contiguous()
        rid = cache.add_request()
        n_pre = length - 1
        if n_pre > 0:
            need = (n_pre + page - 1) // page
            pages, free = free[:need], free[need:]
            for li in range(n_layers):
                kk = case.k[:n_pre].permute(1, 0, 2)[None].to(dev)
                vv = case.v[:n_pre].permute(1, 0, 2)[None].to(dev)
                cache.write_prefill(li, rid, kk, vv, physical_pages=pages if li == 0 else None)
            sf, sn = (False, False) if skip_states is None else skip_states[i]
            cache.freeze(rid, [sf] * n_layers, [sn] * n_layers)
        cases.append(case)
        req_ids.append(rid)
    attention = SimpleNamespace(indexer=indexer, scaling=float(d) ** -0.5, layer_idx=0)
    q = torch.stack([c.q for c in cases]).to(dev)                                    # [B, Hq, D]
    k_new = torch.stack([c.k[c.length - 1] for c in cases])[:, :, None].to(dev)      # [B, Hkv, 1, D]
    v_new = torch.stack([c.v[c.length - 1] for c in cases])[:, :, None].to(dev)
    return SimpleNamespace(cache=cache, cases=cases, req_ids=req_ids, attention=attention, q=q,
                           k_new=k_new, v_new=v_new, lengths=list(lengths), dev=dev, indexer=indexer,
                           args=args, page=page, max_blocks=max_blocks, max_visible=max_visible,
                           skip_states=skip_states)
