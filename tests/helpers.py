"""Glue between the package's case builder and the oracle for the GPU tests."""
from __future__ import annotations

import importlib

from oracle import loda_oracle as O

PKG = "two-level-attention_b200"


def mod(sub):
    return importlib.import_module(f"{PKG}.{sub}")


def bf16_to_f32_np(t):
    return t.detach().float().cpu().numpy()


def oracle_config(setup):
    import numpy as np
    a, ix, c = setup.args, setup.indexer, setup.cache
    lo0, lo1, dsub = ix.subspace_ranges()
    dims = np.concatenate((np.arange(lo0, lo0 + dsub // 2), np.arange(lo1, lo1 + dsub // 2)))
    return O.SelectorConfig(
        dims=dims,
        head_dim=c.layers[0].head_dim_k, num_q_heads=c.num_query_heads, num_kv_heads=c.num_kv_heads,
        block_size=setup.page, max_blocks=setup.max_blocks, level1_topk=int(a.tia_level1_topk),
        near_pages=int(a.nfa_near_pages), near_len=int(a.nfa_near_len), level2_topk=int(a.tia_level2_topk),
        cmp_ratio=int(a.tia_level2_cmp_ratio), sink=ix.sink_tokens, swa=ix.sliding_window_size,
        max_visible=setup.max_visible, mode="bf16", near_tokens=ix.nt_near_tokens, far_method=ix.far_method,
        near_method=ix.near_method, geometry_near=c.geometry.near)


def make_setup(lengths, **kw):
    setup = mod("testing").make_setup(lengths, **kw)
    setup.cfg = oracle_config(setup)
    return setup


def oracle_selection(setup, i):
    case = setup.cases[i]
    skips = getattr(setup, "skip_states", None)
    sf, sn = (False, False) if skips is None else skips[i]
    return O.select_request(bf16_to_f32_np(case.q), bf16_to_f32_np(case.k), case.length,
                            setup.cfg, setup.attention.scaling, skip_far=sf, skip_near=sn)


def pools_np(layer):
    return (bf16_to_f32_np(layer.kv_pool_k[:, 0]), bf16_to_f32_np(layer.kv_pool_v[:, 0]))
