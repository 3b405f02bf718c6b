"""The allocation-free gather attention entry point.

`loda_gather_attend_static` serves hosts that cannot allocate device memory at
the call site (a plugin inside another runtime's fixed memory plan, a process
whose memory was carved up at start): its split-K scratch is a fixed array
inside the library.  Here it is called twice in a row through the C ABI on the
same inputs as the regular entry point, whose output it must reproduce, and it
must refuse calls beyond its stated limit.  The file sorts last so that a run
stopping at the first failure has already exercised everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_attention_matches_workspace_attention_twice():
    from helpers import make_setup, mod
    capi = mod("_capi")
    lib = capi.lib()
    sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
    nfa = mod("sparse_attn.ops.paged_region_kernels_nfa")
    setup = make_setup([5000, 900, 2600], seed=9)
    cache = setup.cache
    n = len(setup.req_ids)
    cache.plan_common(setup.req_ids)
    slots = cache.slot_mapping_for_layer(0)[:n]
    sel_mod.select_topk_for_layer_batched(cache, 0, setup.req_ids, setup.q, attention=setup.attention,
                                          decode_write=(setup.k_new, setup.v_new, slots))
    want = nfa.decode_graph_ready(setup.attention, setup.q, cache)     # regular entry point
    rt = cache._runtime
    gather = cache.gather_indices_for_layer(0)
    lens = cache.visible_lens_for_layer(0)
    for attempt in range(2):
        got = torch.full_like(want, float("nan"))
        rc = lib.loda_gather_attend_static(
            C.byref(rt.geometry), C.byref(rt.layer_structs[0]), capi.ptr(setup.q), capi.ptr(gather),
            capi.ptr(lens), capi.ptr(cache.query_to_req_buf), n, cache.max_requests,
            float(setup.attention.scaling), capi.ptr(got), capi.current_stream())
        assert rc == 0, lib.loda_last_error()
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2,
                                   msg=lambda m: f"call {attempt}: {m}")


def test_static_scratch_attention_rejects_sizes_beyond_its_limit():
    from helpers import mod
    capi = mod("_capi")
    lib = capi.lib()
    # 16 query rows x 8 kv heads = 128 pairs > 64: refused before anything is launched
    g = capi.Geometry(dtype=0, num_q_heads=32, num_kv_heads=8, head_dim=128, head_dim_v=128, sub_dims=32,
                      sub_lo0=48, sub_lo1=112, page=16, num_pages=64, max_blocks=64, max_requests=16,
                      max_query_tokens=16, max_visible=1024, k_far=32, k_near=32, level2_topk=1024, sink=4,
                      swa=128, near_len=4096, pool_near_len=4096)
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda:0")
    layer = capi.Layer(pool_k=dummy.data_ptr(), pool_v=dummy.data_ptr())
    p = capi.ptr(dummy)
    rc = lib.loda_gather_attend_static(C.byref(g), C.byref(layer), p, p, p, p, 16, 16, 1.0, p,
                                       capi.current_stream())
    assert rc == capi.LODA_ERR_UNSUPPORTED
    assert b"limited to" in lib.loda_last_error()
