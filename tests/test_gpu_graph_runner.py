"""DecodeGraphRunner (the mirror of the reference's GraphRunner for this path, sparse_attn/engine/graph_runner.py:
78-133 capture, 155-200 step): host-side planning into fixed device buffers, one graph replay over all layers
with pinned host inputs and outputs.  Three consecutive decode steps through the runner must give the same
lists and the same attention bits as the same steps issued eagerly, layer by layer, on an identical cache."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lengths", [[12000], [6000, 900, 20000]], ids=["one_launch_chained_layers", "batch_chain"])
def test_runner_steps_equal_eager_steps(lengths):
    from helpers import make_setup, mod
    sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
    gr = mod("sparse_attn.engine.graph_runner")
    n_layers, steps, nb = 2, 3, len(lengths)
    a = make_setup(lengths, seed=81, n_layers=n_layers)
    b = make_setup(lengths, seed=81, n_layers=n_layers)
    for s in (a, b):
        s.cache.selector_diagnostics = False
    hq, hkv = a.cache.num_query_heads, a.cache.num_kv_heads
    d = a.q.shape[-1]
    g = torch.Generator().manual_seed(5)
    qh = torch.randn(steps, n_layers, nb, hq, d, generator=g).to(torch.bfloat16).pin_memory()
    kh = torch.randn(steps, n_layers, nb, hkv, 1, d, generator=g).to(torch.bfloat16).pin_memory()
    vh = torch.randn(steps, n_layers, nb, hkv, 1, d, generator=g).to(torch.bfloat16).pin_memory()

    def attn_objs(setup):
        return [types.SimpleNamespace(indexer=setup.attention.indexer, scaling=setup.attention.scaling, layer_idx=li)
                for li in range(n_layers)]

    runner = gr.DecodeGraphRunner(a.cache, attn_objs(a), nb)
    runner.q.copy_(qh[0]); runner.k.copy_(kh[0]); runner.v.copy_(vh[0])
    runner.capture(a.req_ids)
    eager_attn = attn_objs(b)
    for s in range(steps):
        out_a = runner.step(qh[s], kh[s], vh[s]).clone()
        cache = b.cache
        cache.plan_common(b.req_ids)
        outs = []
        for li in range(n_layers):
            slots = cache.slot_mapping_for_layer(li)[:nb]
            outs.append(sel_mod.decode_step_fused(cache, li, b.req_ids, qh[s, li].cuda(), eager_attn[li],
                                                  (kh[s, li].cuda(), vh[s, li].cuda(), slots)).clone())
        torch.cuda.synchronize()
        cache.commit_step()
        assert a.cache.read_status() == 0 and cache.read_status() == 0
        for li in range(n_layers):
            la, lb = a.cache.visible_lens_for_layer(li)[:nb], cache.visible_lens_for_layer(li)[:nb]
            assert torch.equal(la, lb)
            n = int(la.max())
            assert torch.equal(a.cache.gather_indices_for_layer(li)[:nb, :, :n], cache.gather_indices_for_layer(li)[:nb, :, :n])
            assert torch.equal(out_a[li].cuda(), outs[li])
    assert runner.replays == steps
    assert a.cache.get_seq_length() == b.cache.get_seq_length()
