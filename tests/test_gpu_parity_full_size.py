"""GPU parity at the sizes the benchmark runs: the 131 072-token request of the latency case (a
cluster of 8 CTAs per row with three double-buffered tiles per CTA), lengths around it, the
32-request batch with lengths in [8 192, 65 536], and cases built so that a stale read would show:
a newest token that carries most of the softmax mass, heavily tied page scores, and a device kernel
that advances the lengths directly before the step."""
import numpy as np
import pytest
import torch

from oracle import loda_oracle as O
from test_gpu_parity import ATOL, RTOL, _check_against_oracle, _run_decode_step, _run_step

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("length", [131072, 65537, 100000])
def test_one_launch_decode_step_at_benchmarked_lengths(length):
    """One request of the benchmark's length through loda_decode_step: every CTA of a row's cluster
    scores several tiles (two staging buffers), and the attention tile is laid over both buffers."""
    from helpers import make_setup
    setup = make_setup([length], seed=31)
    out, launches = _run_decode_step(setup)
    assert launches == 1
    _check_against_oracle(setup, out)


def test_one_launch_and_split_paths_agree_at_131072(monkeypatch):
    from helpers import make_setup
    a = make_setup([131072], seed=33)
    out_a, launches = _run_decode_step(a)
    assert launches == 1
    monkeypatch.setenv("LODA_B200_SELECT_PATH", "split")
    b = make_setup([131072], seed=33)
    out_b, launches_b = _run_decode_step(b)
    assert launches_b == 3
    _check_against_oracle(b, out_b)
    n = int(a.cache.visible_lens_for_layer(0).max())
    assert torch.equal(a.cache.visible_lens_for_layer(0), b.cache.visible_lens_for_layer(0))
    assert torch.equal(a.cache.gather_indices_for_layer(0)[..., :n], b.cache.gather_indices_for_layer(0)[..., :n])
    assert torch.allclose(out_a.float(), out_b.float(), atol=ATOL, rtol=RTOL)


def test_batch_of_32_requests_with_lengths_8k_to_64k():
    """The batched configuration: 32 requests, lengths uniform in [8 192, 65 536], one shared pool
    with shuffled page tables; every row's page lists, token lists and attention are checked."""
    import random
    from helpers import make_setup
    rnd = random.Random(5)
    lengths = [rnd.randint(8192, 65536) for _ in range(32)]
    lengths[3], lengths[17] = 8192, 65536
    setup = make_setup(lengths, seed=35)
    out = _run_step(setup)
    _check_against_oracle(setup, out)


def _dominant_newest_token(setup, c=60.0):
    """Make the decoded token carry almost all of the softmax mass of every head: its key points
    along the group-mean query, its value is a constant no other token has; the slot it will be
    written to is poisoned first, so that an attention that misses the write sees other data."""
    cache, dev = setup.cache, setup.dev
    cache.plan_common(setup.req_ids)
    slots = cache.slot_mapping_for_layer(0)[:len(setup.req_ids)].cpu().tolist()
    layer = cache.layers[0]
    page = setup.page
    for b, case in enumerate(setup.cases):
        hkv = case.k.shape[1]
        qbar = case.q.float().view(hkv, -1, case.q.shape[-1]).mean(1)
        k_new = (c * qbar / qbar.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
        v_new = torch.full_like(k_new, 3.0)
        case.k[case.length - 1] = k_new
        case.v[case.length - 1] = v_new
        setup.k_new[b, :, 0] = k_new.to(dev)
        setup.v_new[b, :, 0] = v_new.to(dev)
        ph, off = divmod(slots[b], page)
        layer.kv_pool_k[ph, 0, :, off] = 0.0
        layer.kv_pool_v[ph, 0, :, off] = -50.0


@pytest.mark.parametrize("path", ["one_launch", "two_launch", "three_launch"])
@pytest.mark.parametrize("lengths", [[20000], [131072]], ids=["20000", "131072"])
def test_newest_token_is_read_by_the_attention_of_the_same_step(path, lengths, monkeypatch):
    from helpers import bf16_to_f32_np, make_setup
    if path == "two_launch":
        monkeypatch.setenv("LODA_B200_DECODE_PATH", "split")
    if path == "three_launch":
        monkeypatch.setenv("LODA_B200_SELECT_PATH", "split")
    setup = make_setup(lengths, seed=37)
    _dominant_newest_token(setup)
    out, launches = _run_decode_step(setup)
    assert launches == {"one_launch": 1, "two_launch": 2, "three_launch": 3}[path]
    got = bf16_to_f32_np(out)
    assert np.abs(got - 3.0).max() < 0.05, "the decoded token's value must dominate the output"
    _check_against_oracle(setup, out)


@pytest.mark.parametrize("path", ["one_launch", "split"])
def test_heavily_tied_page_scores_take_the_bisection_branch(path, monkeypatch):
    """More than 1 024 far pages share one score (constant keys), so the prefilter gives up and the
    16-bit bisection selects; ties must still go to the lower page and the lower token."""
    from helpers import make_setup
    if path == "split":
        monkeypatch.setenv("LODA_B200_SELECT_PATH", "split")
    setup = make_setup([30000], seed=39)
    case = setup.cases[0]
    # every page of the far pool (pages 1 .. 1 609) holds one and the same key: all their scores tie
    case.k[16:25760] = case.k[16].clone()
    # rebuild the cache with the edited keys
    from helpers import mod
    cache = setup.cache
    rid = setup.req_ids[0]
    n_pre = case.length - 1
    kk = case.k[:n_pre].permute(1, 0, 2)[None].to(setup.dev)
    vv = case.v[:n_pre].permute(1, 0, 2)[None].to(setup.dev)
    ops = mod("sparse_attn.ops.paged_region_kernels")
    ops.paged_write_prefill(cache.layers[0], kk, vv, cache.block_table_buf[0, rid])
    out, _ = _run_decode_step(setup)
    _check_against_oracle(setup, out)


@pytest.mark.parametrize("replay", [False, True], ids=["eager", "graph"])
def test_lengths_advanced_by_a_device_kernel_directly_before_the_step(replay):
    """A caller may advance the lengths on the device right before loda_decode_step (no host round
    trip): the step must read the new length.  Run eagerly and as a captured graph."""
    from helpers import make_setup, mod
    sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
    setup = make_setup([12001], seed=41, extra_blocks=8)
    cache = setup.cache
    out0, launches = _run_decode_step(setup)                 # step at length 12 001: builds the index
    assert launches == 1
    _check_against_oracle(setup, out0)
    cache.commit_step()
    # next token: planned on the host (slot, block table), but the device length is set back by one
    # and advanced by a device kernel right before the step
    synth = mod("synth")
    nxt = synth.make_decode_case(12002, seed=41 * 1000 + 7, dtype=torch.bfloat16, device="cpu")
    case = setup.cases[0]
    case.k = torch.cat((case.k, nxt.k[-1:]))
    case.v = torch.cat((case.v, nxt.v[-1:]))
    case.length = 12002
    setup.k_new.copy_(nxt.k[-1][None, :, None].to(setup.dev))
    setup.v_new.copy_(nxt.v[-1][None, :, None].to(setup.dev))
    cache.plan_common(setup.req_ids)
    slots = cache.slot_mapping_for_layer(0)[:1]
    static_out = torch.empty_like(out0)
    one = torch.ones(1, dtype=torch.int32, device=setup.dev)

    def step():
        cache.planned_lengths_buf[:1].add_(one)             # a device kernel writes the length ...
        sel_mod.decode_step_fused(cache, 0, setup.req_ids, setup.q, setup.attention,
                                  (setup.k_new, setup.v_new, slots), out=static_out)   # ... the step follows

    if replay:
        cache.planned_lengths_buf[:1].sub_(1)
        step()                                               # warm-up at the right length
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        cache.planned_lengths_buf[:1].sub_(1)
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                step()
        cache.gather_indices_for_layer(0).fill_(-7)
        static_out.zero_()
        graph.replay()
    else:
        cache.planned_lengths_buf[:1].sub_(1)
        step()
    torch.cuda.synchronize()
    assert cache.read_status() == 0
    assert int(cache.planned_lengths_buf[0]) == 12002
    _check_against_oracle(setup, static_out)
