"""GPU parity of the selector modes beside the default: frozen region-skip decisions per request
(far-only, near-only, both skipped, mixed in one batch), the numeric near-token quota, the other
level-1 scoring methods; and the device-side guard on request slots.  All against the CPU oracle,
integers identical, attention within the bf16 tolerance."""
import numpy as np
import pytest
import torch

from test_gpu_parity import _check_against_oracle, _run_decode_step, _run_step

pytestmark = pytest.mark.gpu

NS, FAR, NEAR, BOTH = (False, False), (True, False), (False, True), (True, True)


def test_mixed_skip_states_in_one_batch():
    from helpers import make_setup
    lengths = [9000, 9001, 20000, 4400, 131, 6000, 300, 12289]
    skips = [NS, FAR, NEAR, BOTH, FAR, BOTH, NEAR, FAR]
    setup = make_setup(lengths, seed=51, skip_states=skips)
    out = _run_step(setup)
    _check_against_oracle(setup, out)
    lens = setup.cache.visible_lens_for_layer(0).cpu().numpy()
    # both regions skipped: exactly sink + window
    assert (lens[3] == 4 + 128).all() and (lens[5] == 4 + 128).all()


@pytest.mark.parametrize("skip", [FAR, NEAR, BOTH], ids=["skip_far", "skip_near", "skip_both"])
@pytest.mark.parametrize("length", [20000, 131072])
def test_single_request_skip_states_on_the_one_launch_path(skip, length, monkeypatch):
    from helpers import make_setup
    a = make_setup([length], seed=53, skip_states=[skip])
    out_a, launches = _run_decode_step(a)
    assert launches == 1
    _check_against_oracle(a, out_a)
    monkeypatch.setenv("LODA_B200_SELECT_PATH", "split")
    b = make_setup([length], seed=53, skip_states=[skip])
    out_b, launches_b = _run_decode_step(b)
    assert launches_b == 3
    _check_against_oracle(b, out_b)
    assert torch.equal(a.cache.visible_lens_for_layer(0), b.cache.visible_lens_for_layer(0))


@pytest.mark.parametrize("page", [16, 64])
def test_skip_states_with_other_geometries(page):
    from helpers import make_setup
    ov = {"tia_level1_topk": 32, "nfa_near_pages": 8, "tia_level2_topk": 256, "nfa_swa_size": 64, "nfa_near_len": 1024}
    lengths = [4241, 4242, 4300, 4400, 900, 70]
    setup = make_setup(lengths, seed=55, page=page, selector_overrides=ov, max_visible=256,
                       skip_states=[NS, FAR, NEAR, BOTH, FAR, NEAR])
    out = _run_step(setup)
    _check_against_oracle(setup, out)


@pytest.mark.parametrize("near_tokens", [0, 48, 128])
def test_numeric_near_token_quota(near_tokens):
    """nfa_near_tokens as a number: the far and the near region select separately, each with its own
    hole fill; the far region's unused budget goes to the near region."""
    from helpers import make_setup
    ov = {"tia_level1_topk": 32, "nfa_near_pages": 8, "tia_level2_topk": 256, "nfa_swa_size": 64,
          "nfa_near_len": 1024, "nfa_near_tokens": near_tokens}
    lengths = [4241, 2500, 1100, 300, 9000, 4242, 4300, 4400]
    skips = [NS, NS, NS, NS, NS, FAR, NEAR, BOTH]
    setup = make_setup(lengths, seed=57, selector_overrides=ov, max_visible=256, skip_states=skips)
    out = _run_step(setup)
    _check_against_oracle(setup, out)
    one = make_setup([20000], seed=57, selector_overrides=ov, max_visible=256)
    out1, launches = _run_decode_step(one)
    assert launches == 3            # the one-launch kernel serves the default quota only
    _check_against_oracle(one, out1)


@pytest.mark.parametrize("overrides", [
    {"nfa_far_method": "avg"},
    {"nfa_near_method": "minmax"},
    {"nfa_far_method": "avg_top2"},
    {"nfa_far_method": "avg", "nfa_near_method": "minmax", "tia_level2_cmp_ratio": 2},
], ids=["far_avg", "near_minmax", "far_avg_top2", "swapped_sub64"])
def test_other_level1_methods(overrides):
    from helpers import make_setup
    setup = make_setup([9000, 20000, 700, 40000], seed=59, selector_overrides=overrides,
                       skip_states=[NS, NS, NS, FAR])
    out = _run_step(setup)
    _check_against_oracle(setup, out)


@pytest.mark.parametrize("lengths", [[6000], [6000, 900, 3000]], ids=["one_launch", "chain"])
def test_request_slot_outside_the_cache_sets_a_status_bit_and_touches_nothing(lengths):
    """An active row whose request slot is out of range must not address memory with it: the row
    behaves like a padding row and LODA_STATUS_BAD_REQ is raised."""
    from helpers import make_setup, mod
    sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
    capi = mod("_capi")
    setup = make_setup(lengths, seed=61)
    cache = setup.cache
    out_ok, _ = _run_decode_step(setup)                    # builds the index; a normal step
    cache.plan_common(setup.req_ids)
    cache.valid_req_ids_buf[0] = 1 << 40                   # row 0: slot far outside [0, max_requests)
    mm_before = cache.layers[0].page_mm.clone()
    slots = cache.slot_mapping_for_layer(0)[:len(lengths)]
    out = sel_mod.decode_step_fused(cache, 0, setup.req_ids, setup.q, setup.attention,
                                    (setup.k_new, setup.v_new, slots))
    torch.cuda.synchronize()
    status = cache.read_status()
    assert status & capi.STATUS_BAD_REQ
    assert (cache.visible_lens_for_layer(0)[0] == 0).all()
    assert (out[0] == 0).all()
    assert torch.equal(cache.layers[0].page_mm[setup.req_ids[0]], mm_before[setup.req_ids[0]])
    if len(lengths) > 1:
        assert torch.equal(out[1:], out_ok[1:])


def test_token_selection_type_matches_the_reference_contract():
    from helpers import make_setup, mod
    sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
    selection = mod("sparse_attn.indexer.selection.selector")
    setup = make_setup([5000, 700], seed=63)
    _run_step(setup)
    picked = sel_mod.last_middle_selection(setup.cache, 2)
    indices, counts = picked                               # a NamedTuple: callers unpack it
    assert picked.valid().sum(-1).eq(counts).all()
    mask = picked.to_mask(5000)
    assert mask.sum(-1).eq(counts).all()
    again = selection.canonical_selection(torch.where(picked.valid(), indices, -1), picked.valid(), 5000,
                                          width=indices.shape[-1])
    assert torch.equal(again.counts, counts)
    assert torch.equal(again.indices * again.valid(), indices * picked.valid())


@pytest.mark.parametrize("nreq", [10, 12, 18])
def test_batches_whose_attention_splits_in_two(nreq):
    """Between 74 and 147 (request, kv head) pairs the attention splits every list over two CTAs, each of
    which merges more output elements than it has threads."""
    from helpers import make_setup
    lengths = [3000 + 517 * i for i in range(nreq)]
    setup = make_setup(lengths, seed=65)
    out = _run_step(setup)
    _check_against_oracle(setup, out)


@pytest.mark.parametrize("path", ["grid", "stream"])
def test_level1_grid_and_streaming_kernels(path, monkeypatch):
    """The two forms of the batched level-1 launch (a CTA per item; a resident grid that streams its
    items' tiles and then selects rows from a queue) on a batch with empty, short and long rows and
    all region-skip states; twice on the same cache, so that the queue and the tickets are rearmed."""
    from helpers import make_setup
    monkeypatch.setenv("LODA_B200_L1_PATH", path)
    lengths = [9000, 131, 20000, 4400, 70000, 6000, 300, 12289, 33000, 5, 4241, 65537]
    skips = [NS, NS, NEAR, BOTH, NS, FAR, NS, FAR, NS, NS, NEAR, NS]
    setup = make_setup(lengths, seed=67, skip_states=skips)
    out = _run_step(setup)
    _check_against_oracle(setup, out)
    again = _run_step(setup)
    assert torch.equal(out, again)


@pytest.mark.parametrize("overrides,page", [
    ({"nfa_far_method": "avg_top2", "nfa_near_method": "minmax"}, 16),
    ({"tia_level2_cmp_ratio": 2}, 16),
    ({"tia_level2_cmp_ratio": 8}, 64),
], ids=["other_methods", "sub64", "sub16_page64"])
def test_level1_streaming_kernel_other_shapes(overrides, page, monkeypatch):
    from helpers import make_setup
    monkeypatch.setenv("LODA_B200_L1_PATH", "stream")
    setup = make_setup([9000, 20000, 700, 40000, 2500], seed=69, page=page, selector_overrides=overrides,
                       skip_states=[NS, NS, NS, FAR, NEAR])
    out = _run_step(setup)
    _check_against_oracle(setup, out)


def test_streaming_kernel_gives_up_on_a_row_that_never_completes(monkeypatch):
    """The streaming level-1 kernel waits for a row's ticket before it selects the row.  The wait is bounded:
    with the ticket of one row made unreachable (a count that its items can never bring up to the full
    number) the launch returns after the poll limit, raises LODA_STATUS_TIMEOUT, leaves that row alone and
    serves the others; with the scratch zeroed again the next step is exact."""
    from helpers import make_setup, mod
    sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
    capi = mod("_capi")
    monkeypatch.setenv("LODA_B200_L1_PATH", "stream")
    lengths = [9000, 20000, 700]
    setup = make_setup(lengths, seed=71)
    cache = setup.cache
    out_ok = _run_step(setup)                                  # a normal step (builds the index)
    _check_against_oracle(setup, out_ok)
    lens_ok = cache.visible_lens_for_layer(0).clone()
    rt = cache._runtime
    rows = len(lengths) * cache.num_kv_heads
    tickets = rt.workspace[:4 * (rows + 2)].view(torch.int32)  # the tickets lead the scratch; then queue, exit count
    stuck = 1 * cache.num_kv_heads + 3                         # request 1, kv head 3
    tickets[stuck] = -(1 << 24)
    cache.plan_common(setup.req_ids)
    slots = cache.slot_mapping_for_layer(0)[:len(lengths)]
    out = sel_mod.decode_step_fused(cache, 0, setup.req_ids, setup.q, setup.attention,
                                    (setup.k_new, setup.v_new, slots))
    torch.cuda.synchronize()
    status = cache.read_status()
    assert status & capi.STATUS_TIMEOUT
    assert int(tickets[rows]) == 0 and int(tickets[rows + 1]) == 0      # queue and exit count rearmed
    heads = [h for h in range(out.shape[1]) if h // (cache.num_query_heads // cache.num_kv_heads) != 3]
    assert torch.equal(out[0], out_ok[0]) and torch.equal(out[2], out_ok[2])
    assert torch.equal(out[1][heads], out_ok[1][heads])
    assert torch.equal(cache.visible_lens_for_layer(0), lens_ok)        # the stuck row kept its list of the step before
    tickets.zero_()
    again = _run_step(setup)
    assert torch.equal(again, out_ok)
