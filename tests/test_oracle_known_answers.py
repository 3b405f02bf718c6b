"""The oracle against the known answers the reference's own selector tests assert
(tests/test_nfa_current_query_selector.py:228-276 numeric near-token quota and region-skip budget
semantics; tests/test_jssa_nfa_semantic.py:89-119 the packed-key order of the filtered top-k;
tests/test_nfa_current_query_selector.py:483-497 the strict region sets).  These pin, on the CPU,
the rules that decide the final token set after level 1: tie order, quota split, bypass pages,
hole fill bounds, region skipping and the union."""
import numpy as np
import pytest

from oracle import loda_oracle as O

PAGE, D = 64, 128


def _fixed_quota_case(near_tokens, skip, l2_quant):
    """The scene of _make_fixed_quota_cache: one KV head, two query heads, 448 prompt tokens whose
    key is 8 on dim 48 for tokens [4, 256) and 1 for [256, 384), one decoded token (random), the
    query 1 on dim 48, scale 1; sink 4, window 64, near 128, K1 4 (2 near pages), K2 128."""
    rng = np.random.default_rng(20261102)
    length = 449
    k = np.zeros((length, 1, D), np.float32)
    k[4:256, 0, 48] = 8
    k[256:384, 0, 48] = 1
    k[448] = O.bf16_rn(rng.standard_normal((1, D), dtype=np.float32))
    q = np.zeros((2, D), np.float32)
    q[:, 48] = 1
    cfg = O.SelectorConfig(head_dim=D, num_q_heads=2, num_kv_heads=1, block_size=PAGE, max_blocks=16,
                           level1_topk=4, near_pages=2, near_len=128, level2_topk=128, cmp_ratio=4,
                           sink=4, swa=64, max_visible=640, near_tokens=near_tokens, l2_quant=l2_quant)
    sel = O.select_request(q, k, length, cfg, 1.0, skip_far=skip[0], skip_near=skip[1])
    ids = [int(t) for t in sel.logical[0]]
    return sum(4 <= t < 256 for t in ids), sum(256 <= t < 384 for t in ids), ids


@pytest.mark.parametrize("l2_quant", [False, True], ids=["raw_keys", "int4_keys"])
def test_numeric_near_token_quota_changes_the_selection(l2_quant):
    far, near, ids = _fixed_quota_case(None, (False, False), l2_quant)
    assert (far, near, len(ids)) == (60, 0, 128)
    far, near, ids = _fixed_quota_case(16, (False, False), l2_quant)
    assert (far, near, len(ids)) == (44, 16, 128)
    assert ids == sorted(set(ids))
    # ties go to the lower token: the 44 far tokens are the first 44 of the tied run, the near ones likewise
    assert ids[:4 + 44] == list(range(48)) and ids[48:64] == list(range(256, 272))


@pytest.mark.parametrize("skip,expected", [
    ((False, False), (44, 16, 128)),
    ((True, False), (0, 60, 128)),
    ((False, True), (44, 0, 112)),
    ((True, True), (0, 0, 68)),
])
def test_numeric_near_token_quota_skip_budget_semantics(skip, expected):
    far, near, ids = _fixed_quota_case(16, skip, False)
    assert (far, near, len(ids)) == expected


def _strict_region_sets(length, skip_far, skip_near, sink=4, window=64, near=128):
    sink_hi = min(sink, length)
    near_hi = max(sink_hi, length - window)
    far_hi = min(near_hi, max(sink_hi, ((length - window - near) // PAGE) * PAGE))
    protected = set(range(sink_hi)) | set(range(near_hi, length))
    selectable = set(range(sink_hi, far_hi)) | set(range(far_hi, near_hi))
    excluded = set()
    if skip_far:
        excluded.update(range(sink_hi, far_hi))
    if skip_near:
        excluded.update(range(far_hi, near_hi))
    return protected, selectable, excluded


@pytest.mark.parametrize("hkv", [1, 2])
def test_region_skip_states_obey_the_strict_region_sets(hkv):
    """Lengths and skip states of test_batched_rows_match_isolated_noncontiguous_requests_and_skip_states:
    protected tokens always attended, nothing from a skipped region, both skipped = protected only."""
    rng = np.random.default_rng(3)
    for length, skip in zip((449, 450, 511, 514), ((False, False), (True, False), (False, True), (True, True))):
        k = O.bf16_rn(rng.standard_normal((length, hkv, D), dtype=np.float32))
        q = O.bf16_rn(rng.standard_normal((2 * hkv, D), dtype=np.float32))
        cfg = O.SelectorConfig(head_dim=D, num_q_heads=2 * hkv, num_kv_heads=hkv, block_size=PAGE, max_blocks=16,
                               level1_topk=4, near_pages=2, near_len=128, level2_topk=128, sink=4, swa=64,
                               max_visible=640, l2_quant=False)
        sel = O.select_request(q, k, length, cfg, 1.0, skip_far=skip[0], skip_near=skip[1])
        protected, selectable, excluded = _strict_region_sets(length, *skip)
        for kv in range(hkv):
            got = [int(t) for t in sel.logical[kv]]
            assert len(got) == len(set(got)) and got == sorted(got)
            assert protected <= set(got) <= protected | selectable
            assert not set(got) & excluded
            if all(skip):
                assert set(got) == protected


def test_filtered_topk_follows_the_packed_key_order():
    """(score descending, lower token first) = top-k of (ordered_bf16 << 32) + capacity - token."""
    rng = np.random.default_rng(20261118)
    capacity, budget = 20000, 1024
    # few distinct values: long runs of ties
    scores = O.bf16_rn(rng.integers(-6, 7, capacity).astype(np.float32) * np.float32(0.25))
    tokens = np.arange(capacity, dtype=np.int64)
    cfg = O.SelectorConfig(level2_topk=budget, sink=0, swa=16, near_len=4096)
    got = O.filtered_topk(tokens, scores, 0, capacity, budget, cfg)
    bits = O.bf16_bits(scores).astype(np.int64)
    ordered = np.where(bits & 0x8000, (~bits) & 0xFFFF, bits | 0x8000) - 0x8000
    keys = (ordered << 32) + capacity - tokens
    want = np.sort(capacity - (np.sort(keys)[::-1][:budget] & 0xFFFFFFFF))
    assert np.array_equal(got, want)


def test_hole_fill_takes_the_first_missing_ids_bounded_by_the_range():
    """Fewer scored candidates than the quota: the missing entries are the first ids of
    [low, high) that were not chosen (nfa_layer_batch_selector.py:545-566)."""
    cfg = O.SelectorConfig(level2_topk=64, sink=4, swa=16, near_len=4096)
    tokens = np.array([10, 11, 40, 41], np.int64)
    logits = np.array([1.0, 2.0, 3.0, -np.inf], np.float32)
    got = O.filtered_topk(tokens, logits, 0, 30, 8, cfg)
    # chosen {10, 11} (40 is outside [0, 30), 41 unscored); holes 0..5 -> ids below the sink dropped
    assert got.tolist() == [4, 5, 10, 11]
    got = O.filtered_topk(tokens, logits, 8, 12, 8, cfg)
    assert got.tolist() == [8, 9, 10, 11]          # bounded by high: only two holes exist
