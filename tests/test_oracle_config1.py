"""Configuration 1 as specified, on the CPU oracle: one Qwen3-8B-shaped layer, fp32, seed 0, 32 query /
8 KV heads, head_dim 128, 32 768 tokens in 16-token pages, N(0,1) keys with RoPE (theta 1e6), four
outlier channels per head scaled x8, eight needle tokens whose keys point along the query; L1 top-128
pages (min/max far pool, mean near pool, 32 near pages / 4 096 tokens), L2 top-1 024 tokens on the 4-bit
tail half-subspace (cmp_ratio 4), sink 4, window 128.  The needles are what the configuration is for
(selection recall): a KV head whose outlier channels lie outside the scoring subspace must select all
eight; where an outlier channel falls inside the 32 scoring dims (here heads 1, 4 and 7) ordinary tokens
outscore the needles on it and the page-level filter drops some — every needle whose page level 1 keeps
is kept by level 2.  Over the eight heads the recall is 51 of 64, the same in both arithmetic modes."""
import importlib

import numpy as np
import pytest
import torch

from oracle import loda_oracle as O

synth = importlib.import_module("two-level-attention_b200.synth")


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_config1_selects_every_needle_in_every_head(mode):
    length = 32768
    case = synth.make_decode_case(length, num_q_heads=32, num_kv_heads=8, head_dim=128, seed=0, theta=1e6,
                                  n_needles=8, dtype=torch.float32, device="cpu")
    assert len(case.needles) == 8
    cfg = O.SelectorConfig(head_dim=128, num_q_heads=32, num_kv_heads=8, block_size=16,
                           max_blocks=length // 16 + 4, level1_topk=128, near_pages=32, near_len=4096,
                           level2_topk=1024, cmp_ratio=4, sink=4, swa=128, max_visible=1024, mode=mode)
    sel = O.select_request(case.q.numpy(), case.k.numpy(), length, cfg, case.scale)
    needles = set(int(t) for t in case.needles.tolist())
    dims = set(int(d) for d in cfg.dims)
    total = 0
    for kv in range(8):
        ids = set(int(t) for t in sel.logical[kv])
        assert len(ids) == 1024
        assert set(range(4)) <= ids and set(range(length - 128, length)) <= ids
        kept_pages = set(int(p) for p in sel.i_far[kv, :sel.n_far[kv]])
        found = needles & ids
        total += len(found)
        # level 2 loses no needle that level 1 kept
        assert {t for t in needles if t // 16 in kept_pages} == found, kv
        if not (set(int(c) for c in case.outlier_channels[kv]) & dims):
            assert found == needles, (kv, sorted(needles - found))
    assert total >= 48, total            # 51 of 64 with this seed
