"""The CPU oracle against outputs of the reference's PRODUCTION selector and gather attention,
run unmodified (Triton) on a B200 by tests/golden/make_golden_gpu.py and committed as
tests/golden/ref_selector.npz.

"exact" cases use small-integer keys and queries: every dot product of the selector is exact in
fp32 whatever the summation order, so the oracle (level 2 on the raw keys, as the reference scores
them) must reproduce the reference's token lists bit for bit — page ties, token ties, quota, hole
fill, bypass pages, region skipping, the numeric near-token quota, the other level-1 methods and the
final union included.  "normal" cases (N(0,1) inputs) are compared as set overlap: there the
reference's reduction order may move a score by an ulp."""
import importlib.util
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN, golden
from oracle import loda_oracle as O

_spec = importlib.util.spec_from_file_location("make_golden_gpu", os.path.join(GOLDEN, "make_golden_gpu.py"))
gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(gen)

G = golden("ref_selector.npz")
NAMES = sorted({k.split("/")[0] for k in G.files})


def _meta(name):
    return json.loads(bytes(G[f"{name}/meta"]).decode())


def _oracle_case(name):
    m = _meta(name)
    cfg_d = m["cfg"]
    hkv, group = cfg_d["hkv"], cfg_d["group"]
    nt = cfg_d["near_tokens"]
    cfg = O.SelectorConfig(
        head_dim=128, num_q_heads=hkv * group, num_kv_heads=hkv, block_size=m["page"], max_blocks=m["max_blocks"],
        level1_topk=cfg_d["k1"], near_pages=cfg_d["near_pages"], near_len=cfg_d["near_len"],
        level2_topk=cfg_d["k2"], cmp_ratio=4, sink=cfg_d["sink"], swa=cfg_d["window"], max_visible=cfg_d["k2"],
        mode="bf16", l2_quant=False, near_tokens=None if nt == "off" else int(nt),
        far_method=cfg_d["far_method"], near_method=cfg_d["near_method"])
    data = gen.case_inputs(name, m["kind"], m["lengths"], hkv, group)
    out = []
    for (k, v, q), length, skip in zip(data, m["lengths"], m["skips"]):
        sel = O.select_request(O.bf16_rn(q), O.bf16_rn(k), length, cfg, m["scaling"],
                               skip_far=skip[0], skip_near=skip[1])
        out.append((sel, k, v, q))
    return m, cfg, out


@pytest.mark.parametrize("name", [n for n in NAMES if n.startswith("exact")])
def test_exact_cases_reproduce_the_reference_token_lists(name):
    m, cfg, rows = _oracle_case(name)
    for row, (sel, _, _, _) in enumerate(rows):
        for kv in range(cfg.num_kv_heads):
            want = G[f"{name}/ids/{row}/{kv}"]
            assert np.all(np.diff(want) > 0), "the reference's gather list is in ascending logical order"
            got = np.asarray(sel.logical[kv], np.int32)
            assert np.array_equal(got, want), (name, row, kv, m["lengths"][row], m["skips"][row])


@pytest.mark.parametrize("name", [n for n in NAMES if n.startswith("normal")])
def test_normal_cases_overlap_with_the_reference(name):
    m, cfg, rows = _oracle_case(name)
    for row, (sel, _, _, _) in enumerate(rows):
        for kv in range(cfg.num_kv_heads):
            want = set(G[f"{name}/ids/{row}/{kv}"].tolist())
            got = set(int(t) for t in sel.logical[kv])
            assert len(got) == len(want)
            jaccard = len(got & want) / len(got | want)
            assert jaccard >= 0.97, (name, row, kv, jaccard)


@pytest.mark.parametrize("name", ["exact_p16_mid", "exact_p64_small", "normal_p16_prod"])
def test_gather_attention_matches_the_reference_output(name):
    """The oracle's attention over the REFERENCE's token lists against the reference's output."""
    m, cfg, rows = _oracle_case(name)
    page = m["page"]
    ref_out = G[f"{name}/out"]
    for row, (_, k, v, q) in enumerate(rows):
        length = m["lengths"][row]
        nblk = (length + page - 1) // page
        pad = nblk * page - length
        kk = np.concatenate((O.bf16_rn(k), np.zeros((pad,) + k.shape[1:], np.float32)))
        vv = np.concatenate((O.bf16_rn(v), np.zeros((pad,) + v.shape[1:], np.float32)))
        pool_k = kk.reshape(nblk, page, cfg.num_kv_heads, 128).transpose(0, 2, 1, 3)
        pool_v = vv.reshape(nblk, page, cfg.num_kv_heads, 128).transpose(0, 2, 1, 3)
        gather = np.full((1, cfg.num_kv_heads, cfg.max_visible), -1, np.int32)
        lens = np.zeros((1, cfg.num_kv_heads), np.int32)
        for kv in range(cfg.num_kv_heads):
            ids = G[f"{name}/ids/{row}/{kv}"]
            gather[0, kv, :len(ids)] = ids            # identity block table: slot == logical id
            lens[0, kv] = len(ids)
        out = O.gather_attention(O.bf16_rn(q)[None], pool_k, pool_v, gather, lens, np.array([0]), m["scaling"], "bf16")
        np.testing.assert_allclose(out[0], ref_out[row], atol=2e-2, rtol=2e-2)
