"""Pin the CPU oracle against outputs of the reference's own PyTorch code
(fixtures made by tests/golden/make_golden.py)."""
import numpy as np
import torch

from conftest import golden
from oracle import loda_oracle as O


def test_quant4_bit_exact_bf16():
    g = golden("quant4.npz")
    x = O.bits_to_f32(g["x_bf16"])
    code, scale, zero, deq = O.quant4(x, "bf16")
    assert np.array_equal(O.bf16_bits(deq), g["y_bf16"])
    # the packed form (code, scale, zero) de-quantises to the same bits
    assert np.array_equal(O.bf16_bits(O.dequant4(code, scale, zero, "bf16")), g["y_bf16"])
    assert code.max() <= 15


def test_quant4_bit_exact_fp32():
    g = golden("quant4.npz")
    code, scale, zero, deq = O.quant4(g["x_fp32"], "fp32")
    assert np.array_equal(deq.view(np.uint32), g["y_fp32"].view(np.uint32))
    assert np.array_equal(O.dequant4(code, scale, zero, "fp32").view(np.uint32),
                          g["y_fp32"].view(np.uint32))


def _load(g, name, mode):
    a = g[f"{name}_{mode}"]
    return O.bits_to_f32(a) if mode == "bf16" else a


def test_page_minmax_and_tail_quant_match_tia_index():
    g = golden("tia_index.npz")
    length = int(g["length"])
    for mode in ("bf16", "fp32"):
        k = _load(g, "k", mode)
        cfg = O.SelectorConfig(num_q_heads=8, num_kv_heads=2, mode=mode)
        full = length // 16          # the reference zero-pads the ragged last block
        vmin, vmax, _ = O.page_stats(k[..., cfg.dims], length, 16, mode)
        assert np.array_equal(vmin[:full], _load(g, "kmin", mode)[:full][..., cfg.dims])
        assert np.array_equal(vmax[:full], _load(g, "kmax", mode)[:full][..., cfg.dims])
        # the ragged last block excludes padding instead of zero-filling it
        tail = k[full * 16:length][..., cfg.dims]
        assert np.array_equal(vmin[full], tail.min(axis=0))
        assert np.array_equal(vmax[full], tail.max(axis=0))
        idx = O.build_index(k, length, cfg)
        deq = O.dequant4(idx.code, idx.scale, idx.zero, mode)
        ref = _load(g, "kqat", mode)[..., cfg.dims]
        assert np.array_equal(deq.view(np.uint32), np.ascontiguousarray(ref).view(np.uint32))


def test_bound_score_matches_tia_compute_score():
    """Full-width min/max bound of the reference (tia_indexer.py:87-90) against
    the canonical-order dot of the oracle: equal up to fp32 re-association."""
    g = golden("tia_index.npz")
    length = int(g["length"])
    full = length // 16
    for mode, tol in (("fp32", 2e-5), ("bf16", 1.6e-2)):
        k, q = _load(g, "k", mode), _load(g, "q", mode)
        ref = _load(g, "coarse", mode)                    # [Hq, kt]
        vmin = np.stack([k[t * 16:(t + 1) * 16].min(axis=0) for t in range(full)])
        vmax = np.stack([k[t * 16:(t + 1) * 16].max(axis=0) for t in range(full)])
        qs = (q * np.float32(128 ** -0.5)).astype(np.float32)
        for h in range(q.shape[0]):
            kv = h // 4
            mm = (O._chunk_tree_dot(vmin[:, kv], np.minimum(qs[h], 0))
                  + O._chunk_tree_dot(vmax[:, kv], np.maximum(qs[h], 0)))
            np.testing.assert_allclose(O.act(mm, mode), ref[h, :full], rtol=tol, atol=tol)


def test_fine_score_matches_tia_compute_score():
    g = golden("tia_index.npz")
    k, q = g["k_fp32"], g["q_fp32"]
    cfg = O.SelectorConfig(num_q_heads=8, num_kv_heads=2, mode="fp32")
    idx = O.build_index(k, int(g["length"]), cfg)
    deq = O.dequant4(idx.code, idx.scale, idx.zero, "fp32")
    qs = (q * np.float32(128 ** -0.5)).astype(np.float32)[:, cfg.dims]
    for h in range(8):
        s = O._chain_dot(deq[:, h // 4], qs[h])
        np.testing.assert_allclose(s, g["fine_fp32"][h], rtol=2e-5, atol=2e-5)


def test_paged_write_and_gather_attention_match_reference_cpu_branch():
    g = golden("paged_ops.npz")
    pool_k = np.zeros_like(g["pool_k"])
    pool_v = np.zeros_like(g["pool_v"])
    O.paged_write_prefill(pool_k, pool_v, g["k"][0], g["v"][0], g["table"])
    O.paged_write_decode(pool_k, pool_v, g["kd"][:, :, 0], g["vd"][:, :, 0], g["slots"])
    assert np.array_equal(pool_k, g["pool_k"])
    assert np.array_equal(pool_v, g["pool_v"])
    out = O.gather_attention(g["q"], pool_k, pool_v, g["gather"], g["lens"], g["q2r"],
                             128 ** -0.5, "fp32")
    np.testing.assert_allclose(out, g["out"], rtol=1e-5, atol=1e-5)
    assert np.all(out[1] == 0)       # padded query row stays zero


def _arch_inputs(g, tag):
    length, seed = int(g[f"{tag}_length"]), int(g[f"{tag}_seed"])
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(1, 1, 32, 128, generator=gen)
    k = torch.randn(1, length, 8, 128, generator=gen)
    chk = np.array([k.double().sum().item(), q.double().sum().item()])
    assert np.allclose(chk, g[f"{tag}_checksum"], rtol=0, atol=1e-6), "torch CPU RNG changed"
    return q[0, 0].numpy(), k[0].numpy(), length


def test_l1_page_sets_match_archived_pytorch_pipeline():
    """The archived PyTorch near/far indexer and the oracle choose the same
    far and near pages (fp32, unrounded query as in that pipeline)."""
    g = golden("arch_tli.npz")
    for tag in ("a", "b"):
        q, k, length = _arch_inputs(g, tag)
        cfg = O.SelectorConfig(mode="fp32", q_round=False)
        sel = O.select_request(q, k, length, cfg, 128 ** -0.5)
        rg = sel.regions
        assert int(g[f"{tag}_far_width"]) == rg.near_blks - 1
        far_ref = np.sort(g[f"{tag}_far_idx"] + 1, axis=-1)
        near_ref = np.sort(g[f"{tag}_near_idx"] + rg.near_blks, axis=-1)
        assert np.array_equal(np.sort(sel.i_far, axis=-1), far_ref)
        assert np.array_equal(np.sort(sel.i_near, axis=-1), near_ref)


def test_final_mask_overlap_with_archived_pipeline():
    """Token sets: the probability-mean metric reproduces the archived mask
    almost exactly; the live grouped-logit metric is a different ranking."""
    g = golden("arch_tli.npz")
    q, k, length = _arch_inputs(g, "a")
    ref = np.unpackbits(g["a_mask"], axis=-1)[:, :length].astype(bool)
    jac = {}
    for metric in ("softmax_prob_mean", "grouped_logit"):
        cfg = O.SelectorConfig(mode="fp32", q_round=False, l2_metric=metric)
        sel = O.select_request(q, k, length, cfg, 128 ** -0.5)
        js = []
        for kv in range(8):
            m = np.zeros(length, bool)
            m[sel.logical[kv]] = True
            js.append((m & ref[kv]).sum() / (m | ref[kv]).sum())
            assert m[:4].all() and m[length - 128:].all()
        jac[metric] = float(np.mean(js))
    assert jac["softmax_prob_mean"] > 0.97
    assert jac["grouped_logit"] > 0.5
