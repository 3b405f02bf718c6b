"""GPU tests of the prototype chain on a contiguous KV cache (tls_attn.ops): store KV,
store K index, level-1 and level-2 indexers, then sparse attention over the chosen tokens.
Each operator is compared with a plain PyTorch statement of the reference operator's
semantics (the reference states them in its ``*Reference`` classes and ``ref_indexer_topk``
functions); copies and min / max are exact, scores within fp32 re-association."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from helpers import mod
    return mod("tls_attn.ops")


def test_store_kv_prefill_and_decode_are_exact_copies():
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    max_b, max_s, hkv, dk, dv, b, s = 5, 300, 4, 128, 64, 3, 260
    st = ops.MHAStoreKVInterface(max_b, max_s, hkv, dk, dv)
    k = torch.randn(b, s, hkv, dk, generator=g).bfloat16().to(DEV)
    v = torch.randn(b, s, hkv, dv, generator=g).bfloat16().to(DEV)
    offsets = torch.tensor([0, 17, 259], dtype=torch.int32, device=DEV)
    kc = torch.zeros(max_b, max_s, hkv, dk, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros(max_b, max_s, hkv, dv, dtype=torch.bfloat16, device=DEV)
    st.prefill_forward(k, v, offsets, kc, vc)
    kr, vr = torch.zeros_like(kc), torch.zeros_like(vc)
    for i in range(b):
        o = int(offsets[i])
        kr[i, :s - o] = k[i, o:]
        vr[i, :s - o] = v[i, o:]
    assert torch.equal(kc, kr) and torch.equal(vc, vr)
    lengths = torch.tensor([261, 5, 300], dtype=torch.int32, device=DEV)
    k1 = torch.randn(b, 1, hkv, dk, generator=g).bfloat16().to(DEV)
    v1 = torch.randn(b, 1, hkv, dv, generator=g).bfloat16().to(DEV)
    st.decode_forward(k1, v1, lengths, kc, vc)
    for i in range(b):
        kr[i, int(lengths[i]) - 1] = k1[i, 0]
        vr[i, int(lengths[i]) - 1] = v1[i, 0]
    assert torch.equal(kc, kr) and torch.equal(vc, vr)


def _index_reference(k_rows, block, cmp):
    """k_rows [n, Hkv, D] -> (min, max [ceil(n / block), Hkv, D] with zero padding, tail dims [n, Hkv, D / cmp])."""
    n, hkv, d = k_rows.shape
    nb = (n + block - 1) // block
    pad = torch.zeros(nb * block, hkv, d, dtype=k_rows.dtype, device=k_rows.device)
    pad[:n] = k_rows
    blk = pad.view(nb, block, hkv, d).float()
    hc = d // 2 // cmp
    tail = torch.cat([k_rows[..., d // 2 - hc:d // 2], k_rows[..., d - hc:]], dim=-1)
    return blk.amin(1).to(k_rows.dtype), blk.amax(1).to(k_rows.dtype), tail


def test_store_k_index_prefill_then_decode_matches_the_block_statistics():
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    max_b, max_s, hkv, d, block, cmp, b, s = 4, 256, 2, 128, 16, 4, 3, 200
    ix = ops.MHAStoreKIndexInterface(max_b, max_s, hkv, d, block, cmp)
    k = torch.randn(b, s, hkv, d, generator=g).bfloat16().to(DEV)
    offsets = torch.tensor([0, 9, 150], dtype=torch.int32, device=DEV)
    l1min = torch.zeros(max_b, max_s // block, hkv, d, dtype=torch.bfloat16, device=DEV)
    l1max = torch.zeros_like(l1min)
    l2k = torch.zeros(max_b, max_s, hkv, d // cmp, dtype=torch.bfloat16, device=DEV)
    ix.prefill_forward(k, offsets, l1min, l1max, l2k)
    for i in range(b):
        rows = k[i, int(offsets[i]):]
        mn, mx, tail = _index_reference(rows, block, cmp)
        nb = mn.shape[0]
        assert torch.equal(l1min[i, :nb], mn) and torch.equal(l1max[i, :nb], mx)
        assert torch.equal(l2k[i, :rows.shape[0]], tail)
        assert not l1min[i, nb:].any() and not l2k[i, rows.shape[0]:].any()
    # decode: the cache already holds the new token; row 0 completes a block, row 1 does not
    kc = torch.randn(max_b, max_s, hkv, d, generator=g).bfloat16().to(DEV)
    lengths = torch.tensor([208, 37, 51], dtype=torch.int32, device=DEV)
    before_min = l1min.clone()
    ix.decode_forward(kc, lengths, l1min, l1max, l2k)
    hc = d // 2 // cmp
    for i in range(b):
        idx = int(lengths[i]) - 1
        want = torch.cat([kc[i, idx, :, d // 2 - hc:d // 2], kc[i, idx, :, d - hc:]], dim=-1)
        assert torch.equal(l2k[i, idx], want)
        j = idx // block
        if (idx + 1) % block == 0:
            blk = kc[i, j * block:(j + 1) * block].float()
            assert torch.equal(l1min[i, j], blk.amin(0).bfloat16()) and torch.equal(l1max[i, j], blk.amax(0).bfloat16())
        else:
            assert torch.equal(l1min[i, j], before_min[i, j])


def _level1_reference(q, kmin, kmax, lengths, sliding, scaling):
    """fp64 statement: sum over the group of max(q s, 0) . kmax + min(q s, 0) . kmin, q s rounded to bf16."""
    b, _, hq, d = q.shape
    hkv = kmin.shape[2]
    g = hq // hkv
    qs = (q[:, 0].float() * scaling).bfloat16().double()                   # [B, Hq, D]
    qp, qn = qs.clamp(min=0), qs.clamp(max=0)
    out = torch.full((b, hkv, int(lengths.max())), float("-inf"), dtype=torch.float64)
    for i in range(b):
        n = int(lengths[i]) - sliding
        if n <= 0:
            continue
        for h in range(hkv):
            s = torch.zeros(n, dtype=torch.float64)
            for j in range(g):
                s += kmax[i, :n, h].double() @ qp[i, h * g + j] + kmin[i, :n, h].double() @ qn[i, h * g + j]
            out[i, h, :n] = s
    return out


def test_level1_scores_and_topk_blocks():
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    b, hq, hkv, d, topk, sliding = 3, 8, 2, 128, 16, 3
    lengths = torch.tensor([700, 12, 90, 4], dtype=torch.int32)           # blocks; [maxB]
    nblk = 704
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16()
    kmin = (torch.randn(4, nblk, hkv, d, generator=g) - 1).bfloat16()
    kmax = (torch.randn(4, nblk, hkv, d, generator=g) + 1).bfloat16()
    l1 = ops.MHAIndexerLevel1Interface(hq, hkv, d, topk, sliding)
    scores, tk_s, tk_i = l1.forward(q.to(DEV), kmin.to(DEV), kmax.to(DEV), lengths.to(DEV))
    want = _level1_reference(q, kmin, kmax, lengths[:b], sliding, d ** -0.5)
    width = int(lengths.max())
    assert scores.shape == (b, hkv, width)
    got = scores.double().cpu()
    finite = torch.isfinite(want[..., :width])
    assert torch.equal(torch.isfinite(got[:b]), finite)
    torch.testing.assert_close(got[:b][finite], want[..., :width][finite], atol=2e-3, rtol=1e-4)
    # top-k of the kernel's own scores: exact order (score descending, lower block first), -1 where missing
    for i in range(b):
        for h in range(hkv):
            row = scores[i, h].cpu()
            valid = torch.nonzero(torch.isfinite(row)).flatten()
            order = sorted(valid.tolist(), key=lambda t: (-float(row[t]), t))[:topk]
            want_i = order + [-1] * (topk - len(order))
            assert tk_i[i, h].cpu().tolist() == want_i
            want_s = [float(row[t]) for t in order] + [float("-inf")] * (topk - len(order))
            assert tk_s[i, h].cpu().tolist() == want_s


def test_level2_scores_topk_tokens_and_the_chain_into_sparse_attention():
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    b, hq, hkv, dsub, block, k1, k2, sliding = 2, 8, 2, 32, 16, 6, 64, 2
    s = 512
    lengths = torch.tensor([500, 333, 77], dtype=torch.int32)              # tokens; [maxB]
    q = torch.randn(b, 1, hq, dsub, generator=g).bfloat16()
    k = torch.randn(3, s, hkv, dsub, generator=g).bfloat16()
    bi = torch.tensor([[[3, 0, 7, -1, 12, 20], [1, 2, -1, -1, 9, 4]],
                       [[5, 6, 0, 2, -1, 10], [-1, -1, -1, -1, -1, -1]]], dtype=torch.int32)
    l2 = ops.MHAIndexerLevel2Interface(hq, hkv, dsub, k1, k2, block, sliding)
    scores, indices, tk_s, tk_i = l2.forward(q.to(DEV), k.to(DEV), bi.to(DEV), lengths.to(DEV))
    gsz = hq // hkv
    qs = (q[:, 0].float() * dsub ** -0.5).bfloat16().double()
    for i in range(b):
        for h in range(hkv):
            logits = torch.full((gsz, k1 * block), float("-inf"), dtype=torch.float64)
            want_idx = torch.full((k1 * block,), -1, dtype=torch.int64)
            for c in range(k1):
                blk = int(bi[i, h, c])
                if blk < 0:
                    continue
                kk = k[i, blk * block:(blk + 1) * block, h].double()
                logits[:, c * block:(c + 1) * block] = qs[i, h * gsz:(h + 1) * gsz] @ kk.T
                want_idx[c * block:(c + 1) * block] = torch.arange(blk * block, (blk + 1) * block)
            assert indices[i, h].cpu().tolist() == want_idx.tolist()
            got = scores[i, h].double().cpu()
            if torch.isfinite(logits).any():
                want = (logits - logits.max()).exp().sum(0)
                want[want_idx < 0] = float("-inf")
                fin = torch.isfinite(want)
                assert torch.equal(torch.isfinite(got), fin)
                torch.testing.assert_close(got[fin], want[fin], atol=1e-5, rtol=2e-4)
            else:
                assert torch.isinf(got).all() and (got < 0).all()
            # top-k: the sliding blocks first (+inf, ascending tokens), then the kernel's own scores in order
            n = int(lengths[i])
            start = ((n - 1) // block - sliding + 1) * block
            forced = [t for t in range(max(start, 0), min(start + sliding * block, n))][:k2]
            row = scores[i, h].cpu()
            cand = torch.nonzero(torch.isfinite(row)).flatten().tolist()
            order = sorted(cand, key=lambda t: (-float(row[t]), t))[:k2 - len(forced)]
            want_i = forced + [int(want_idx[t]) for t in order]
            want_i += [-1] * (k2 - len(want_i))
            assert tk_i[i, h].cpu().tolist() == want_i
            assert all(x == float("inf") for x in tk_s[i, h, :len(forced)].cpu().tolist())
    # the chosen tokens feed the sparse attention unchanged (holes are skipped there)
    v = torch.randn(3, s, hkv, 128, generator=g).bfloat16()
    kf = torch.randn(3, s, hkv, 128, generator=g).bfloat16()
    qf = torch.randn(b, 1, hq, 128, generator=g).bfloat16()
    att = ops.SparseMHAInterface(hq, hkv, 128, 128, k2)
    out = att.forward(qf.to(DEV), kf.to(DEV), v.to(DEV), tk_i)
    for i in range(b):
        for h in range(hkv):
            t = tk_i[i, h].cpu()
            t = t[t >= 0].long()
            p = torch.softmax(qf[i, 0, h * gsz:(h + 1) * gsz].double() @ kf[i, t, h].double().T * 128 ** -0.5, dim=-1)
            torch.testing.assert_close(out[i, 0, h * gsz:(h + 1) * gsz].double().cpu(), p @ v[i, t, h].double(),
                                       atol=2e-2, rtol=2e-2)


# ---------------------------------------------------------------------------
# The same operators against outputs of the reference's own PyTorch reference functions
# (tests/golden/tls_ref.npz, made by tests/golden/make_golden.py from MHAStoreKIndexReference,
# the two ref_indexer_topk and ref_attn of tls_attn/ops).
# ---------------------------------------------------------------------------
def _bf16(g, name):
    from oracle import loda_oracle as O
    return torch.from_numpy(O.bits_to_f32(g[name])).bfloat16()


def _same_topk_up_to_ties(got, want, score_of, tol):
    """Two top-k id sets agree except where the scores around the cut differ by less than tol."""
    got, want = set(int(x) for x in got if x >= 0), set(int(x) for x in want if x >= 0)
    if got == want:
        return True
    if len(got) != len(want):
        return False
    cut = min(score_of(t) for t in want)
    return all(abs(score_of(t) - cut) < tol for t in got ^ want)


def test_store_k_index_equals_the_reference_class_outputs():
    from conftest import golden
    ops = _ops()
    g = golden("tls_ref.npz")
    max_b, max_s, hkv, d, block, cmp = (int(x) for x in g["ix_shape"])
    ix = ops.MHAStoreKIndexInterface(max_b, max_s, hkv, d, block, cmp)
    l1min = torch.zeros(max_b, max_s // block, hkv, d, dtype=torch.bfloat16, device=DEV)
    l1max = torch.zeros_like(l1min)
    l2k = torch.zeros(max_b, max_s, hkv, d // cmp, dtype=torch.bfloat16, device=DEV)
    ix.prefill_forward(_bf16(g, "ix_k").to(DEV), torch.from_numpy(g["ix_offsets"]).to(DEV), l1min, l1max, l2k)
    assert torch.equal(l1min.cpu(), _bf16(g, "ix_l1min")) and torch.equal(l1max.cpu(), _bf16(g, "ix_l1max"))
    assert torch.equal(l2k.cpu(), _bf16(g, "ix_l2k"))
    ix.decode_forward(_bf16(g, "ix_kc").to(DEV), torch.from_numpy(g["ix_lengths"]).to(DEV), l1min, l1max, l2k)
    assert torch.equal(l1min.cpu(), _bf16(g, "ix_l1min_dec")) and torch.equal(l1max.cpu(), _bf16(g, "ix_l1max_dec"))
    assert torch.equal(l2k.cpu(), _bf16(g, "ix_l2k_dec"))


def test_level1_equals_ref_indexer_topk_outputs():
    from conftest import golden
    ops = _ops()
    g = golden("tls_ref.npz")
    b, hq, hkv, d, topk, sliding, nblk = (int(x) for x in g["l1_shape"])
    lengths = torch.from_numpy(g["l1_lengths"])
    l1 = ops.MHAIndexerLevel1Interface(hq, hkv, d, topk, sliding)
    scores, _, tk_i = l1.forward(_bf16(g, "l1_q").to(DEV), _bf16(g, "l1_kmin").to(DEV), _bf16(g, "l1_kmax").to(DEV),
                                 lengths.to(DEV))
    want = torch.from_numpy(g["l1_scores"])[..., :scores.shape[-1]]
    got = scores[:b].float().cpu()
    fin = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got), fin)
    # the reference function keeps q * scale in fp32, the operator rounds it to bf16 like the reference's kernel
    torch.testing.assert_close(got[fin], want[fin], atol=5e-2, rtol=5e-3)
    for i in range(b):
        for h in range(hkv):
            assert _same_topk_up_to_ties(tk_i[i, h].cpu().tolist(), g["l1_topk"][i, h].tolist(),
                                         lambda t: float(want[i, h, t]), 0.1), (i, h)


def test_level2_equals_ref_indexer_topk_outputs():
    from conftest import golden
    ops = _ops()
    g = golden("tls_ref.npz")
    b, hq, hkv, dsub, block, k1, k2, sliding, s = (int(x) for x in g["l2_shape"])
    l2 = ops.MHAIndexerLevel2Interface(hq, hkv, dsub, k1, k2, block, sliding)
    scores, indices, _, tk_i = l2.forward(_bf16(g, "l2_q").to(DEV), _bf16(g, "l2_k").to(DEV),
                                          torch.from_numpy(g["l2_bi"]).to(DEV), torch.from_numpy(g["l2_lengths"]).to(DEV))
    n = k1 * block
    want_s, want_i = torch.from_numpy(g["l2_scores"])[..., :n], torch.from_numpy(g["l2_indices"])[..., :n]
    assert torch.equal(indices[:b].cpu().int(), want_i)
    got = scores[:b].float().cpu()
    # the reference function leaves 0 (a hole beside scored blocks) or NaN (a row of holes only) at the holes,
    # the operator -inf: compare where a token stands
    fin = torch.isfinite(want_s) & (want_i >= 0)
    assert torch.equal(torch.isfinite(got), fin)
    torch.testing.assert_close(got[fin], want_s[fin], atol=1e-4, rtol=3e-2)
    full_s, full_i = torch.from_numpy(g["l2_scores"]), torch.from_numpy(g["l2_indices"])
    for i in range(b):
        for h in range(hkv):
            if torch.isnan(full_s[i, h]).any():
                continue      # a row of holes only: the reference function ranks its NaN scores above the sliding tokens
            score_of = {int(t): float(sc) for t, sc in zip(full_i[i, h].tolist(), full_s[i, h].tolist()) if t >= 0}
            assert _same_topk_up_to_ties(tk_i[i, h].cpu().tolist(), g["l2_topk"][i, h].tolist(),
                                         lambda t: min(score_of.get(t, -1e30), 1e30), 0.05), (i, h)


def test_sparse_mha_equals_ref_attn_output():
    from conftest import golden
    ops = _ops()
    g = golden("tls_ref.npz")
    q, k, v = _bf16(g, "at_q"), _bf16(g, "at_k"), _bf16(g, "at_v")
    idx = torch.from_numpy(g["at_idx"])
    att = ops.SparseMHAInterface(q.shape[2], k.shape[2], q.shape[3], v.shape[3], idx.shape[-1])
    out = att.forward(q.to(DEV), k.to(DEV), v.to(DEV), idx.to(DEV))
    torch.testing.assert_close(out[:, 0].float().cpu(), torch.from_numpy(g["at_out"]), atol=2e-2, rtol=2e-2)
