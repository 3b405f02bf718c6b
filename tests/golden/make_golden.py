"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference checkout is available (it is pure Python on these
paths and runs on CPU):

    python tests/golden/make_golden.py --reference /path/to/two-level-attention

The script imports the reference's own PyTorch code — the TIA indexer
(sparse_attn/indexer/tia_indexer.py), the CPU branches of the paged write and
gather attention (sparse_attn/ops/paged_region_kernels.py), and the archived
PyTorch near/far pipeline (TLIIndexer, with its Triton switch forced off) —
runs them on seeded inputs and stores inputs (when small) and outputs as
compressed npz files.  Tests never import the reference; they only read these
files.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_REL = ("agent_doc/results/frozen_near_far_v1_16_independent005_20261030/"
            "ai_supervision/independent_final_20261030T0715/source/v1")


def bits(t):
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16)


def tia(reference, block=16):
    sys.path.insert(0, reference)
    from sparse_attn.indexer.tia_indexer import TIAIndexer
    from sparse_attn.ops.paged_region_kernels_nfa import nfa_args
    args = nfa_args("tail")
    args.tia_block_size = block
    return TIAIndexer(args)


def make_quant(ix):
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(96, 32, generator=g)
    x[0] = 0.75                       # constant row
    x[1] = 0.0
    x[2, :] = 1.0
    x[2, 5] = 1.0 + 2 ** -7           # range of one bf16 ulp
    x[3] *= 1e-6
    x[4] *= 300.0
    x[5, 7] = 40.0                    # outlier channel
    x[6] = torch.linspace(-3, 3, 32)
    xb = x.bfloat16()
    np.savez_compressed(
        os.path.join(HERE, "quant4.npz"),
        x_bf16=bits(xb), y_bf16=bits(ix.min_max_per_token_quant(xb)),
        x_fp32=x.numpy(), y_fp32=ix.min_max_per_token_quant(x).numpy())


def make_tia_index(ix):
    g = torch.Generator().manual_seed(77)
    length, hkv, hq = 150, 2, 8
    k = torch.randn(1, length, hkv, 128, generator=g)
    q = torch.randn(1, 1, hq, 128, generator=g)
    out = {}
    for name, dt in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        kk, qq = k.to(dt), q.to(dt)
        idx = ix.prepare_index(kk, torch.tensor([0, length]))
        sc = ix.compute_score(qq, torch.tensor([length - 1]), idx, 128 ** -0.5)
        conv = bits if dt == torch.bfloat16 else (lambda t: t.numpy())
        out[f"k_{name}"] = conv(kk[0])
        out[f"q_{name}"] = conv(qq[0, 0])
        out[f"kmin_{name}"] = conv(idx["k_min"][0])
        out[f"kmax_{name}"] = conv(idx["k_max"][0])
        out[f"kqat_{name}"] = conv(idx["k_qat"][0])
        out[f"coarse_{name}"] = conv(sc["score_coarse"][0, 0])
        out[f"fine_{name}"] = conv(sc["score_fine"][0, 0])
    np.savez_compressed(os.path.join(HERE, "tia_index.npz"), length=length, **out)


def make_paged_ops(reference):
    sys.path.insert(0, reference)
    from sparse_attn.ops import paged_region_kernels as gat
    from sparse_attn.cache.paged_region_cache import GraphReadyPagedRegionLayer
    from sparse_attn.policies.region_geometry import RegionGeometry
    g = torch.Generator().manual_seed(5)
    page, hkv, hq, d, pages = 16, 2, 8, 128, 12
    layer = GraphReadyPagedRegionLayer(
        geometry=RegionGeometry(page=page), max_physical_pages=pages,
        num_kv_heads=hkv, head_dim_k=d, head_dim_v=d, dtype=torch.float32, device="cpu")
    layer.kv_pool_k.zero_()
    layer.kv_pool_v.zero_()
    n = 70
    k = torch.randn(1, hkv, n, d, generator=g)
    v = torch.randn(1, hkv, n, d, generator=g)
    table = torch.tensor([7, 2, 9, 0, 4, pages, pages], dtype=torch.int32)
    gat.paged_write_prefill(layer, k, v, table)
    kd = torch.randn(2, hkv, 1, d, generator=g)
    vd = torch.randn(2, hkv, 1, d, generator=g)
    slots = torch.tensor([4 * page + 6, -1], dtype=torch.int32)      # token 70 and a PAD row
    gat.paged_write_decode(layer, kd, vd, slots)
    length = n + 1
    q = torch.randn(3, hq, d, generator=g)
    ids0 = torch.tensor(sorted(set(range(4)) | set(range(20, 40, 3)) | set(range(60, 71))))
    ids1 = torch.tensor(sorted(set(range(4)) | set(range(9, 55, 5)) | set(range(64, 71))))
    gather = torch.full((2, hkv, 32), -1, dtype=torch.int32)
    lens = torch.zeros((2, hkv), dtype=torch.int32)
    for kv, ids in enumerate((ids0, ids1)):
        slots_l = table[ids // page].long() * page + ids % page
        gather[0, kv, :len(ids)] = slots_l.int()
        lens[0, kv] = len(ids)
    gather[0, 1, 3] = -1                                              # a hole inside the list
    q2r = torch.tensor([0, -1, 0], dtype=torch.int32)
    out = gat.sparse_paged_attention_gather(layer, q, gather, lens, q2r, scale=d ** -0.5)
    np.savez_compressed(
        os.path.join(HERE, "paged_ops.npz"),
        k=k.numpy(), v=v.numpy(), table=table.numpy(), kd=kd.numpy(), vd=vd.numpy(),
        slots=slots.numpy(), pool_k=layer.kv_pool_k[:, 0].numpy(),
        pool_v=layer.kv_pool_v[:, 0].numpy(), q=q.numpy(), gather=gather.numpy(),
        lens=lens.numpy(), q2r=q2r.numpy(), out=out.numpy(), length=length)


def make_arch(reference):
    """L1 page sets and the final mask of the archived PyTorch near/far
    pipeline, fp32, for inputs that tests regenerate from the same seed."""
    arch = os.path.join(reference, ARCH_REL)
    for name in [m for m in sys.modules if m.startswith("sparse_attn")]:
        del sys.modules[name]
    sys.path.insert(0, arch)
    import sparse_attn.indexer.tli_indexer as tli
    from sparse_attn.arguments import add_sparse_attn_args
    tli._HAS_TRITON = False
    p = argparse.ArgumentParser()
    add_sparse_attn_args(p)
    flags = ("--method tli --tli_far_method minmax --tli_near_method avg --tli_near_pages 32 "
             "--tli_near_tokens off --tli_near_len 4096 --tli_subspace tail "
             "--tia_level2_cmp_ratio 4 --tli_sink_tokens 4 --tli_swa_size 128 "
             "--tia_level1_topk 128 --tia_level2_topk 1024 --tli_enable_layer_skip false "
             "--tli_l2_quant true --tia_block_size 16 --tli_far_skip_backend legacy "
             "--tli_far_skip_cache retain").split()
    ix = tli.TLIIndexer(p.parse_args(flags))
    out = {}
    for tag, length, seed in (("a", 12289, 0), ("b", 9000, 3)):
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(1, 1, 32, 128, generator=g)
        k = torch.randn(1, length, 8, 128, generator=g)
        calls = []
        orig = torch.topk

        def rec(x, k, dim=-1, **kw):
            r = orig(x, k, dim=dim, **kw)
            calls.append((tuple(x.shape), int(k), r.indices.clone()))
            return r
        torch.topk = rec
        try:
            mask, _ = ix.prepare_mask(q, torch.tensor([length - 1]), k, torch.tensor([0, length]))
        finally:
            torch.topk = orig
        far = [c for c in calls if c[1] == 96][0]
        near = [c for c in calls if c[1] == 32][0]
        out[f"{tag}_length"] = length
        out[f"{tag}_seed"] = seed
        out[f"{tag}_far_width"] = far[0][-1]
        out[f"{tag}_near_width"] = near[0][-1]
        out[f"{tag}_far_idx"] = far[2][0, 0].numpy().astype(np.int32)     # relative to the far pool
        out[f"{tag}_near_idx"] = near[2][0, 0].numpy().astype(np.int32)   # relative to the near pool
        out[f"{tag}_mask"] = np.packbits(mask[0, 0].numpy(), axis=-1)
        out[f"{tag}_checksum"] = np.array([k.double().sum().item(), q.double().sum().item()])
        ix.clear()
    np.savez_compressed(os.path.join(HERE, "arch_tli.npz"), **out)


def make_tls(reference):
    """Outputs of the PyTorch reference functions the reference ships beside its tls_attn operators
    (tls_attn/ops: MHAStoreKIndexReference mha_store_k_index.py:188-310, ref_indexer_topk
    mha_indexer_level1.py:252-276 and mha_indexer_level2.py:293-402, ref_attn sparse_mha.py:199-232),
    with their inputs.  The two ref_indexer_topk functions are called one batch row (and one KV head)
    at a time: written for the single-row, single-head shapes of the reference's own checks, they
    apply row i's sliding mask to every row and the last head's sliding entries only."""
    sys.path.insert(0, reference)
    from tls_attn.ops.mha_indexer_level1 import ref_indexer_topk as ref_l1
    from tls_attn.ops.mha_indexer_level2 import ref_indexer_topk as ref_l2
    from tls_attn.ops.mha_store_k_index import MHAStoreKIndexReference as RefIndex
    from tls_attn.ops.sparse_mha import ref_attn
    out = {}
    # ---- store K index: prefill, then decode ----
    g = torch.Generator().manual_seed(1)
    max_b, max_s, hkv, d, block, cmp, b, s = 4, 256, 2, 128, 16, 4, 3, 200
    k = torch.randn(b, s, hkv, d, generator=g).bfloat16()
    offsets = torch.tensor([0, 9, 150], dtype=torch.int32)
    l1min = torch.zeros(max_b, max_s // block, hkv, d, dtype=torch.bfloat16)
    l1max = torch.zeros_like(l1min)
    l2k = torch.zeros(max_b, max_s, hkv, d // cmp, dtype=torch.bfloat16)
    RefIndex.prefill_forward(k, offsets, l1min, l1max, l2k, block, cmp)
    out.update(ix_k=bits(k), ix_offsets=offsets.numpy(), ix_l1min=bits(l1min), ix_l1max=bits(l1max), ix_l2k=bits(l2k))
    kc = torch.randn(max_b, max_s, hkv, d, generator=g).bfloat16()
    lengths = torch.tensor([208, 37, 51], dtype=torch.int32)
    RefIndex.decode_forward(kc, lengths, l1min, l1max, l2k, block, cmp)
    out.update(ix_kc=bits(kc), ix_lengths=lengths.numpy(), ix_l1min_dec=bits(l1min), ix_l1max_dec=bits(l1max),
               ix_l2k_dec=bits(l2k), ix_shape=np.array([max_b, max_s, hkv, d, block, cmp]))
    # ---- level 1 ----
    g = torch.Generator().manual_seed(2)
    b, hq, hkv, d, topk, sliding, nblk = 3, 8, 2, 128, 16, 3, 160
    lengths = torch.tensor([150, 12, 90, 4], dtype=torch.int32)
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16()
    kmin = (torch.randn(4, nblk, hkv, d, generator=g) - 1).bfloat16()
    kmax = (torch.randn(4, nblk, hkv, d, generator=g) + 1).bfloat16()
    scores = torch.full((b, hkv, nblk), float("-inf"))
    tk = torch.full((b, hkv, topk), -1, dtype=torch.int64)
    for i in range(b):
        n = int(lengths[i])
        sc, _, ti = ref_l1(q[i:i + 1, 0].float(), kmin[i:i + 1, :n].float(), kmax[i:i + 1, :n].float(),
                           lengths[i:i + 1], min(topk, n), sliding)
        scores[i, :, :n] = sc[0]
        valid = torch.isfinite(sc[0].gather(-1, ti[0]))
        tk[i, :, :ti.shape[-1]] = torch.where(valid, ti[0], -1)
    out.update(l1_q=bits(q), l1_kmin=bits(kmin), l1_kmax=bits(kmax), l1_lengths=lengths.numpy(),
               l1_scores=scores.numpy(), l1_topk=tk.numpy().astype(np.int32),
               l1_shape=np.array([b, hq, hkv, d, topk, sliding, nblk]))
    # ---- level 2 ----
    g = torch.Generator().manual_seed(4)
    b, hq, hkv, dsub, block, k1, k2, sliding, s = 2, 8, 2, 32, 16, 6, 64, 2, 512
    gs = hq // hkv
    lengths = torch.tensor([500, 333, 77], dtype=torch.int32)
    q = torch.randn(b, 1, hq, dsub, generator=g).bfloat16()
    k = torch.randn(3, s, hkv, dsub, generator=g).bfloat16()
    bi = torch.tensor([[[3, 0, 7, -1, 12, 20], [1, 2, -1, -1, 9, 4]],
                       [[5, 6, 0, 2, -1, 10], [-1, -1, -1, -1, -1, -1]]], dtype=torch.int32)
    width = (k1 + sliding) * block
    sc_all = torch.full((b, hkv, width), float("-inf"))
    ix_all = torch.full((b, hkv, width), -1, dtype=torch.int64)
    tk_all = torch.full((b, hkv, k2), -1, dtype=torch.int64)
    for i in range(b):
        for h in range(hkv):
            sc, ix, ts, ti = ref_l2(q[i:i + 1, 0, h * gs:(h + 1) * gs].float(), k[i:i + 1, :, h:h + 1].float(),
                                    bi[i:i + 1, h:h + 1], lengths[i:i + 1], block, sliding, k2)
            sc_all[i, h], ix_all[i, h] = sc[0, 0], ix[0, 0]
            tk_all[i, h] = torch.where(torch.isinf(ts[0, 0]) & (ts[0, 0] < 0), -1, ti[0, 0])
    out.update(l2_q=bits(q), l2_k=bits(k), l2_bi=bi.numpy(), l2_lengths=lengths.numpy(), l2_scores=sc_all.numpy(),
               l2_indices=ix_all.numpy().astype(np.int32), l2_topk=tk_all.numpy().astype(np.int32),
               l2_shape=np.array([b, hq, hkv, dsub, block, k1, k2, sliding, s]))
    # ---- sparse attention over chosen tokens ----
    g = torch.Generator().manual_seed(6)
    b, s, hq, hkv, d, topk = 2, 300, 8, 2, 128, 96
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16()
    k = torch.randn(b, s, hkv, d, generator=g).bfloat16()
    v = torch.randn(b, s, hkv, d, generator=g).bfloat16()
    idx = torch.stack([torch.stack([torch.randperm(s, generator=g)[:topk].sort().values for _ in range(hkv)])
                       for _ in range(b)]).int()
    idx[0, 1, 10:40] = -1
    o = ref_attn(q[:, 0].float(), k.float(), v.float(), idx.long())
    out.update(at_q=bits(q), at_k=bits(k), at_v=bits(v), at_idx=idx.numpy(), at_out=o.numpy())
    np.savez_compressed(os.path.join(HERE, "tls_ref.npz"), **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a checkout of the reference project")
    ap.add_argument("--only", default=None, help="tls: regenerate tls_ref.npz alone")
    a = ap.parse_args()
    if a.only == "tls":
        make_tls(a.reference)
        return
    ix = tia(a.reference)
    make_quant(ix)
    make_tia_index(ix)
    make_paged_ops(a.reference)
    make_tls(a.reference)
    make_arch(a.reference)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
