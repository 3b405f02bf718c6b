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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a checkout of the reference project")
    a = ap.parse_args()
    ix = tia(a.reference)
    make_quant(ix)
    make_tia_index(ix)
    make_paged_ops(a.reference)
    make_arch(a.reference)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
