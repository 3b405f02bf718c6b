"""Golden vectors from the reference's PRODUCTION selector (Triton, GPU only).

The reference's production path — select_topk_for_layer_batched
(sparse_attn/indexer/nfa_layer_batch_selector.py:2649) followed by
sparse_paged_attention_gather (sparse_attn/ops/paged_region_kernels.py:800) — only exists as
Triton kernels, so its outputs have to be produced on a GPU.  Two steps:

    python tests/golden/make_golden_gpu.py --install --reference /path/to/two-level-attention
        packages the reference's two Python packages (sparse_attn, tls_attn), unmodified, into
        baseline/_ref with pip (the project itself declares no package, so a three-line setup.py
        is written next to a temporary copy); baseline/_ref is not tracked by git.

    python tests/golden/make_golden_gpu.py --out <dir>/ref_selector.npz             (on a GPU)
        imports the reference from baseline/_ref, builds its GraphReadyPagedRegionCache, runs the
        selector and the gather attention on seeded inputs and stores inputs (as seeds and
        parameters) and outputs.  The resulting file is committed as tests/golden/ref_selector.npz.

Inputs.  "exact" cases draw keys and queries from small integers, so that every dot product of the
selector is exact in fp32 whatever the summation order, and every bf16 rounding acts on an exact
value: the CPU oracle (with l2_quant=False: the reference scores level 2 on the raw keys) must
reproduce the reference's token lists bit for bit, ties, quota, hole fill, bypass pages, region
skipping and union included.  "normal" cases use N(0,1) inputs; there the reference's reduction
order (left to the Triton compiler) may move a score by an ulp, so they are compared as set overlap.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
import traceback
from types import SimpleNamespace

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

# (name, kind, page, lengths, skip states per request, selector settings)
BASE = dict(k1=32, near_pages=8, k2=256, sink=4, window=64, near_len=1024, near_tokens="off",
            far_method="minmax", near_method="avg", hkv=2, group=4)
PROD = dict(k1=128, near_pages=32, k2=1024, sink=4, window=128, near_len=4096, near_tokens="off",
            far_method="minmax", near_method="avg", hkv=2, group=4)
NS = (False, False)
CASES = [
    ("exact_p64_small", "exact", 64, [300, 449, 1500], [NS] * 3, dict(BASE, k1=4, near_pages=2, k2=128, near_len=128)),
    ("exact_p16_small", "exact", 16, [300, 77, 1003], [NS] * 3, dict(BASE, k1=8, near_pages=4, k2=128, near_len=256)),
    ("exact_p16_mid", "exact", 16, [4241, 2500, 4229], [NS] * 3, BASE),
    ("exact_p64_mid", "exact", 64, [4241, 9000], [NS] * 2, BASE),
    ("exact_p16_skip", "exact", 16, [4241, 4242, 4300, 4400], [NS, (True, False), (False, True), (True, True)], BASE),
    ("exact_p64_skipfar", "exact", 64, [5000, 3000], [(True, False)] * 2, BASE),
    ("exact_p64_skipnear", "exact", 64, [5000, 3000], [(False, True)] * 2, BASE),
    ("exact_p16_skipboth", "exact", 16, [5000, 3000], [(True, True)] * 2, BASE),
    ("exact_p16_quota16", "exact", 16, [4241, 2500], [NS] * 2, dict(BASE, near_tokens=48)),
    ("exact_p16_quota_skip", "exact", 16, [4241, 4242, 4300, 4400],
     [NS, (True, False), (False, True), (True, True)], dict(BASE, near_tokens=32)),
    ("exact_p16_faravg", "exact", 16, [4241, 2500], [NS] * 2, dict(BASE, far_method="avg")),
    ("exact_p16_nearmm", "exact", 16, [4241, 2500], [NS] * 2, dict(BASE, near_method="minmax")),
    ("exact_p16_prod", "exact", 16, [20000, 6000], [NS] * 2, PROD),
    ("exact_p64_prod", "exact", 64, [20000], [NS], PROD),
    ("normal_p16_prod", "normal", 16, [20000, 9000], [NS] * 2, PROD),
    ("normal_p64_prod", "normal", 64, [20000, 9000], [NS] * 2, PROD),
    ("normal_p16_top2", "normal", 16, [6000], [NS], dict(BASE, far_method="avg_top2")),
]
D = 128


def install(reference):
    tmp = tempfile.mkdtemp(prefix="ref_pkg_")
    try:
        for pkg in ("sparse_attn", "tls_attn"):
            shutil.copytree(os.path.join(reference, pkg), os.path.join(tmp, pkg))
        with open(os.path.join(tmp, "setup.py"), "w") as f:
            f.write("from setuptools import setup, find_namespace_packages\n"
                    "setup(name='two-level-attention-reference', version='0', packages=find_namespace_packages(include=['sparse_attn*', 'tls_attn*']))\n")
        if os.path.isdir(REF_DIR):
            shutil.rmtree(REF_DIR)
        os.makedirs(REF_DIR, exist_ok=True)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", REF_DIR, tmp]
        res = subprocess.run(cmd, capture_output=True, text=True)
        print(res.stdout[-2000:], res.stderr[-2000:])
        return res.returncode
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def case_inputs(name, kind, lengths, hkv, group):
    """Seeded inputs of a case: per request the prompt keys / values [1, Hkv, L - 1, D], the decoded
    token's key / value, and the query [Hq, D].  The seed is derived from the case name, so a test
    regenerates exactly these arrays."""
    seed = int.from_bytes(name.encode(), "little") % (2 ** 31)
    rng = np.random.default_rng(seed)
    out = []
    for length in lengths:
        if kind == "exact":
            k = rng.integers(-2, 3, (length, hkv, D)).astype(np.float32)
            # a few pages of equal keys: whole-page ties at level 1 and runs of tied tokens at level 2
            k[length // 3:length // 3 + 200] = k[length // 3]
            q = rng.integers(-3, 4, (hkv * group, D)).astype(np.float32)
        else:
            k = rng.standard_normal((length, hkv, D)).astype(np.float32)
            q = rng.standard_normal((hkv * group, D)).astype(np.float32)
        v = rng.standard_normal((length, hkv, D)).astype(np.float32)
        out.append((k, v, q))
    return out


def run_case(torch, mods, name, kind, page, lengths, skips, cfg, log):
    (GraphReadyPagedRegionCache, NFAIndexer, select_topk, gather_attn, nfa_args, RegionGeometry) = mods
    dev = torch.device("cuda")
    hkv, group = cfg["hkv"], cfg["group"]
    hq = hkv * group
    args = nfa_args("tail")
    args.tia_block_size = page
    args.tia_level1_topk, args.tia_level2_topk = cfg["k1"], cfg["k2"]
    args.nfa_near_pages, args.nfa_near_tokens, args.nfa_near_len = cfg["near_pages"], cfg["near_tokens"], cfg["near_len"]
    args.nfa_sink_tokens, args.nfa_swa_size = cfg["sink"], cfg["window"]
    args.nfa_far_method, args.nfa_near_method = cfg["far_method"], cfg["near_method"]
    indexer = NFAIndexer(args)
    geometry = RegionGeometry(sink=cfg["sink"], near=cfg["near_len"], window=cfg["window"], page=page, max_new_tokens=8)
    max_blocks = (max(lengths) + 8 + page - 1) // page + 2
    pages = sum((n + 8 + page - 1) // page for n in lengths) + 8
    nreq = len(lengths)
    cache = GraphReadyPagedRegionCache(
        1, geometry, max_requests=nreq + 2, max_physical_pages=pages, max_blocks=max_blocks,
        max_visible_len=cfg["k2"], max_query_tokens=nreq, num_kv_heads=hkv, num_query_heads=hq,
        head_dim_k=D, head_dim_v=D, dtype=torch.bfloat16, device=dev)
    data = case_inputs(name, kind, lengths, hkv, group)
    req_ids = [i + 1 for i in range(nreq)]          # non-contiguous from slot 0 on purpose
    for rid, length, (k, v, _), (sf, sn) in zip(req_ids, lengths, data, skips):
        cache.add_request(rid)
        kk = torch.from_numpy(k[:length - 1]).permute(1, 0, 2)[None].to(dev).to(torch.bfloat16)
        vv = torch.from_numpy(v[:length - 1]).permute(1, 0, 2)[None].to(dev).to(torch.bfloat16)
        cache.write_prefill(0, rid, kk, vv)
        cache.freeze(rid, [sf], [sn])
    cache.new_step(req_ids)
    cache.plan_common(req_ids)
    k_new = torch.stack([torch.from_numpy(k[length - 1]) for (k, _, _), length in zip(data, lengths)])[:, :, None]
    v_new = torch.stack([torch.from_numpy(v[length - 1]) for (_, v, _), length in zip(data, lengths)])[:, :, None]
    k_new, v_new = k_new.to(dev).to(torch.bfloat16), v_new.to(dev).to(torch.bfloat16)
    cache.write_decode(0, k_new, v_new, cache.slot_mapping_for_layer(0)[:nreq])
    q = torch.stack([torch.from_numpy(qq) for (_, _, qq) in data]).to(dev).to(torch.bfloat16)
    attention = SimpleNamespace(indexer=indexer, scaling=1.0 if kind == "exact" else D ** -0.5)
    select_topk(cache, 0, req_ids, q, attention=attention)
    torch.cuda.synchronize()
    gather = cache.gather_indices_for_layer(0)
    lens = cache.visible_lens_for_layer(0)
    out = gather_attn(cache.layers[0], q, gather, lens,
                      torch.arange(nreq, dtype=torch.int32, device=dev), scale=attention.scaling)
    torch.cuda.synchronize()
    gather_c, lens_c = gather.cpu().numpy(), lens.cpu().numpy()
    res = {}
    for row, rid in enumerate(req_ids):
        table = cache.states[rid].block_tables[0]
        table = dict(table) if isinstance(table, dict) else dict(enumerate(table))
        inverse = {int(p): int(l) for l, p in table.items()}
        for kv in range(hkv):
            n = int(lens_c[row, kv])
            slots = gather_c[row, kv, :n]
            ids = np.array([inverse[int(s) // page] * page + int(s) % page for s in slots], np.int32)
            res[f"{name}/ids/{row}/{kv}"] = ids            # in gather order: also pins "ascending"
    ws = getattr(cache, "_nfa_selector_workspace", {}) or {}
    for key in ("topk_far", "topk_near"):
        t = ws.get(key)
        if hasattr(t, "cpu"):
            res[f"{name}/{key}"] = t.cpu().numpy().astype(np.int32)
    res[f"{name}/out"] = out.float().cpu().numpy()
    res[f"{name}/meta"] = np.frombuffer(json.dumps(dict(
        kind=kind, page=page, lengths=lengths, skips=[list(s) for s in skips], cfg=cfg,
        scaling=attention.scaling, max_blocks=max_blocks)).encode(), dtype=np.uint8)
    log(f"{name}: ok, vis_lens {lens_c.tolist()}")
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--install", action="store_true")
    ap.add_argument("--reference", default=None, help="checkout of the reference project (with --install)")
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "ref_selector.new.npz"))
    ap.add_argument("--only", default=None, help="comma-separated case names")
    a = ap.parse_args()
    if a.install:
        if not a.reference:
            ap.error("--install needs --reference <checkout>")
        sys.exit(install(a.reference))
    os.makedirs(os.path.dirname(a.out), exist_ok=True)
    logf = open(os.path.splitext(a.out)[0] + ".log", "w")

    def log(msg):
        print(msg, flush=True)
        logf.write(msg + "\n")
        logf.flush()

    sys.path.insert(0, REF_DIR)
    import torch
    try:
        from sparse_attn.cache import GraphReadyPagedRegionCache
        from sparse_attn.indexer.nfa_indexer import NFAIndexer
        from sparse_attn.indexer.nfa_layer_batch_selector import select_topk_for_layer_batched
        from sparse_attn.ops.paged_region_kernels import sparse_paged_attention_gather
        from sparse_attn.ops.paged_region_kernels_nfa import nfa_args
        from sparse_attn.policies.region_geometry import RegionGeometry
    except Exception:
        log("import of the reference failed:\n" + traceback.format_exc())
        sys.exit(3)
    mods = (GraphReadyPagedRegionCache, NFAIndexer, select_topk_for_layer_batched, sparse_paged_attention_gather,
            nfa_args, RegionGeometry)
    only = set(a.only.split(",")) if a.only else None
    results, failed = {}, []
    for name, kind, page, lengths, skips, cfg in CASES:
        if only and name not in only:
            continue
        t0 = time.time()
        log(f"{name}: start")
        try:
            results.update(run_case(torch, mods, name, kind, page, lengths, skips, cfg, log))
        except Exception:
            failed.append(name)
            log(f"{name}: FAILED\n" + traceback.format_exc())
            if "CUDA error" in traceback.format_exc():
                log("a CUDA error ends the run: nothing after it can be trusted")
                break
        log(f"{name}: {time.time() - t0:.1f} s")
        np.savez_compressed(a.out, **results)      # rewritten after every case: a later failure keeps the earlier ones
    log(f"done: {len(results)} arrays, failed: {failed}")


if __name__ == "__main__":
    main()
