"""Benchmark of the two-level select + gather-attend decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload = "cfg2-qwen3-8b-128k"): Qwen3-8B-shaped attention
stack — 36 layers, 32 query / 8 KV heads, head_dim 128, bf16 — one request of
131 072 tokens in 16-token pages, selector settings K1 128 (32 near pages,
near length 4096), K2 1024 on the 32-dim tail subspace quantised to 4 bits,
sink 4, window 128.  One "step" decodes one token through every layer:
append + L1 + L2 + gather attention per layer.  Data are seeded synthetic
tensors (N(0,1) keys with RoPE and outlier channels); every layer has its own
KV pool and index, so one step touches about 36 x 12.8 MB = 460 MB, more than
the 126 MB L2: no separate L2 flush is needed.

`value` (tok/s) times K steps captured in one CUDA graph with every input
already on the device.  `e2e` times the public Python API the way the reference serves (its
GraphRunner.step): the step's q/k/v arrive in pinned host memory and are copied
to the device, cache.plan_common plans the step on the host, one CUDA-graph
replay runs every layer, and the outputs are copied back to the host.
At N GPUs every rank runs the same workload on its own shard (requests are
independent; no collective on the data path): weak scaling.
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
PKG = "two-level-attention_b200"

N_LAYERS, HQ, HKV, D, PAGE = 36, 32, 8, 128, 16
CONTEXT = 131072
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the one-launch decode step on this
# workload, from one ncu capture (profiles/fused_chain_cfg2_128k_batch1.md)
DECODE_STEP_DRAM_BYTES = 13007616
SUB = 32
METRIC = "decode tok/s at 128K ctx, two-level select+attend path over all layers"


def mod(sub):
    return importlib.import_module(f"{PKG}.{sub}")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def algorithmic_bytes(length):
    """Bytes one layer-step must move (bf16, d'=32, 16-token pages)."""
    w, near_len, sink = 128, 4096, 4
    kt = (length + PAGE - 1) // PAGE
    near_blks = max((length - w - near_len) // PAGE, 0)
    n_far = max(min(near_blks, kt) - 1, 0)
    n_near = max(kt - w // PAGE - near_blks, 0)
    l1 = HKV * (n_far * 2 * SUB * 2 + n_near * SUB * 2)
    l2 = HKV * (96 + 32 + 2) * PAGE * (SUB // 2 + 4)
    vis = min(length, 1024)
    attn = HKV * vis * (D + D) * 2 + HKV * vis * 4
    append = HKV * (D + D) * 2 * 2 + HKV * 3 * SUB * 2
    out = HQ * D * 2 + HQ * D * 2
    return {"l1": l1, "l2": l2, "attn": attn, "append": append, "select": l1 + l2 + append,
            "total": l1 + l2 + attn + append + out}


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_workload(torch, dev, total_steps, seed, lengths=None, n_layers=None):
    """Cache with `n_layers` layers holding one request per entry of `lengths`
    (tokens already in the cache), index buffers allocated, plus device-resident
    inputs for `total_steps` steps."""
    cache_mod = mod("sparse_attn.cache.paged_region_cache")
    geo_mod = mod("sparse_attn.policies.region_geometry")
    nfa = mod("sparse_attn.ops.paged_region_kernels_nfa")
    idx_mod = mod("sparse_attn.indexer.nfa_indexer")
    synth = mod("synth")
    from types import SimpleNamespace
    lengths = [CONTEXT - 1] if lengths is None else list(lengths)
    n_layers = N_LAYERS if n_layers is None else n_layers
    nb = len(lengths)
    args = nfa.nfa_args("tail", tia_block_size=PAGE)
    indexer = idx_mod.NFAIndexer(args)
    geometry = geo_mod.RegionGeometry(sink=4, near=4096, window=128, page=PAGE, max_new_tokens=4096)
    max_blocks = (max(lengths) + 1 + 4096 + PAGE - 1) // PAGE
    pages = sum((n + 4096 + PAGE - 1) // PAGE for n in lengths) + 8
    cache = cache_mod.GraphReadyPagedRegionCache(
        n_layers, geometry, max_requests=nb, max_physical_pages=pages, max_blocks=max_blocks,
        max_visible_len=1024, max_query_tokens=nb, num_kv_heads=HKV, num_query_heads=HQ,
        head_dim_k=D, head_dim_v=D, dtype=torch.bfloat16, device=dev)
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    rids = [cache.add_request() for _ in lengths]
    for li in range(n_layers):
        perm = torch.randperm(pages, generator=g, device=dev).tolist()     # shuffled free list of this layer
        used = 0
        for r, n_pre in enumerate(lengths):
            need = (n_pre + PAGE - 1) // PAGE
            case = synth.make_decode_case(n_pre, num_q_heads=HQ, num_kv_heads=HKV, head_dim=D,
                                          seed=seed * 1000 + li * 97 + r, dtype=torch.bfloat16, device=dev)
            cache.write_prefill(li, rids[r], case.k.permute(1, 0, 2)[None], case.v.permute(1, 0, 2)[None],
                                physical_pages=perm[used:used + need])
            used += need
            del case
    for rid in rids:
        cache.freeze(rid)
    attention = SimpleNamespace(indexer=indexer, scaling=float(D) ** -0.5, layer_idx=0)
    rt = cache.ensure_index(indexer)
    q = torch.randn(total_steps, n_layers, nb, HQ, D, generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn(total_steps, n_layers, nb, HKV, 1, D, generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn(total_steps, n_layers, nb, HKV, 1, D, generator=g, device=dev).to(torch.bfloat16)
    return SimpleNamespace(cache=cache, rid=rids[0], rids=rids, attention=attention, rt=rt, q=q, k=k, v=v,
                           indexer=indexer, lengths=lengths, n_layers=n_layers, batch=nb)


def preplan(torch, wl, n_steps):
    """Device-resident lengths / slots of the next `n_steps` decode steps; grows the block tables."""
    cache = wl.cache
    nb, nl = wl.batch, wl.n_layers
    lengths = torch.zeros(n_steps, nb, dtype=torch.int32)
    slots = torch.zeros(n_steps, nl, nb, dtype=torch.int32)
    for r, rid in enumerate(wl.rids):
        state = cache.states[rid]
        first_len = state.logical_length
        for s in range(n_steps):
            planned = first_len + s + 1
            lp, off = divmod(planned - 1, PAGE)
            lengths[s, r] = planned
            for li in range(nl):
                cache._grow_table(state, rid, li, lp + 1)
                slots[s, li, r] = state.block_tables[li][lp] * PAGE + off
        cache.block_table_buf[:, rid].copy_(cache._cpu_block_table[:, rid])
    ids = torch.tensor(wl.rids, dtype=torch.int64)
    cache.active_req_ids_buf[:nb] = ids.to(cache.device)
    cache.valid_req_ids_buf[:nb] = ids.to(cache.device)
    cache.query_to_req_buf[:nb] = torch.arange(nb, dtype=torch.int32, device=cache.device)
    return lengths.to(cache.device), slots.to(cache.device)


def launch_step(capi, lib, wl, s, lengths, slots, out, which="fused", layers=None):
    """One decode step over the layers through the C ABI (device-resident inputs)."""
    rt, cache = wl.rt, wl.cache
    g = C.byref(rt.geometry)
    stream = capi.current_stream()
    status = C.c_void_p(cache.status_buf.data_ptr())
    ws = capi.ptr(rt.workspace)
    scale = float(wl.attention.scaling)
    nb = wl.batch
    batch = capi.Batch(batch=nb, lengths=lengths[s].data_ptr(), valid_req_ids=cache.valid_req_ids_buf.data_ptr(),
                       active_req_ids=cache.active_req_ids_buf.data_ptr())
    for li in (range(wl.n_layers) if layers is None else layers):
        layer = C.byref(rt.layer_structs[li])
        sel = rt.selection_struct(cache.gather_indices_for_layer(li), cache.visible_lens_for_layer(li), False, False)
        qp = capi.ptr(wl.q[s, li])
        if which == "fused":      # the product path: append rides in the L1 launch, then L2, then attention
            capi.check(lib.loda_decode_step(
                g, layer, C.byref(batch), qp, capi.ptr(wl.k[s, li]), capi.ptr(wl.v[s, li]),
                capi.ptr(slots[s, li]), scale, C.byref(sel), capi.ptr(cache.query_to_req_buf),
                capi.ptr(out[li]), status, ws, stream))
            continue
        if "select" in which:     # append + both selector levels, as the product path launches them
            capi.check(lib.loda_select_step(
                g, layer, C.byref(batch), qp, capi.ptr(wl.k[s, li]), capi.ptr(wl.v[s, li]),
                capi.ptr(slots[s, li]), scale, C.byref(sel), status, ws, stream))
        if "append" in which:
            capi.check(lib.loda_append_decode(g, layer, C.byref(batch), capi.ptr(wl.k[s, li]), capi.ptr(wl.v[s, li]),
                                              capi.ptr(slots[s, li]), status, stream))
        if "l1" in which:
            capi.check(lib.loda_select_l1(g, layer, C.byref(batch), qp, scale, C.byref(sel), ws, stream))
        if "l2" in which:
            capi.check(lib.loda_select_l2(g, layer, C.byref(batch), qp, scale, C.byref(sel), status, ws, stream))
        if "attn" in which:
            capi.check(lib.loda_gather_attend(g, layer, qp, capi.ptr(cache.gather_indices_for_layer(li)),
                                              capi.ptr(cache.visible_lens_for_layer(li)),
                                              capi.ptr(cache.query_to_req_buf), nb, nb, scale, capi.ptr(out[li]),
                                              ws, stream))


def time_kernel(torch, fn, reps):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps     # us per call of fn


def dense_decode_us(torch, wl):
    """Dense FlashAttention decode over all CONTEXT tokens of one layer (timing arm only)."""
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as exc:      # noqa: BLE001
        return None, f"flash_attn unavailable: {type(exc).__name__}"
    try:
        cache = wl.cache
        dev = cache.device
        kc = torch.randn(3, CONTEXT, HKV, D, device=dev, dtype=torch.bfloat16)   # 3 x 268 MB > L2
        vc = torch.randn(3, CONTEXT, HKV, D, device=dev, dtype=torch.bfloat16)
        q = torch.randn(1, 1, HQ, D, device=dev, dtype=torch.bfloat16)
        lens = torch.tensor([CONTEXT], dtype=torch.int32, device=dev)
        fn = lambda i: flash_attn_with_kvcache(q, kc[i:i + 1], vc[i:i + 1], cache_seqlens=lens,
                                               softmax_scale=D ** -0.5)
        for i in range(3):
            fn(i)
        it = [0]

        def call():
            fn(it[0] % 3)
            it[0] += 1
        return time_kernel(torch, call, 30), "flash_attn_with_kvcache, contiguous KV, 131072 tokens"
    except Exception as exc:      # noqa: BLE001
        return None, f"flash_attn failed: {type(exc).__name__}: {exc}"


def measure_device(torch, capi, lib, wl, W, K, barrier):
    """Device-resident timing of a workload: W eager warm-up steps, K steps in one
    CUDA graph between events, then each kernel kind alone over all layers."""
    cache = wl.cache
    sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
    lengths, slots = preplan(torch, wl, W + K)
    out = torch.zeros(wl.n_layers, wl.batch, HQ, D, dtype=torch.bfloat16, device=cache.device)
    # the index of the prefilled pages is built by one bulk pass before the first step
    for li in range(wl.n_layers):
        sel_mod._ensure_index_built(cache, wl.rt, li, wl.rids, has_current_token_in_pool=True)
    torch.cuda.synchronize()
    for s in range(W):
        launch_step(capi, lib, wl, s, lengths, slots, out)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for s in range(W, W + K):
                launch_step(capi, lib, wl, s, lengths, slots, out)
    time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with torch.cuda.stream(stream):
        e0.record(stream)
        graph.replay()
        e1.record(stream)
    stream.synchronize()
    barrier()
    ms_total = e0.elapsed_time(e1)
    status = cache.read_status()
    # Each kernel kind is captured alone in a graph over all layers (rotating pools defeat the
    # L2 cache like the real chain does) so that host launch cost is not part of the figure.
    s_last = W + K - 1
    per_kernel = {}
    for name in ("append", "l1", "l2", "attn", "select"):
        launch_step(capi, lib, wl, s_last, lengths, slots, out, which=(name,))
        torch.cuda.synchronize()
        kgraph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(kgraph, stream=stream):
                launch_step(capi, lib, wl, s_last, lengths, slots, out, which=(name,))
        with torch.cuda.stream(stream):
            kgraph.replay()
            ke0, ke1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ke0.record(stream)
            for _ in range(5):
                kgraph.replay()
            ke1.record(stream)
        stream.synchronize()
        per_kernel[name] = ke0.elapsed_time(ke1) * 1e3 / (5 * wl.n_layers)
    for rid in wl.rids:      # the cache now holds W + K more tokens per request
        st = cache.states[rid]
        st.logical_length += W + K
        for li in range(wl.n_layers):
            st.index_len[li] = st.logical_length
    return ms_total, per_kernel, status, stream, out


def batched_arm(torch, capi, lib, dev, seed, barrier):
    """Config 3 shape: 32 requests with lengths uniform in [8192, 65536] in one shared pool with
    shuffled page tables, two layers (so that a step's touched bytes exceed L2); reports the
    kernels' durations and the L1 kernel's bandwidth at a batch where it is not latency bound."""
    import random
    rnd = random.Random(seed)
    lens = [rnd.randint(8192, 65536) for _ in range(32)]
    wl = build_workload(torch, dev, 3 + 5 + 2, seed, lengths=lens, n_layers=2)
    ms_total, per_kernel, status, _, _ = measure_device(torch, capi, lib, wl, 3, 5, barrier)
    l1_bytes = sum(algorithmic_bytes(n + 1)["l1"] for n in lens)
    tot_bytes = sum(algorithmic_bytes(n + 1)["total"] for n in lens)
    peak, kind = peaks()
    us_layer = ms_total * 1e3 / (5 * wl.n_layers)
    return {"workload": "cfg3: 32 requests, context uniform in [8192, 65536], shuffled pages, 2 layers",
            "tokens_in_cache": sum(lens), "us_per_decode_step_per_layer": us_layer,
            "tok_s_per_layer_stack": 32 / (us_layer * 1e-6 * N_LAYERS),
            "kernel_us_per_launch": per_kernel, "device_status": status,
            "l1_roofline": {"bound": "hbm", "achieved": l1_bytes / (per_kernel["l1"] * 1e-6) / 1e9, "peak": peak,
                            "unit": "GB/s", "frac": l1_bytes / (per_kernel["l1"] * 1e-6) / 1e9 / peak,
                            "peak_kind": f"of {kind}", "algorithmic_bytes": l1_bytes},
            "chain_hbm_frac_of_8TBs": tot_bytes / (us_layer * 1e-6) / 8e12}


def tls_chain_arm(torch, dev, warm=10, iters=100):
    """The prototype chain on a contiguous cache at the shape of the reference's own micro-benchmark
    (benchmark/efficiency/benchmark_mha_kernel.py:21-37): batch 4, 4 query heads on 1 KV head, D 128,
    131 072 tokens, 64-token blocks, cmp ratio 4, level-1 top 128 blocks, level-2 top 1 024 tokens, 3
    sliding blocks; level 1 -> level 2 -> sparse attention timed together (each feeds the next), and
    the dense attention over the whole cache beside it.  Random bf16 tensors as in that script."""
    ops = mod("tls_attn.ops")
    batch, hq, hkv, d, s, block, cmp, k1, k2, sliding = 4, 4, 1, 128, 131072, 64, 4, 128, 1024, 3
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *shape: torch.randn(*shape, dtype=torch.bfloat16, device=dev, generator=g)
    q, k, v = rn(batch, 1, hq, d), rn(batch, s, hkv, d), rn(batch, s, hkv, d)
    lengths = torch.full((batch,), s, dtype=torch.int32, device=dev)
    l1q, kmin, kmax = rn(batch, 1, hq, d), rn(batch, s // block, hkv, d), rn(batch, s // block, hkv, d)
    l1_scores = torch.full((batch, hkv, s // block), float("-inf"), dtype=torch.float32, device=dev)
    l1_ts = torch.zeros((batch, hkv, k1), dtype=torch.float32, device=dev)
    l1_ti = torch.zeros((batch, hkv, k1), dtype=torch.int32, device=dev)
    l1_len = lengths // block
    l2q, l2k = rn(batch, 1, hq, d // cmp), rn(batch, s, hkv, d // cmp)
    l2_scores = torch.full((batch, hkv, k1 * block), float("-inf"), dtype=torch.float32, device=dev)
    l2_idx = torch.full((batch, hkv, k1 * block), -1, dtype=torch.int32, device=dev)
    l2_cm = torch.full((batch, hkv, k1 * block), float("-inf"), dtype=torch.float32, device=dev)
    l2_ts = torch.zeros((batch, hkv, k2), dtype=torch.float32, device=dev)
    l2_ti = torch.zeros((batch, hkv, k2), dtype=torch.int32, device=dev)
    o = torch.zeros(batch, 1, hq, d, dtype=torch.bfloat16, device=dev)
    lvl1 = ops.MHAIndexerLevel1Interface(hq, hkv, d, k1, sliding)
    lvl2 = ops.MHAIndexerLevel2Interface(hq, hkv, d // cmp, k1, k2, block, sliding)
    sparse = ops.SparseMHAInterface(hq, hkv, d, d, k2)
    dense = ops.MHAInterface(hq, hkv, d, d)

    def chain():
        lvl1.forward_with_buffer(l1q, kmin, kmax, l1_len, l1_scores, l1_ts, l1_ti)
        lvl2.forward_with_buffer(l2q, l2k, l1_ti, lengths, l2_scores, l2_idx, l2_cm, l2_ts, l2_ti)
        sparse.forward_with_buffer(q, k, v, l2_ti, o)

    def timed(fn):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    out = {"workload": "tls_attn chain: batch 4, 4q/1kv heads, d128, 131072 tokens, block 64, cmp 4, K1 128, K2 1024, "
                       "3 sliding blocks (the reference micro-benchmark's shape)",
           "sparse_chain_ms": timed(chain),
           "level1_ms": timed(lambda: lvl1.forward_with_buffer(l1q, kmin, kmax, l1_len, l1_scores, l1_ts, l1_ti)),
           "level2_ms": timed(lambda: lvl2.forward_with_buffer(l2q, l2k, l1_ti, lengths, l2_scores, l2_idx, l2_cm,
                                                               l2_ts, l2_ti)),
           "sparse_mha_ms": timed(lambda: sparse.forward_with_buffer(q, k, v, l2_ti, o)),
           "dense_mha_ms": timed(lambda: dense.forward_with_buffer(q, k, v, lengths, o)),
           "iters": iters, "warmup": warm}
    torch.cuda.synchronize()
    return out


def run_sequence_sharded(torch, dist, capi, lib, dev, local, rank, world, K, W, barrier):
    """Strong scaling of ONE 131 072-token request: logical page p lives on rank p % world; per layer
    the staged selector with two all-gathers of 16-bit score rows, the attention over the rank's own
    tokens and an all-gather + log-sum-exp merge of the partial outputs (NCCL).  Every rank holds the
    whole synthetic cache here and masks the other ranks' pages out of its block table; the owner of
    the new token's page appends it (the other ranks pass slot -1, the pad slot).  Timed twice: eager
    launches, and the whole step over all layers (kernels and collectives) replayed as one CUDA graph."""
    sharding = mod("sharding")
    total = 2 * (W + K) + 4
    wl = build_workload(torch, dev, total, seed=11)              # the same request on every rank
    cache = wl.cache
    sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
    lengths, slots = preplan(torch, wl, total - 2)
    for li in range(wl.n_layers):
        sel_mod._ensure_index_built(cache, wl.rt, li, wl.rids, has_current_token_in_pool=True)
    shard = sharding.SequenceShard(cache, wl.indexer, rank, world)
    g = C.byref(wl.rt.geometry)
    status = C.c_void_p(cache.status_buf.data_ptr())
    host_len = [int(x) for x in lengths[:, 0].cpu().tolist()]
    own = torch.tensor([shard.owns_token(n - 1) for n in host_len], device=dev)
    my_slots = torch.where(own[:, None, None], slots, torch.full_like(slots, -1))
    # fixed-address inputs of a step (a captured graph reads them)
    q_in, k_in, v_in = wl.q[0].clone(), wl.k[0].clone(), wl.v[0].clone()
    slot_in = my_slots[0].clone()
    batch = capi.Batch(batch=1, lengths=cache.planned_lengths_buf.data_ptr(),
                       valid_req_ids=cache.valid_req_ids_buf.data_ptr(),
                       active_req_ids=cache.active_req_ids_buf.data_ptr())

    def load(s):
        cache.planned_lengths_buf[:1].copy_(lengths[s])
        q_in.copy_(wl.q[s]); k_in.copy_(wl.k[s]); v_in.copy_(wl.v[s]); slot_in.copy_(my_slots[s])

    def body():
        outs = None
        for li in range(wl.n_layers):
            capi.check(lib.loda_append_decode(g, C.byref(wl.rt.layer_structs[li]), C.byref(batch), capi.ptr(k_in[li]),
                                              capi.ptr(v_in[li]), capi.ptr(slot_in[li]), status,
                                              capi.current_stream()))
            outs, _, _ = sharding.sequence_sharded_decode_step(shard, li, wl.rids, q_in[li], wl.attention)
        return outs

    def timed(run, first):
        for s in range(first, first + W):
            load(s); run()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(first + W, first + W + K):
            load(s); run()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / K

    sampler = ClockSampler(local)
    sampler.start()
    eager_ms = timed(body, 0)
    graph_ms, graph_note = None, None
    try:
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        load(W + K)
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                body()
        torch.cuda.current_stream().wait_stream(stream)
        graph_ms = timed(graph.replay, W + K)
    except Exception as exc:            # capture of the collectives refused: the eager figure stands
        graph_note = f"graph capture failed: {type(exc).__name__}"
    clocks = sampler.stop()
    ms_per_step = graph_ms if graph_ms is not None else eager_ms
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": 1e3 / ms_per_step, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg2-qwen3-8b-128k", "layers": N_LAYERS, "context": CONTEXT, "batch": 1,
                       "page": PAGE, "sharding": f"sequence: pages round robin over {world} GPUs, all-gather of "
                                                 "16-bit score rows after each selector level, LSE merge of the "
                                                 "partial attentions (NCCL)"},
            "us_per_decode_step_per_layer": ms_per_step * 1e3 / N_LAYERS,
            "eager_us_per_layer": eager_ms * 1e3 / N_LAYERS,
            "graph_us_per_layer": None if graph_ms is None else graph_ms * 1e3 / N_LAYERS, "graph_note": graph_note,
            "gpu_launches": K * N_LAYERS * 6, "device_status": cache.read_status(), "clocks": clocks,
            "roofline": None, "e2e": None}), flush=True)


def cpu_baseline(sample_steps=3, threads=1):
    """One layer of the workload on the host cores with the CPU oracle (index
    prebuilt, as the reference maintains its page statistics incrementally)."""
    import numpy as np

    from oracle import loda_oracle as O
    rng = np.random.default_rng(0)
    length = CONTEXT
    k = O.bf16_rn(rng.standard_normal((length, HKV, D), dtype=np.float32))
    v = O.bf16_rn(rng.standard_normal((length, HKV, D), dtype=np.float32))
    cfg = O.SelectorConfig(max_blocks=(length + PAGE - 1) // PAGE + 8, block_size=PAGE)
    index = O.build_index(k, length, cfg)
    pool_k = k.reshape(-1, PAGE, HKV, D).transpose(0, 2, 1, 3).copy()
    pool_v = v.reshape(-1, PAGE, HKV, D).transpose(0, 2, 1, 3).copy()
    table = np.arange(pool_k.shape[0])
    times = []
    for s in range(sample_steps):
        q = O.bf16_rn(rng.standard_normal((HQ, D), dtype=np.float32))
        t0 = time.perf_counter()
        sel = O.select_request(q, k, length, cfg, D ** -0.5, index=index)
        gather = np.full((1, HKV, 1024), -1, np.int32)
        lens = np.zeros((1, HKV), np.int32)
        for kv in range(HKV):
            ids = sel.logical[kv]
            gather[0, kv, :len(ids)] = O.to_slots(ids, table, PAGE)
            lens[0, kv] = len(ids)
        O.gather_attention(q[None], pool_k, pool_v, gather, lens, np.array([0]), D ** -0.5, "bf16")
        times.append(time.perf_counter() - t0)
    per_layer = sum(times) / len(times)
    return {"value": 1.0 / (per_layer * N_LAYERS), "unit": "tok/s", "cores": threads, "kind": "port",
            "us_per_step_per_layer": per_layer * 1e6,
            "sample": f"{sample_steps} decode steps of 1 of {N_LAYERS} layers at {CONTEXT} tokens "
                      f"(numpy oracle, selector index prebuilt), scaled to {N_LAYERS} layers"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    t0 = time.perf_counter()
    base = cpu_baseline(sample_steps=max(1, min(args.steps, 5)))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / base["value"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": "cfg2-qwen3-8b-128k", "layers": N_LAYERS,
                                        "context": CONTEXT, "batch": 1, "page": PAGE},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's hot path is GPU-only Triton; its CPU form is the numpy restatement "
                "under oracle/, run on one host thread",
        "wall_s": None}
    line["wall_s"] = round(time.perf_counter() - t0, 1)
    print(json.dumps(line), flush=True)


def main():
    global N_LAYERS, HQ, HKV
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-dense", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-batched", action="store_true")
    ap.add_argument("--skip-tls", action="store_true")
    ap.add_argument("--shard", default="request", choices=("request", "kvhead", "sequence"),
                    help="multi-GPU partition: one independent request shard per GPU (weak scaling, default), "
                         "the KV-head groups of ONE request split over the GPUs, or the pages of ONE request "
                         "dealt round robin over the GPUs with NCCL all-gathers between the stages (strong scaling)")
    ap.add_argument("--layers", type=int, default=N_LAYERS,
                    help="profiling aid: fewer layers than the 36 of the named workload (not a bench line)")
    args = ap.parse_args()
    N_LAYERS = args.layers
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.warmup < 3:
        args.warmup = 3
    kvhead = args.shard == "kvhead" and world > 1
    if kvhead:
        shard = mod("sharding").kv_head_shard(HQ, HKV, world, rank)
        HQ, HKV = shard.num_q_heads, shard.num_kv_heads      # this rank's heads of the same request

    import torch
    import torch.distributed as dist
    capi = mod("_capi")
    lib = capi.lib()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    K, W = args.steps, args.warmup
    if args.shard == "sequence" and world > 1:
        run_sequence_sharded(torch, dist, capi, lib, dev, local, rank, world, K, W, barrier)
        dist.barrier()
        dist.destroy_process_group()
        return
    e2e_steps = K
    total = W + K + W + e2e_steps + 8
    wl = build_workload(torch, dev, total, seed=11 + (0 if kvhead else rank))
    cache = wl.cache
    sampler = ClockSampler(local)
    sampler.start()
    ms_total, per_kernel, status, stream, out = measure_device(torch, capi, lib, wl, W, K, barrier)
    clocks = sampler.stop()

    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / K
    tok_s = (1.0 if kvhead else world) / (ms_per_step * 1e-3)

    # ---- end to end through the public Python API with host buffers ----------------
    base_s = W + K
    hq_ = wl.q[base_s:base_s + W + e2e_steps].cpu().pin_memory()
    hk_ = wl.k[base_s:base_s + W + e2e_steps].cpu().pin_memory()
    hv_ = wl.v[base_s:base_s + W + e2e_steps].cpu().pin_memory()
    attn_objs = [type(wl.attention)(indexer=wl.indexer, scaling=wl.attention.scaling, layer_idx=li)
                 for li in range(N_LAYERS)]
    runner = mod("sparse_attn.engine.graph_runner").DecodeGraphRunner(cache, attn_objs, 1)

    def e2e_step(i):
        # pinned host q/k/v in, plan on the host, one graph replay over all layers, outputs back to the host
        return runner.step(hq_[i, :, :, :, :], hk_[i], hv_[i])

    if not args.skip_e2e:
        runner.q.copy_(hq_[0]); runner.k.copy_(hk_[0]); runner.v.copy_(hv_[0])
        runner.capture([wl.rid])
    dq, dk, dv, hout = runner.q, runner.k, runner.v, runner.host_out
    if args.skip_e2e:
        e2e_steps = 0
    for i in range(W if e2e_steps else 0):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(W, W + e2e_steps):
        e2e_step(i)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / max(e2e_steps, 1)
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    h2d = int(dq.numel() + dk.numel() + dv.numel()) * 2 + (N_LAYERS * 4 + 8 + 8 + 4 + 4)
    d2h = int(hout.numel()) * 2

    # kernels per layer-step of the product path as the library last ran it: 1 = selection and attention
    # in one launch, 2 = one-launch selection + attention, 3 = L1, L2, attention
    launches_per_layer = int(lib.loda_last_decode_launches()) or 2
    if rank == 0:
        peak, peak_kind = peaks()
        ab = algorithmic_bytes(CONTEXT)
        # the product path launches the selector ("select": append + both levels, one launch at this
        # batch) and the attention; l1 / l2 / append are the selector's parts as stand-alone launches
        us_layer = ms_per_step * 1e3 / N_LAYERS
        if launches_per_layer == 1:
            # one launch per layer-step does everything: its average duration is the chain's time per layer
            per_kernel["decode_step"] = us_layer
            ab["decode_step"] = ab["total"]
            dominant = "decode_step"
        else:
            dominant = max(("select", "attn"), key=per_kernel.get)
        achieved = ab[dominant] / (per_kernel[dominant] * 1e-6) / 1e9
        dense_us, dense_note = (None, "skipped") if args.skip_dense else dense_decode_us(torch, wl)
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if kvhead else "weak",
            "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg2-qwen3-8b-128k", "layers": N_LAYERS, "context": CONTEXT, "batch": 1,
                       "page": PAGE, "heads": f"{HQ}q/{HKV}kv", "head_dim": D,
                       "selector": "K1=128 (32 near), K2=1024, tail32 int4, sink 4, swa 128",
                       "l2_flush": "none needed: 36 layers x 12.8 MB touched per step exceeds the 126 MB L2",
                       "sharding": (f"KV-head groups of one request, {HKV} KV heads per GPU, no data-path collective"
                                    if kvhead else "one independent request shard per GPU, no data-path collective")},
            "us_per_decode_step_per_layer": us_layer,
            "kernel_us_per_launch": per_kernel,
            "algorithmic_bytes_per_layer_step": ab,
            "chain_hbm_frac_of_8TBs": ab["total"] / (us_layer * 1e-6) / 8e12,
            "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of that launch on
                         # this workload (profiles/fused_chain_cfg2_128k_batch1.md); not measured live
                         "traffic": {"select": 8821504, "decode_step": DECODE_STEP_DRAM_BYTES}.get(dominant)},
            "dense_decode": {"us_per_layer": dense_us, "note": dense_note,
                             "ours_over_dense": (us_layer / dense_us) if dense_us else None},
            "e2e": None if args.skip_e2e else {
                "value": (1 if kvhead else world) * 1e3 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": K * N_LAYERS * launches_per_layer, "device_status": status, "clocks": clocks,
            "launches_per_layer_step": launches_per_layer,
        }
        if not args.skip_batched and not kvhead:
            del wl, runner, cache
            torch.cuda.empty_cache()
            line["batched"] = batched_arm(torch, capi, lib, dev, 5, lambda: torch.cuda.synchronize())
        if kvhead:
            line.pop("batched", None)
        if not args.skip_tls and not kvhead and world == 1:
            torch.cuda.empty_cache()
            line["tls_chain"] = tls_chain_arm(torch, dev)
        if not args.skip_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(sample_steps=3)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
