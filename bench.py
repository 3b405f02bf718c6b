"""Benchmark of the two-level select + gather-attend decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload = "cfg2-qwen3-8b-128k"): Qwen3-8B-shaped attention stack — 36 layers, 32
query / 8 KV heads, head_dim 128, bf16 — one request of 131 072 tokens in 16-token pages, selector
settings K1 128 (32 near pages, near length 4096), K2 1024 on the 32-dim tail subspace quantised to
4 bits, sink 4, window 128.  One "step" decodes one token through every layer: append + L1 + L2 +
gather attention per layer.  Data are seeded synthetic tensors (N(0,1) keys with RoPE and outlier
channels); every layer has its own KV pool and index, so one step touches about 36 x 12.8 MB =
460 MB, more than the 126 MB L2: no separate L2 flush is needed.

`value` (tok/s) times K steps captured in one CUDA graph with every input already on the device;
the graph is replayed until the timed region lasts at least half a second (the appends rewrite the
same slots: idempotent), every replay is bracketed by events, and the line carries the median and
the spread of the replays.  `e2e` times the public Python API the way the reference serves (its
GraphRunner.step): the step's q/k/v arrive in pinned host memory and are copied to the device,
cache.plan_common plans the step on the host, one CUDA-graph replay runs every layer, and the
outputs are copied back to the host.  After the timed region the lists and the attention output
of layer 0 of the last step are checked against the CPU oracle (`parity_checked`).

At N GPUs the KV heads of the request are split over the ranks (8 / N KV heads and their query
heads per GPU); after every layer the ranks all-gather the attention output (NCCL, inside the
captured graph and the timed region): strong scaling of one decode stream.  `--shard request`
runs one independent request per GPU instead (weak scaling, no collective), `--shard sequence`
deals the pages of the one request over the GPUs.  The `cfg4` object repeats the measurement on
the batched shape of the Llama-3.1-8B configuration (8 requests of 131 072 tokens, RoPE theta 5e5
with llama3 scaling, a stated number of its 32 layers) with the same KV-head partition.  On one GPU
the line also carries `batched` (32 requests of 8 192..65 536 tokens: the three-launch chain and the
level-1 kernel's bandwidth; `--only-batched` runs it alone), `cfg5` (the MLA shared-latent shape: 16
requests of 131 072 tokens on one 576-dim latent row per token; `--only-cfg5`), the `tls_attn` chain,
the reference's own Triton selector on the same GPU (when its packages are installed under
baseline/_ref) and the CPU baseline.
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib
import json
import os
import statistics
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
SUB = 32
METRIC = "decode tok/s at 128K ctx, two-level select+attend path over all layers"
SELECTOR = "K1=128 (32 near), K2=1024, tail32 int4, sink 4, swa 128"
MIN_TIMED_S = 0.5


def mod(sub):
    return importlib.import_module(f"{PKG}.{sub}")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_traffic(kernel, workload):
    """DRAM bytes per launch of `kernel` on `workload` from the ncu figures kept as text beside the
    profile summaries (lines "<kernel> <workload> <bytes>"); None when no capture is recorded."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    try:
        with open(path) as f:
            for line in f:
                parts = line.split()
                if len(parts) >= 3 and parts[0] == kernel and parts[1] == workload:
                    return int(parts[2])
    except OSError:
        pass
    return None


def algorithmic_bytes(length, hkv=HKV, hq=HQ):
    """Bytes one layer-step must move (bf16, d'=32, 16-token pages)."""
    w, near_len = 128, 4096
    kt = (length + PAGE - 1) // PAGE
    near_blks = max((length - w - near_len) // PAGE, 0)
    n_far = max(min(near_blks, kt) - 1, 0)
    n_near = max(kt - w // PAGE - near_blks, 0)
    l1 = hkv * (n_far * 2 * SUB * 2 + n_near * SUB * 2)
    l2 = hkv * (96 + 32 + 2) * PAGE * (SUB // 2 + 4)
    vis = min(length, 1024)
    attn = hkv * vis * (D + D) * 2 + hkv * vis * 4
    append = hkv * (D + D) * 2 * 2 + hkv * 3 * SUB * 2
    out = hq * D * 2 + hq * D * 2
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


def build_workload(torch, dev, total_steps, seed, lengths=None, n_layers=None, hq=None, hkv=None,
                   theta=1e6, llama3=False, page=None, d=None, dv=None, shared_latent=False):
    """Cache with `n_layers` layers holding one request per entry of `lengths` (tokens already in
    the cache), index buffers allocated, plus device-resident inputs for `total_steps` steps."""
    cache_mod = mod("sparse_attn.cache.paged_region_cache")
    geo_mod = mod("sparse_attn.policies.region_geometry")
    nfa = mod("sparse_attn.ops.paged_region_kernels_nfa")
    idx_mod = mod("sparse_attn.indexer.nfa_indexer")
    synth = mod("synth")
    from types import SimpleNamespace
    lengths = [CONTEXT - 1] if lengths is None else list(lengths)
    n_layers = N_LAYERS if n_layers is None else n_layers
    hq = HQ if hq is None else hq
    hkv = HKV if hkv is None else hkv
    nb = len(lengths)
    page = PAGE if page is None else page
    d = D if d is None else d
    dv = d if dv is None else dv
    args = nfa.nfa_args("tail", tia_block_size=page, **({} if d == 128 else {"head_dim": d}))
    indexer = idx_mod.NFAIndexer(args)
    geometry = geo_mod.RegionGeometry(sink=4, near=4096, window=128, page=page, max_new_tokens=4096)
    max_blocks = (max(lengths) + 1 + 4096 + page - 1) // page
    pages = sum((n + 4096 + page - 1) // page for n in lengths) + 8
    cache = cache_mod.GraphReadyPagedRegionCache(
        n_layers, geometry, max_requests=nb, max_physical_pages=pages, max_blocks=max_blocks,
        max_visible_len=1024, max_query_tokens=nb, num_kv_heads=hkv, num_query_heads=hq,
        head_dim_k=d, head_dim_v=dv, dtype=torch.bfloat16, device=dev,
        **({"shared_latent": True} if shared_latent else {}))
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    rids = [cache.add_request() for _ in lengths]
    for li in range(n_layers):
        perm = torch.randperm(pages, generator=g, device=dev).tolist()     # shuffled free list of this layer
        used = 0
        for r, n_pre in enumerate(lengths):
            need = (n_pre + page - 1) // page
            case = synth.make_decode_case(n_pre, num_q_heads=hq, num_kv_heads=hkv, head_dim=d,
                                          seed=seed * 1000 + li * 97 + r, dtype=torch.bfloat16, device=dev,
                                          theta=theta, llama3_scaling=llama3)
            vals = case.k[..., :dv] if shared_latent else case.v[..., :dv]
            cache.write_prefill(li, rids[r], case.k.permute(1, 0, 2)[None], vals.permute(1, 0, 2)[None],
                                physical_pages=perm[used:used + need])
            used += need
            del case, vals
    for rid in rids:
        cache.freeze(rid)
    attention = SimpleNamespace(indexer=indexer, scaling=float(d) ** -0.5, layer_idx=0)
    rt = cache.ensure_index(indexer)
    q = torch.randn(total_steps, n_layers, nb, hq, d, generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn(total_steps, n_layers, nb, hkv, 1, d, generator=g, device=dev).to(torch.bfloat16)
    v = k[..., :dv] if shared_latent else torch.randn(total_steps, n_layers, nb, hkv, 1, dv, generator=g,
                                                      device=dev).to(torch.bfloat16)
    return SimpleNamespace(cache=cache, rid=rids[0], rids=rids, attention=attention, rt=rt, q=q, k=k, v=v,
                           indexer=indexer, lengths=lengths, n_layers=n_layers, batch=nb, hq=hq, hkv=hkv,
                           page=page, d=d, dv=dv)


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
            lp, off = divmod(planned - 1, wl.page)
            lengths[s, r] = planned
            for li in range(nl):
                cache._grow_table(state, rid, li, lp + 1)
                slots[s, li, r] = state.block_tables[li][lp] * wl.page + off
        cache.block_table_buf[:, rid].copy_(cache._cpu_block_table[:, rid])
    ids = torch.tensor(wl.rids, dtype=torch.int64)
    cache.active_req_ids_buf[:nb] = ids.to(cache.device)
    cache.valid_req_ids_buf[:nb] = ids.to(cache.device)
    cache.query_to_req_buf[:nb] = torch.arange(nb, dtype=torch.int32, device=cache.device)
    return lengths.to(cache.device), slots.to(cache.device)


def launch_step(capi, lib, wl, s, lengths, slots, out, which="fused", layers=None, after_layer=None,
                chain=True):
    """One decode step over the layers through the C ABI (device-resident inputs).  after_layer(li):
    what follows a layer's attention (the all-gather of the heads' outputs under KV-head sharding);
    a launch directly behind the decode step of the layer before it carries LODA_SEL_CHAINED."""
    rt, cache = wl.rt, wl.cache
    g = C.byref(rt.geometry)
    stream = capi.current_stream()
    status = C.c_void_p(cache.status_buf.data_ptr())
    ws = capi.ptr(rt.workspace)
    scale = float(wl.attention.scaling)
    nb = wl.batch
    batch = capi.Batch(batch=nb, lengths=lengths[s].data_ptr(), valid_req_ids=cache.valid_req_ids_buf.data_ptr(),
                       active_req_ids=cache.active_req_ids_buf.data_ptr())
    first = True
    for li in (range(wl.n_layers) if layers is None else layers):
        layer = C.byref(rt.layer_structs[li])
        chained = chain and which == "fused" and after_layer is None and not first
        first = False
        sel = rt.selection_struct(cache.gather_indices_for_layer(li), cache.visible_lens_for_layer(li), False, False,
                                  chained=chained)
        qp = capi.ptr(wl.q[s, li])
        if which == "fused":      # the product path: one call per layer
            capi.check(lib.loda_decode_step(
                g, layer, C.byref(batch), qp, capi.ptr(wl.k[s, li]), capi.ptr(wl.v[s, li]),
                capi.ptr(slots[s, li]), scale, C.byref(sel), capi.ptr(cache.query_to_req_buf),
                capi.ptr(out[li]), status, ws, stream))
            if after_layer is not None:
                after_layer(li)
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


def dense_decode_us(torch, dev):
    """Dense decode attention over all CONTEXT tokens of one layer (timing arms only): FlashAttention-2's
    flash_attn_with_kvcache and FlashInfer's paged batch decode, each over rotating caches larger than L2."""
    arms = {}
    q = torch.randn(1, 1, HQ, D, device=dev, dtype=torch.bfloat16)
    try:
        from flash_attn import flash_attn_with_kvcache
        kc = torch.randn(3, CONTEXT, HKV, D, device=dev, dtype=torch.bfloat16)   # 3 x 268 MB > L2
        vc = torch.randn(3, CONTEXT, HKV, D, device=dev, dtype=torch.bfloat16)
        lens = torch.tensor([CONTEXT], dtype=torch.int32, device=dev)
        fn = lambda i: flash_attn_with_kvcache(q, kc[i:i + 1], vc[i:i + 1], cache_seqlens=lens, softmax_scale=D ** -0.5)
        for i in range(3):
            fn(i)
        it = [0]

        def call():
            fn(it[0] % 3)
            it[0] += 1
        arms["flash_attn_with_kvcache"] = time_kernel(torch, call, 60)
        del kc, vc
    except Exception as exc:      # noqa: BLE001
        arms["flash_attn_with_kvcache"] = f"unavailable: {type(exc).__name__}: {exc}"[:160]
    try:
        import flashinfer
        page = 16
        n_pages = CONTEXT // page
        kv = torch.randn(3, n_pages, 2, page, HKV, D, device=dev, dtype=torch.bfloat16)   # NHD pages
        ws = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        wrapper = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
        indptr = torch.tensor([0, n_pages], dtype=torch.int32, device=dev)
        indices = torch.arange(n_pages, dtype=torch.int32, device=dev)
        last = torch.tensor([page], dtype=torch.int32, device=dev)
        wrapper.plan(indptr, indices, last, HQ, HKV, D, page, q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16,
                     sm_scale=D ** -0.5)
        q1 = q[0]
        for i in range(3):
            wrapper.run(q1, kv[i])
        it = [0]

        def call2():
            wrapper.run(q1, kv[it[0] % 3])
            it[0] += 1
        arms["flashinfer_paged_decode"] = time_kernel(torch, call2, 60)
        del kv, ws
    except Exception as exc:      # noqa: BLE001
        arms["flashinfer_paged_decode"] = f"unavailable: {type(exc).__name__}: {exc}"[:160]
    torch.cuda.empty_cache()
    return arms


def agree_max(torch, value):
    """The largest of the ranks' values (every rank must replay a graph that holds collectives equally often)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return int(value)
    t = torch.tensor([int(value)], device="cuda" if dist.get_backend() == "nccl" else "cpu", dtype=torch.int64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return int(t.item())


def measure_device(torch, capi, lib, wl, W, K, barrier, after_layer=None, kernels=True, min_timed_s=MIN_TIMED_S,
                   out=None):
    """Device-resident timing of a workload: W eager warm-up steps, K steps captured in one CUDA graph
    and replayed between events until the timed region lasts min_timed_s, then each kernel kind alone
    over all layers.  Returns (ms of one K-step replay as total / replays, statistics, per-kernel us,
    device status, stream, out, (lengths, slots))."""
    cache = wl.cache
    sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
    lengths, slots = preplan(torch, wl, W + K)
    if out is None:
        out = torch.zeros(wl.n_layers, wl.batch, wl.hq, wl.dv, dtype=torch.bfloat16, device=cache.device)
    # the index of the prefilled pages is built by one bulk pass before the first step
    for li in range(wl.n_layers):
        sel_mod._ensure_index_built(cache, wl.rt, li, wl.rids, has_current_token_in_pool=True)
    torch.cuda.synchronize()
    for s in range(W):
        launch_step(capi, lib, wl, s, lengths, slots, out, after_layer=after_layer)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for s in range(W, W + K):
                launch_step(capi, lib, wl, s, lengths, slots, out, after_layer=after_layer)
    time.sleep(0.3)
    # one untimed replay sizes the timed region
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        graph.replay()
        e1.record(stream)
    stream.synchronize()
    one_ms = max(e0.elapsed_time(e1), 1e-3)
    replays = max(1, min(2000, int(1.1 * min_timed_s * 1e3 / one_ms) + 2))
    replays = agree_max(torch, replays)      # the same count on every rank: the graph may hold collectives
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
    barrier()
    with torch.cuda.stream(stream):
        marks[0].record(stream)
        for r in range(replays):
            graph.replay()
            marks[r + 1].record(stream)
    stream.synchronize()
    barrier()
    total_ms = marks[0].elapsed_time(marks[-1])
    each = [marks[r].elapsed_time(marks[r + 1]) for r in range(replays)]
    stats = {"replays": replays, "timed_region_ms": total_ms, "replay_ms_median": statistics.median(each),
             "replay_ms_min": min(each), "replay_ms_max": max(each),
             "replay_ms_stdev": statistics.pstdev(each) if len(each) > 1 else 0.0}
    status = cache.read_status()
    # Each kernel kind is captured alone in a graph over all layers (rotating pools defeat the
    # L2 cache like the real chain does) so that host launch cost is not part of the figure.
    s_last = W + K - 1
    per_kernel = {}
    for name in (("append", "l1", "l2", "attn", "select") if kernels else ()):
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
            for _ in range(20):
                kgraph.replay()
            ke1.record(stream)
        stream.synchronize()
        per_kernel[name] = ke0.elapsed_time(ke1) * 1e3 / (20 * wl.n_layers)
    if kernels:      # leave layer 0 in the state of the product path's last step (the parity check reads it)
        launch_step(capi, lib, wl, s_last, lengths, slots, out)
        torch.cuda.synchronize()
    for rid in wl.rids:      # the cache now holds W + K more tokens per request
        st = cache.states[rid]
        st.logical_length += W + K
        for li in range(wl.n_layers):
            st.index_len[li] = st.logical_length
    return total_ms / replays, stats, per_kernel, status, stream, out, (lengths, slots)


def parity_check(torch, wl, out, lengths, s_last, rows=None):
    """Layer 0 of the last timed step against the CPU oracle (outside every timed region): the keys
    and values are read back from the paged pool through the block table, the oracle selects from
    them, and its token lists (as physical slots) and attention must equal the GPU's."""
    import numpy as np

    from oracle import loda_oracle as O
    cache, layer = wl.cache, wl.cache.layers[0]
    ix = wl.indexer
    rows = list(range(wl.batch)) if rows is None else rows
    f32 = lambda t: t.detach().float().cpu().numpy()
    gather = cache.gather_indices_for_layer(0).cpu().numpy()
    lens = cache.visible_lens_for_layer(0).cpu().numpy()
    pool_k, pool_v = f32(layer.kv_pool_k[:, 0]), f32(layer.kv_pool_v[:, 0])
    cfg = O.SelectorConfig(
        num_q_heads=wl.hq, num_kv_heads=wl.hkv, block_size=PAGE, max_blocks=cache.max_blocks,
        level1_topk=int(ix.args.tia_level1_topk), near_pages=int(ix.nt_near_pages), near_len=int(ix.nt_near_len),
        level2_topk=int(ix.args.tia_level2_topk), cmp_ratio=ix.cmp_ratio, sink=ix.sink_tokens,
        swa=ix.sliding_window_size, max_visible=cache.max_visible_len, mode="bf16")
    identical, worst = True, 0.0
    q_all = f32(wl.q[s_last, 0])
    for b in rows:
        rid = wl.rids[b]
        length = int(lengths[s_last, b])
        table = cache.block_table_buf[0, rid].cpu().numpy()
        k_log = O.logical_keys(pool_k, table, length)
        sel = O.select_request(q_all[b], k_log, length, cfg, wl.attention.scaling)
        for kv in range(wl.hkv):
            want = O.to_slots(sel.logical[kv], table, PAGE)
            if lens[b, kv] != len(want) or not np.array_equal(gather[b, kv, :len(want)], want):
                identical = False
    ref = O.gather_attention(q_all, pool_k, pool_v, gather, lens, np.arange(wl.batch), wl.attention.scaling, "bf16")
    got = f32(out[0])
    for b in rows:
        worst = max(worst, float(np.abs(got[b] - ref[b]).max()))
    return {"rows": len(rows), "identical": bool(identical), "attn_max_err": worst, "attn_tolerance": 2e-2,
            "what": "layer 0 of the last timed step: gather lists and visible lengths equal to the CPU oracle's, "
                    "attention against the oracle's over the same lists"}


def batched_arm(torch, capi, lib, dev, seed, barrier):
    """Config 3 shape: 32 requests with lengths uniform in [8192, 65536] in one shared pool with
    shuffled page tables, two layers (so that a step's touched bytes exceed L2); reports the
    kernels' durations and the L1 kernel's bandwidth at a batch where it is not latency bound."""
    import random
    rnd = random.Random(seed)
    lens = [rnd.randint(8192, 65536) for _ in range(32)]
    wl = build_workload(torch, dev, 3 + 5 + 2, seed, lengths=lens, n_layers=2)
    ms_total, stats, per_kernel, status, _, out, (lengths, _) = measure_device(torch, capi, lib, wl, 3, 5, barrier,
                                                                               min_timed_s=0.2)
    l1_bytes = sum(algorithmic_bytes(n + 1)["l1"] for n in lens)
    tot_bytes = sum(algorithmic_bytes(n + 1)["total"] for n in lens)
    peak, kind = peaks()
    us_layer = ms_total * 1e3 / (5 * wl.n_layers)
    parity = parity_check(torch, wl, out, lengths.cpu(), 3 + 5 - 1, rows=[0, 7, 19, 31])
    return {"workload": "cfg3: 32 requests, context uniform in [8192, 65536], shuffled pages, 2 layers",
            "tokens_in_cache": sum(lens), "us_per_decode_step_per_layer": us_layer,
            "tok_s_per_layer_stack": 32 / (us_layer * 1e-6 * N_LAYERS), "timing": stats,
            "kernel_us_per_launch": per_kernel, "device_status": status, "parity_checked": parity,
            "l1_roofline": {"bound": "hbm", "achieved": l1_bytes / (per_kernel["l1"] * 1e-6) / 1e9, "peak": peak,
                            "unit": "GB/s", "frac": l1_bytes / (per_kernel["l1"] * 1e-6) / 1e9 / peak,
                            "peak_kind": f"of {kind}", "algorithmic_bytes": l1_bytes,
                            "traffic": measured_traffic("l1_stream_kernel", "cfg3-32req")},
            "chain_hbm_frac_of_8TBs": tot_bytes / (us_layer * 1e-6) / 8e12}


def cfg4_arm(torch, dist, capi, lib, dev, rank, world, barrier, layers=8):
    """Config 4 shape: Llama-3.1-8B attention (32 q / 8 kv heads, d128, RoPE theta 5e5 with llama3
    scaling), 8 requests of 131 072 tokens, `layers` of its 32 layers, KV heads split over the ranks with
    an all-gather of the attention output after every layer inside the captured graph."""
    hkv, hq = HKV // world, HQ // world
    wl = build_workload(torch, dev, 3 + 4 + 2, seed=23, lengths=[CONTEXT - 1] * 8, n_layers=layers, hq=hq, hkv=hkv,
                        theta=5e5, llama3=True)
    out = torch.zeros(layers, 8, hq, D, dtype=torch.bfloat16, device=dev)
    full = torch.zeros(layers, world, 8, hq, D, dtype=torch.bfloat16, device=dev) if world > 1 else None

    def after(li):
        dist.all_gather_into_tensor(full[li], out[li])

    ms, stats, _, status, _, _, _ = measure_device(torch, capi, lib, wl, 3, 4, barrier,
                                                   after_layer=after if world > 1 else None, kernels=False,
                                                   min_timed_s=0.3, out=out)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    us_layer = ms * 1e3 / (4 * layers)
    res = {"workload": f"cfg4: Llama-3.1-8B attention shape, 8 requests x 131072 tokens, {layers} of 32 layers, "
                       f"KV heads split over {world} GPU(s), all-gather of the outputs per layer",
           "n_gpus": world, "kv_heads_per_gpu": hkv, "rows_per_gpu": 8 * hkv, "us_per_decode_step_per_layer": us_layer,
           "tok_s_32_layers": 8 / (us_layer * 1e-6 * 32), "timing": stats, "device_status": status,
           "launches_per_layer_step": int(lib.loda_last_decode_launches())}
    del wl, out
    torch.cuda.empty_cache()
    return res


def cfg5_arm(torch, capi, lib, dev, layers=6):
    """Config 5 shape: MLA attention on the shared latent (16 query heads on one 576-dim latent row per token
    that is key and, in its first 512 dims, value), 64-token pages, 16 requests of 131 072 tokens, `layers`
    layers (16 x 131 072 x 1 152 B = 2.4 GB per layer; a step touches ~26 MB per layer, so six layers exceed L2)."""
    wl = build_workload(torch, dev, 3 + 4 + 2, seed=31, lengths=[CONTEXT - 1] * 16, n_layers=layers, hq=16, hkv=1,
                        page=64, d=576, dv=512, shared_latent=True)
    ms, stats, _, status, _, _, _ = measure_device(torch, capi, lib, wl, 3, 4, lambda: torch.cuda.synchronize(),
                                                   kernels=False, min_timed_s=0.3)
    us_layer = ms * 1e3 / (4 * layers)
    n_pages = (CONTEXT + 63) // 64
    # per request: min/max rows of the far pool's pages (d' = 32: 128 B per page), the candidates' codes
    # ((96 + 32 + 2) pages x 64 tokens x 20 B), the latent rows of the 1 024 visible tokens (1 152 B each)
    alg = 16 * (n_pages * 128 + 130 * 64 * 20 + 1024 * 1152)
    peak, kind = peaks()
    res = {"workload": f"cfg5: MLA shared latent 576/512, 16 query heads, 16 requests x {CONTEXT} tokens, 64-token pages, "
                       f"{layers} layers", "us_per_decode_step_per_layer": us_layer,
           "tok_s_27_layers": 16 / (us_layer * 1e-6 * 27), "timing": stats, "device_status": status,
           "launches_per_layer_step": int(lib.loda_last_decode_launches()),
           "algorithmic_bytes_per_layer_step": alg,
           "hbm_frac": alg / (us_layer * 1e-6) / 1e9 / peak, "peak_kind": f"of {kind}"}
    del wl
    torch.cuda.empty_cache()
    return res


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


def reference_triton_arm(torch, dev, budget_s=240.0):
    """The reference's own production chain (its Triton selector and gather attention, unmodified, imported
    from baseline/_ref where tests/golden/make_golden_gpu.py --install put it) on this GPU at the
    workload's shape: one 131 072-token request, `layers` layers with their own pools (touched bytes per
    replay above the L2 size), the chain of all layers captured in one CUDA graph and replayed.  Page 16
    (this workload) and page 64 (the reference's production page).  None if the reference is not there."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "sparse_attn")):
        return {"unavailable": "baseline/_ref holds no install of the reference"}
    t_begin = time.time()
    # the reference's packages must not shadow this repository's: import under the reference's own names
    # from its install directory, in this process, before anything of the repository with those names
    # (the repository's copy lives under two-level-attention_b200.*, so the names do not collide)
    sys.path.insert(0, ref_dir)
    res = {}
    try:
        from types import SimpleNamespace

        from sparse_attn.cache import GraphReadyPagedRegionCache
        from sparse_attn.indexer.nfa_indexer import NFAIndexer
        from sparse_attn.indexer.nfa_layer_batch_selector import select_topk_for_layer_batched
        from sparse_attn.ops.paged_region_kernels import sparse_paged_attention_gather
        from sparse_attn.ops.paged_region_kernels_nfa import nfa_args
        from sparse_attn.policies.region_geometry import RegionGeometry
        for page, layers in ((16, 12), (64, 12)):
            if time.time() - t_begin > budget_s:
                res[f"page{page}"] = "skipped: time budget"
                continue
            args = nfa_args("tail")
            args.tia_block_size = page
            indexer = NFAIndexer(args)
            geometry = RegionGeometry(sink=4, near=4096, window=128, page=page, max_new_tokens=64)
            n_pre = CONTEXT - 1
            max_blocks = (CONTEXT + 64 + page - 1) // page + 2
            cache = GraphReadyPagedRegionCache(
                layers, geometry, max_requests=1, max_physical_pages=max_blocks + 8, max_blocks=max_blocks,
                max_visible_len=1024, max_query_tokens=1, num_kv_heads=HKV, num_query_heads=HQ,
                head_dim_k=D, head_dim_v=D, dtype=torch.bfloat16, device=dev)
            g = torch.Generator(device=dev).manual_seed(7)
            cache.add_request(0)
            for li in range(layers):
                kk = torch.randn(1, HKV, n_pre, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
                cache.write_prefill(li, 0, kk, torch.randn_like(kk))
                del kk
            cache.freeze(0, [False] * layers, [False] * layers)
            attention = SimpleNamespace(indexer=indexer, scaling=D ** -0.5)
            q = torch.randn(layers, 1, HQ, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
            k1 = torch.randn(layers, 1, HKV, 1, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
            q2r = torch.zeros(1, dtype=torch.int32, device=dev)
            cache.new_step([0])
            cache.plan_common([0])
            outs = []

            def chain():
                for li in range(layers):
                    select_topk_for_layer_batched(cache, li, [0], q[li], attention=attention,
                                                  decode_write=(k1[li], k1[li], cache.slot_mapping_for_layer(li)[:1]))
                    outs.append(sparse_paged_attention_gather(cache.layers[li], q[li], cache.gather_indices_for_layer(li),
                                                              cache.visible_lens_for_layer(li), q2r, scale=D ** -0.5))
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                for _ in range(3):
                    outs.clear()
                    chain()
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
            # eager timing (what the reference's launch plans give without a graph)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                outs.clear()
                chain()
            e1.record()
            torch.cuda.synchronize()
            entry = {"layers": layers, "eager_us_per_layer": e0.elapsed_time(e1) * 1e3 / (5 * layers),
                     "eager_is": "steady state of the reference's eager launch plans (its fast path outside a graph)"}
            try:
                graph = torch.cuda.CUDAGraph()
                outs.clear()
                with torch.cuda.graph(graph):
                    chain()
                graph.replay()
                torch.cuda.synchronize()
                e0.record()
                for _ in range(20):
                    graph.replay()
                e1.record()
                torch.cuda.synchronize()
                entry["graph_us_per_layer"] = e0.elapsed_time(e1) * 1e3 / (20 * layers)
                entry["graph_note"] = ("capture of the bare selector call: under capture the reference takes its full "
                                       "path, whose page-statistics pass covers every block on each replay; its engine "
                                       "captures the whole model step instead")
            except Exception as exc:      # noqa: BLE001
                entry["graph_us_per_layer"] = None
                entry["graph_note"] = f"{type(exc).__name__}: {exc}"[:200]
            res[f"page{page}"] = entry
            del cache, q, k1, outs
            torch.cuda.empty_cache()
        res["what"] = ("the reference's Triton selector (select_topk_for_layer_batched with the fused decode write) + "
                       "sparse_paged_attention_gather per layer, one 131072-token request, this GPU")
    except Exception as exc:      # noqa: BLE001
        res["unavailable"] = f"{type(exc).__name__}: {exc}"[:300]
    finally:
        sys.path.remove(ref_dir)
    return res


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


# ---- CPU arms ------------------------------------------------------------------------------------
_CPU = {}


def _cpu_head_task(kv):
    """One KV head of one layer-step on one host core: selection and attention with the CPU oracle."""
    import numpy as np

    from oracle import loda_oracle as O
    st = _CPU
    q = st["q"][kv * st["g"]:(kv + 1) * st["g"]]
    sel = O.select_request(q, st["k"][kv], st["length"], st["cfg"], D ** -0.5, index=st["index"][kv])
    ids = sel.logical[0]
    gather = np.full((1, 1, 1024), -1, np.int32)
    gather[0, 0, :len(ids)] = O.to_slots(ids, st["table"], PAGE)
    lens = np.array([[len(ids)]], np.int32)
    O.gather_attention(q[None], st["pool_k"][kv], st["pool_v"][kv], gather, lens, np.array([0]), D ** -0.5, "bf16")
    return len(ids)


def cpu_baseline(sample_steps=3, threads=None):
    """One layer of the workload on the host cores with the CPU oracle (index prebuilt, as the
    reference maintains its page statistics incrementally): the KV heads of the layer are dealt to
    worker processes, one per core, up to one per KV head."""
    import multiprocessing as mp

    import numpy as np

    from oracle import loda_oracle as O
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    workers = max(1, min(HKV, cores if threads is None else threads))
    rng = np.random.default_rng(0)
    length = CONTEXT
    g = HQ // HKV
    cfg1 = O.SelectorConfig(num_q_heads=g, num_kv_heads=1, max_blocks=(length + PAGE - 1) // PAGE + 8, block_size=PAGE)
    _CPU.update(g=g, length=length, cfg=cfg1, table=np.arange((length + PAGE - 1) // PAGE), k=[], index=[], pool_k=[],
                pool_v=[])
    for kv in range(HKV):
        k = O.bf16_rn(rng.standard_normal((length, 1, D), dtype=np.float32))
        v = O.bf16_rn(rng.standard_normal((length, 1, D), dtype=np.float32))
        _CPU["k"].append(k)
        _CPU["index"].append(O.build_index(k, length, cfg1))
        _CPU["pool_k"].append(k.reshape(-1, PAGE, 1, D).transpose(0, 2, 1, 3).copy())
        _CPU["pool_v"].append(v.reshape(-1, PAGE, 1, D).transpose(0, 2, 1, 3).copy())
    times = []
    ctx = mp.get_context("fork")
    _CPU["q"] = O.bf16_rn(rng.standard_normal((HQ, D), dtype=np.float32))
    with ctx.Pool(workers) as pool:
        pool.map(_cpu_head_task, range(HKV))                       # one untimed layer-step
    for s in range(sample_steps):
        _CPU["q"] = O.bf16_rn(rng.standard_normal((HQ, D), dtype=np.float32))
        with ctx.Pool(workers) as pool:                            # forked after q is set: the children see it
            t0 = time.perf_counter()
            pool.map(_cpu_head_task, range(HKV))
            times.append(time.perf_counter() - t0)
    per_layer = sum(times) / len(times)
    return {"value": 1.0 / (per_layer * N_LAYERS), "unit": "tok/s", "cores": workers, "kind": "port",
            "host_cores_available": cores, "us_per_step_per_layer": per_layer * 1e6, "layer_steps_timed": sample_steps,
            "sample": f"{sample_steps} decode steps of 1 of {N_LAYERS} layers at {CONTEXT} tokens (numpy oracle, "
                      f"selector index prebuilt, {HKV} KV heads over {workers} worker processes), scaled to "
                      f"{N_LAYERS} layers"}


def reference_cpu_code(budget_tokens=32768):
    """The reference's OWN CPU-runnable code for this path, imported unmodified from baseline/_ref and
    timed on the host cores (all torch threads): TIAIndexer.compute_score + compute_mask on a prebuilt
    index (sparse_attn/indexer/tia_indexer.py:64-136) and the CPU branch of
    sparse_paged_attention_gather (sparse_attn/ops/paged_region_kernels.py:1008-1041), one layer, one
    request of `budget_tokens` tokens (the dense fine-score pass of this indexer over 131 072 tokens needs
    several GB and tens of seconds per step: the sample is bounded)."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "sparse_attn")):
        return {"unavailable": "baseline/_ref holds no install of the reference"}
    import torch
    sys.path.insert(0, ref_dir)
    try:
        from sparse_attn.cache.paged_region_cache import GraphReadyPagedRegionLayer
        from sparse_attn.indexer.tia_indexer import TIAIndexer
        from sparse_attn.ops import paged_region_kernels as gat
        from sparse_attn.ops.paged_region_kernels_nfa import nfa_args
        from sparse_attn.policies.region_geometry import RegionGeometry
        args = nfa_args("tail")
        args.tia_block_size = PAGE
        ix = TIAIndexer(args)
        n = budget_tokens
        g = torch.Generator().manual_seed(0)
        k = torch.randn(1, n, HKV, D, generator=g).bfloat16()
        v = torch.randn(1, n, HKV, D, generator=g).bfloat16()
        q = torch.randn(1, 1, HQ, D, generator=g).bfloat16()
        cu = torch.tensor([0, n])
        index = ix.prepare_index(k, cu)
        pages = n // PAGE
        layer = GraphReadyPagedRegionLayer(geometry=RegionGeometry(page=PAGE), max_physical_pages=pages,
                                           num_kv_heads=HKV, head_dim_k=D, head_dim_v=D, dtype=torch.bfloat16,
                                           device="cpu")
        table = torch.arange(pages, dtype=torch.int32)
        gat.paged_write_prefill(layer, k.permute(0, 2, 1, 3).contiguous(), v.permute(0, 2, 1, 3).contiguous(), table)
        q2r = torch.zeros(1, dtype=torch.int32)
        times = []
        for _ in range(3):
            t0 = time.perf_counter()
            score = ix.compute_score(q, torch.tensor([n - 1]), index, D ** -0.5)
            mask = ix.compute_mask(torch.tensor([n - 1]), score)            # [1, 1, Hkv, n] bool
            gather = torch.full((1, HKV, 1024), -1, dtype=torch.int32)
            lens = torch.zeros((1, HKV), dtype=torch.int32)
            for kv in range(HKV):
                ids = torch.nonzero(mask[0, 0, kv]).flatten()[:1024].int()
                gather[0, kv, :len(ids)] = ids
                lens[0, kv] = len(ids)
            gat.sparse_paged_attention_gather(layer, q[0], gather, lens, q2r, scale=D ** -0.5)
            times.append(time.perf_counter() - t0)
        per = min(times[1:]) if len(times) > 1 else times[0]
        return {"us_per_step_per_layer": per * 1e6, "tokens": n, "cores": torch.get_num_threads(),
                "what": "TIAIndexer.compute_score + compute_mask (index prebuilt) + CPU branch of "
                        "sparse_paged_attention_gather, the reference's own code, bf16, one layer"}
    except Exception as exc:      # noqa: BLE001
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    finally:
        sys.path.remove(ref_dir)


def workload_config(world, shard):
    note = ("single GPU" if world == 1 else
            "KV heads of the request split over the GPUs, all-gather of the attention output per layer (NCCL) inside "
            "the timed region" if shard == "kvhead" else
            "one independent request per GPU, no data-path collective" if shard == "request" else
            "pages of the request round robin over the GPUs")
    return {"workload": "cfg2-qwen3-8b-128k", "layers": N_LAYERS, "context": CONTEXT, "batch": 1,
            "page": PAGE, "heads": f"{HQ}q/{HKV}kv", "head_dim": D, "selector": SELECTOR,
            "l2_flush": "none needed: 36 layers x 12.8 MB touched per step exceeds the 126 MB L2",
            "sharding": note}


def run_reference(args, rank, world):
    """--impl reference: the CPU form of the path on the host cores.  Every step of this arm is one
    layer-step of the workload (one of its 36 layers at 131 072 tokens) — W untimed and K timed ones really
    run — and `value` scales their mean to the 36 layers of a full step."""
    if rank != 0:
        return
    t0 = time.perf_counter()
    k = max(1, min(args.steps, 30))
    base = cpu_baseline(sample_steps=k)
    if not args.skip_reference_code:
        base["reference_code"] = reference_cpu_code()
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tok/s", "n_gpus": world,
        "steps": k, "warmup": 1, "ms_per_step": base["us_per_step_per_layer"] * 1e-3,
        "step_is": "one layer-step (1 of 36 layers); value = 1 / (36 x mean step time)",
        "higher_is_better": True, "scaling": "strong" if args.shard == "kvhead" else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world, args.shard),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's production path is GPU-only Triton; its CPU form is the numpy restatement under "
                "oracle/ (pinned against that Triton path), run over the host cores; cpu_baseline.reference_code "
                "times the reference's own PyTorch indexer and CPU gather attention",
        "wall_s": None}
    line["wall_s"] = round(time.perf_counter() - t0, 1)
    print(json.dumps(line), flush=True)


def main():
    global N_LAYERS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-dense", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-batched", action="store_true")
    ap.add_argument("--only-batched", action="store_true",
                    help="run only the 32-request arm and print its object (small captures of its kernels under a profiler)")
    ap.add_argument("--skip-tls", action="store_true")
    ap.add_argument("--skip-cfg4", action="store_true")
    ap.add_argument("--skip-cfg5", action="store_true")
    ap.add_argument("--only-cfg5", action="store_true", help="run only the latent-attention arm and print its object")
    ap.add_argument("--skip-reference-triton", action="store_true")
    ap.add_argument("--skip-parity", action="store_true")
    ap.add_argument("--skip-reference-code", action="store_true",
                    help="reference arm: leave out the timing of the reference's own PyTorch CPU code")
    ap.add_argument("--shard", default="kvhead", choices=("kvhead", "request", "sequence"),
                    help="multi-GPU partition: the KV-head groups of ONE request split over the GPUs with an all-gather "
                         "of the attention output per layer (strong scaling, default), one independent request per GPU "
                         "(weak scaling, no collective), or the pages of ONE request dealt round robin over the GPUs "
                         "with NCCL all-gathers between the stages")
    ap.add_argument("--layers", type=int, default=N_LAYERS,
                    help="profiling aid: fewer layers than the 36 of the named workload (not a bench line)")
    ap.add_argument("--min-timed-s", type=float, default=MIN_TIMED_S)
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
    hq, hkv = HQ, HKV
    if kvhead:
        shard = mod("sharding").kv_head_shard(HQ, HKV, world, rank)
        hq, hkv = shard.num_q_heads, shard.num_kv_heads      # this rank's heads of the same request

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
    if args.only_cfg5:
        if rank == 0:
            print(json.dumps({"cfg5": cfg5_arm(torch, capi, lib, dev)}), flush=True)
        return
    if args.only_batched:
        if rank == 0:
            print(json.dumps({"batched": batched_arm(torch, capi, lib, dev, 5, lambda: torch.cuda.synchronize())}), flush=True)
        return
    if args.shard == "sequence" and world > 1:
        run_sequence_sharded(torch, dist, capi, lib, dev, local, rank, world, K, W, barrier)
        dist.barrier()
        dist.destroy_process_group()
        return
    e2e_steps = K
    total = W + K + W + e2e_steps + 8
    wl = build_workload(torch, dev, total, seed=11 + (0 if kvhead else rank), hq=hq, hkv=hkv)
    cache = wl.cache
    # KV-head sharding: after every layer the ranks exchange their heads' outputs (what the output
    # projection of the surrounding model needs), inside the captured graph and the timed region
    out = torch.zeros(N_LAYERS, 1, hq, D, dtype=torch.bfloat16, device=dev)
    gathered = torch.zeros(N_LAYERS, world, 1, hq, D, dtype=torch.bfloat16, device=dev) if kvhead else None

    def after_layer(li):
        dist.all_gather_into_tensor(gathered[li], out[li])

    if kvhead:      # NCCL warm-up outside any capture
        warm = torch.zeros(world, 4, device=dev)
        dist.all_gather_into_tensor(warm, torch.ones(4, device=dev))
    sampler = ClockSampler(local)
    sampler.start()
    ms_total, stats, per_kernel, status, stream, out, (lengths, slots) = measure_device(
        torch, capi, lib, wl, W, K, barrier, after_layer=after_layer if kvhead else None,
        min_timed_s=args.min_timed_s, out=out)
    clocks = sampler.stop()

    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / K
    tok_s = (1.0 if kvhead else world) / (ms_per_step * 1e-3)
    launches_per_layer = int(lib.loda_last_decode_launches()) or 2
    ctas_per_row = int(lib.loda_last_decode_cluster())
    parity = None
    if not args.skip_parity and rank == 0:
        parity = parity_check(torch, wl, out, lengths.cpu(), W + K - 1)

    # ---- end to end through the public Python API with host buffers ----------------
    base_s = W + K
    hq_ = wl.q[base_s:base_s + W + e2e_steps].cpu().pin_memory()
    hk_ = wl.k[base_s:base_s + W + e2e_steps].cpu().pin_memory()
    hv_ = wl.v[base_s:base_s + W + e2e_steps].cpu().pin_memory()
    attn_objs = [type(wl.attention)(indexer=wl.indexer, scaling=wl.attention.scaling, layer_idx=li)
                 for li in range(N_LAYERS)]
    runner = mod("sparse_attn.engine.graph_runner").DecodeGraphRunner(
        cache, attn_objs, 1, after_layer=(lambda li, o: dist.all_gather_into_tensor(gathered[li], o)) if kvhead else None)

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

    line = None
    if rank == 0:
        peak, peak_kind = peaks()
        ab = algorithmic_bytes(CONTEXT, hkv=hkv, hq=hq)
        us_layer = ms_per_step * 1e3 / N_LAYERS
        if launches_per_layer == 1:
            # one launch per layer-step does everything: its average duration is the chain's time per layer
            # (under KV-head sharding that time also holds the all-gather that follows each launch)
            per_kernel["decode_step"] = us_layer
            ab["decode_step"] = ab["total"]
            dominant = "decode_step"
        else:
            dominant = max(("select", "attn"), key=per_kernel.get)
        achieved = ab[dominant] / (per_kernel[dominant] * 1e-6) / 1e9
        dense = {"skipped": True} if args.skip_dense or world > 1 else dense_decode_us(torch, dev)
        dense_times = [v for v in dense.values() if isinstance(v, float)]
        fastest = min(dense_times) if dense_times else None
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": True,
            # the default series (KV heads over the ranks) keeps the total work fixed as N grows, N = 1 included
            "scaling": "strong" if args.shard == "kvhead" else "weak",
            "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world, args.shard),
            "kv_heads_per_gpu": hkv,
            "us_per_decode_step_per_layer": us_layer,
            "timing": stats,
            "kernel_us_per_launch": per_kernel,
            "algorithmic_bytes_per_layer_step": ab,
            "chain_hbm_frac_of_8TBs": ab["total"] / (us_layer * 1e-6) / 8e12,
            "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         "traffic": measured_traffic(dominant, "cfg2-qwen3-8b-128k") if world == 1 else None},
            "dense_decode": {"us_per_layer": dense, "fastest_us_per_layer": fastest,
                             "ours_over_dense": (us_layer / fastest) if fastest else None},
            "parity_checked": parity,
            "e2e": None if args.skip_e2e else {
                "value": (1 if kvhead else world) * 1e3 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": K * stats["replays"] * N_LAYERS * launches_per_layer, "device_status": status,
            "clocks": clocks, "launches_per_layer_step": launches_per_layer,
            "ctas_per_row": ctas_per_row if launches_per_layer == 1 else None,
        }
    del wl, runner, cache, out, hq_, hk_, hv_
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.skip_batched:
        line["batched"] = batched_arm(torch, capi, lib, dev, 5, lambda: torch.cuda.synchronize())
        torch.cuda.empty_cache()
    if not args.skip_cfg4 and (world == 1 or kvhead):
        res = cfg4_arm(torch, dist, capi, lib, dev, rank, world, barrier)
        if rank == 0:
            line["cfg4"] = res
    if rank == 0:
        if not args.skip_cfg5 and world == 1:
            torch.cuda.empty_cache()
            line["cfg5"] = cfg5_arm(torch, capi, lib, dev)
        if not args.skip_tls and world == 1:
            torch.cuda.empty_cache()
            line["tls_chain"] = tls_chain_arm(torch, dev)
        if not args.skip_reference_triton and world == 1:
            torch.cuda.empty_cache()
            line["reference_triton"] = reference_triton_arm(torch, dev)
        if not args.skip_cpu_baseline and world == 1:
            # in a fresh process: the worker pool of the CPU arm forks, which a process holding a CUDA context must not
            res = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "3"],
                                 capture_output=True, text=True, timeout=900)
            try:
                line["cpu_baseline"] = json.loads(res.stdout.strip().splitlines()[-1])["cpu_baseline"]
            except (IndexError, ValueError, KeyError):
                line["cpu_baseline"] = {"unavailable": (res.stderr or res.stdout)[-300:]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
