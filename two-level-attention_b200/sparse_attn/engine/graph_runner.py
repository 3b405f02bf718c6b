"""CUDA-graph replay of the attention path of a decode step.

Mirrors the capture contract of the reference's GraphRunner
(sparse_attn/engine/graph_runner.py:78-133 capture, :155-200 step): host-side
planning (``cache.plan_common``) refreshes lengths, slots and block tables in
fixed device buffers, then one graph replay runs, for every layer, the fused
append + L1 + L2 + gather attention chain.  The reference captures the whole
HF model; here only the path this package implements is captured, with the
per-layer query / key / value of the step arriving in fixed staging buffers
(what the projections + RoPE of the surrounding model would produce).
"""
from __future__ import annotations

import torch

from ..indexer.nfa_layer_batch_selector import decode_step_fused


class DecodeGraphRunner:
    def __init__(self, cache, attentions, batch, after_layer=None):
        """attentions: one object per layer with .indexer, .scaling, .layer_idx.
        after_layer(layer_idx, out): optional work captured behind a layer's attention (the all-gather of the
        heads' outputs when the KV heads are split over several GPUs)."""
        self.after_layer = after_layer
        if len(attentions) != cache.n_layers:
            raise ValueError("one attention module per cache layer")
        self.cache, self.attentions, self.batch = cache, attentions, batch
        dev, dt = cache.device, cache.dtype
        nl, hq, hkv = cache.n_layers, cache.num_query_heads, cache.num_kv_heads
        d, dv = cache.layers[0].head_dim_k, cache.layers[0].head_dim_v
        self.q = torch.zeros(nl, batch, hq, d, dtype=dt, device=dev)
        self.k = torch.zeros(nl, batch, hkv, 1, d, dtype=dt, device=dev)
        self.v = torch.zeros(nl, batch, hkv, 1, dv, dtype=dt, device=dev)
        self.out = torch.zeros(nl, batch, hq, dv, dtype=dt, device=dev)
        self.host_out = torch.zeros(nl, batch, hq, dv, dtype=dt).pin_memory()
        self.graph = None
        self.stream = torch.cuda.Stream(device=dev)
        self.replays = 0

    def _run_layers(self, req_ids):
        cache = self.cache
        for li, attention in enumerate(self.attentions):
            slots = cache.slot_mapping_for_layer(li)[:self.batch]
            # every layer but the first directly follows the decode step of the layer before it
            decode_step_fused(cache, li, req_ids, self.q[li], attention, (self.k[li], self.v[li], slots),
                              out=self.out[li], chained=li > 0 and self.after_layer is None)
            if self.after_layer is not None:
                self.after_layer(li, self.out[li])

    def capture(self, req_ids):
        """One eager step (builds the index of fresh prefills, warms every launch),
        then capture.  Both write the same token into the same slots: idempotent."""
        cache = self.cache
        cache.plan_common(req_ids)
        self._run_layers(req_ids)
        torch.cuda.synchronize(cache.device)
        self.stream.wait_stream(torch.cuda.current_stream())
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self.stream):
            with torch.cuda.graph(self.graph, stream=self.stream):
                self._run_layers(req_ids)
        torch.cuda.current_stream().wait_stream(self.stream)
        self._req_ids = list(req_ids)

    def step(self, q_host, k_host, v_host, req_ids=None):
        """q_host [L, B, Hq, D], k_host / v_host [L, B, Hkv, 1, D] in pinned host
        memory -> attention outputs [L, B, Hq, Dv] in pinned host memory."""
        cache = self.cache
        req_ids = self._req_ids if req_ids is None else req_ids
        if self.graph is None or list(req_ids) != self._req_ids:
            raise RuntimeError("capture() this batch layout first")
        with torch.cuda.stream(self.stream):
            self.q.copy_(q_host, non_blocking=True)
            self.k.copy_(k_host, non_blocking=True)
            self.v.copy_(v_host, non_blocking=True)
            cache.plan_common(req_ids)
            self.graph.replay()
            self.host_out.copy_(self.out, non_blocking=True)
        self.stream.synchronize()
        cache.commit_step()
        self.replays += 1
        return self.host_out
