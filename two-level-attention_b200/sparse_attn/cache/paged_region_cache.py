"""Fixed-address paged KV cache with the page index the selector streams.

Mirrors GraphReadyPagedRegionLayer / GraphReadyPagedRegionCache (reference:
sparse_attn/cache/paged_region_cache.py:60-319, 429-560, 795-1060): the same
constructor arguments, buffer names, layouts and request lifecycle (add ->
write_prefill per layer -> freeze -> plan_common / commit_step per decode step
-> remove).  Every device buffer is allocated once and keeps its address, so
a captured CUDA graph can be replayed while lengths, block tables and slot
mappings change underneath it.

In addition to the reference's buffers each layer owns the selector index that
the append kernel maintains (see include/loda_b200.h: page_mm, page_sum,
tail_code, tail_sz); it is allocated by ``ensure_index`` once the selector
configuration is known.
"""
from __future__ import annotations

import ctypes as C
import heapq
from dataclasses import dataclass, field

import torch

from ... import _capi
from ..._capi import FallbackRequired

INVALID_PAGE_IDX = -1
INVALID_GATHER_IDX = -1
PAD_SLOT = -1


@dataclass
class RequestState:
    """One request slot.  ``block_tables[layer]`` lists physical page ids by
    logical page; it only ever grows during the request's lifetime."""
    logical_length: int = 0
    prompt_length: int = 0
    block_tables: list = field(default_factory=list)
    index_len: list = field(default_factory=list)     # tokens covered by the selector index, per layer
    index_live: list = field(default_factory=list)    # index maintained by the append kernel since built
    skip_far_by_layer: list = field(default_factory=list)    # frozen per-layer region-skip decisions
    skip_near_by_layer: list = field(default_factory=list)
    frozen: bool = False


class GraphReadyPagedRegionLayer:
    """Per-layer physical arena [pages + 1, 1, Hkv, PAGE, D]; the last page is
    the all-zero PAD page that invalid block-table entries point to."""

    def __init__(self, *, geometry, max_physical_pages, num_kv_heads, num_query_heads=None,
                 head_dim_k, head_dim_v, dtype, device, shared_latent=False):
        self.geometry = geometry
        self.max_physical_pages = max_physical_pages
        self.PAD_PAGE_ID = max_physical_pages
        self.num_kv_heads = num_kv_heads
        self.num_query_heads = num_kv_heads if num_query_heads is None else num_query_heads
        self.head_dim_k = head_dim_k
        self.head_dim_v = head_dim_v
        self.dtype = dtype
        self.device = torch.device(device)
        total, page = max_physical_pages + 1, geometry.page
        self.kv_pool_k = torch.empty((total, 1, num_kv_heads, page, head_dim_k), dtype=dtype, device=device)
        # shared_latent: the value of a token is the first head_dim_v dims of its key row (multi-head latent
        # attention in its absorbed form: one latent per token serves as key and as value); kv_pool_v is
        # then a view of kv_pool_k and the kernels read a token's row once
        self.shared_latent = bool(shared_latent)
        if self.shared_latent:
            if head_dim_v > head_dim_k:
                raise ValueError("a shared latent needs head_dim_v <= head_dim_k")
            self.kv_pool_v = self.kv_pool_k[..., :head_dim_v]
        else:
            self.kv_pool_v = torch.empty((total, 1, num_kv_heads, page, head_dim_v), dtype=dtype, device=device)
        self.kv_pool_k[self.PAD_PAGE_ID].zero_()
        if not self.shared_latent:
            self.kv_pool_v[self.PAD_PAGE_ID].zero_()
        self.free_ids = list(range(max_physical_pages))
        heapq.heapify(self.free_ids)
        # selector index (ensure_index)
        self.page_mm = self.page_sum = self.tail_code = self.tail_sz = None

    def alloc_pages(self, count):
        if len(self.free_ids) < count:
            raise RuntimeError("graph-ready physical page pool exhausted")
        return [heapq.heappop(self.free_ids) for _ in range(count)]


class GraphReadyPagedRegionCache:
    INVALID_REQ_ID = -1
    paged_regions = True
    nfa_regions = True

    def __init__(self, n_layers, geometry, *, max_requests, max_physical_pages, max_blocks,
                 max_visible_len, max_query_tokens, num_kv_heads, num_query_heads=None,
                 head_dim_k, head_dim_v, dtype, device, visible_buckets=None, shared_latent=False):
        device = torch.device(device)
        if device.type != "cuda":
            raise FallbackRequired("the paged cache of this package lives on a CUDA device")
        self.device = device
        self.geometry = geometry
        self.n_layers = n_layers
        self.max_requests = max_requests
        self.max_blocks = max_blocks
        self.max_visible_len = max_visible_len
        self.active_visible_bucket = max_visible_len
        self.max_query_tokens = max_query_tokens
        self.num_kv_heads = num_kv_heads
        self.num_query_heads = num_kv_heads if num_query_heads is None else num_query_heads
        self.dtype = dtype
        self.layers = [
            GraphReadyPagedRegionLayer(
                geometry=geometry, max_physical_pages=max_physical_pages, num_kv_heads=num_kv_heads,
                num_query_heads=self.num_query_heads, head_dim_k=head_dim_k, head_dim_v=head_dim_v,
                dtype=dtype, device=device, shared_latent=shared_latent)
            for _ in range(n_layers)]
        self.states: dict[int, RequestState] = {}
        self.pending_lengths: dict[int, int] = {}
        self.active_req_ids = []
        pad = self.layers[0].PAD_PAGE_ID

        def full(shape, value, dtype):
            return torch.full(shape, value, dtype=dtype, device=device)

        self.block_table_buf = full((n_layers, max_requests, max_blocks), pad, torch.int32)
        # The per-step metadata (slots, query -> request row, lengths, request ids) is one block on the
        # device and one block of pinned host memory with the same layout, moved by ONE copy per step;
        # the buffers below are views of the device block.
        q_cap = max_query_tokens
        n32 = (n_layers + 2) * q_cap
        n32 += n32 & 1                                   # the 64-bit ids start on an 8-byte boundary
        self._meta_dev = torch.zeros(n32 + 4 * q_cap, dtype=torch.int32, device=device)
        self._meta_cpu = torch.zeros(n32 + 4 * q_cap, dtype=torch.int32).pin_memory()

        def carve(block):
            slots = block[:n_layers * q_cap].view(n_layers, q_cap)
            q2r = block[n_layers * q_cap:(n_layers + 1) * q_cap]
            lens = block[(n_layers + 1) * q_cap:(n_layers + 2) * q_cap]
            act = block[n32:n32 + 2 * q_cap].view(torch.int64)
            val = block[n32 + 2 * q_cap:n32 + 4 * q_cap].view(torch.int64)
            return slots, q2r, lens, act, val

        (self.slot_mapping_buf, self.query_to_req_buf, self.planned_lengths_buf, self.active_req_ids_buf,
         self.valid_req_ids_buf) = carve(self._meta_dev)
        self._cpu_slots, cpu_q2r, cpu_lens, cpu_act, cpu_val = carve(self._meta_cpu)
        self._cpu_slots.fill_(PAD_SLOT)
        cpu_q2r.fill_(-1)
        cpu_act.fill_(self.INVALID_REQ_ID)
        self._meta_dev.copy_(self._meta_cpu)
        self.gather_indices_buf = full((n_layers, max_requests, num_kv_heads, max_visible_len),
                                       INVALID_GATHER_IDX, torch.int32)
        self.visible_lens_buf = full((n_layers, max_requests, num_kv_heads), 0, torch.int32)
        self.status_buf = torch.zeros(1, dtype=torch.int32, device=device)
        # frozen region-skip decisions [layer, request slot], read by the selector kernels on the device
        # (reference: skip_far_layer_buf / skip_near_layer_buf, paged_region_cache.py:293-296)
        self.skip_far_layer_buf = torch.zeros((n_layers, max_requests), dtype=torch.int32, device=device)
        self.skip_near_layer_buf = torch.zeros((n_layers, max_requests), dtype=torch.int32, device=device)
        # pinned staging: one H2D copy per buffer per step
        self._cpu_block_table = torch.full((n_layers, max_requests, max_blocks), pad, dtype=torch.int32).pin_memory()
        # numpy views of the same pinned memory: scalar writes without tensor dispatch
        self._np_slots = self._cpu_slots.numpy()
        self._np_block_table = self._cpu_block_table.numpy()
        self._np_meta64 = (cpu_act.numpy(), cpu_val.numpy())
        self._np_meta32 = (cpu_lens.numpy(), cpu_q2r.numpy())
        self._runtime = None
        self._nfa_selector_workspace = {}
        # True: selector calls also write the best-first page lists and the L2
        # survivors before the union (parity checks); off on the hot path
        self.selector_diagnostics = False

    # -- accessors (reference: paged_region_cache.py:351-365) ----------------
    def gather_indices_for_layer(self, layer_idx):
        return self.gather_indices_buf[layer_idx]

    def visible_lens_for_layer(self, layer_idx):
        return self.visible_lens_buf[layer_idx]

    def slot_mapping_for_layer(self, layer_idx):
        return self.slot_mapping_buf[layer_idx]

    def selector_workspace(self):
        return self._nfa_selector_workspace

    # -- request lifecycle ---------------------------------------------------
    def _next_free_slot(self):
        for request_id in range(self.max_requests):
            if request_id not in self.states:
                return request_id
        raise RuntimeError("no free request slot")

    def add_request(self, request_id=None):
        if request_id is None:
            request_id = self._next_free_slot()
        if request_id < 0 or request_id >= self.max_requests:
            raise ValueError("request_id outside fixed batch capacity")
        if request_id in self.states:
            raise ValueError(f"request {request_id} already active")
        self.states[request_id] = RequestState(
            block_tables=[[] for _ in range(self.n_layers)],
            index_len=[0] * self.n_layers, index_live=[False] * self.n_layers,
            skip_far_by_layer=[False] * self.n_layers, skip_near_by_layer=[False] * self.n_layers)
        self.skip_far_layer_buf[:, request_id].zero_()
        self.skip_near_layer_buf[:, request_id].zero_()
        self._cpu_block_table[:, request_id].fill_(self.layers[0].PAD_PAGE_ID)
        self.block_table_buf[:, request_id].fill_(self.layers[0].PAD_PAGE_ID)
        return request_id

    def remove_request(self, request_id):
        state = self.states.pop(request_id, None)
        if state is None:
            return
        # pages go back only after every submitted read or write of them has finished
        torch.cuda.synchronize(self.device)
        self._cpu_block_table[:, request_id].fill_(self.layers[0].PAD_PAGE_ID)
        self.block_table_buf[:, request_id].fill_(self.layers[0].PAD_PAGE_ID)
        for layer_idx, table in enumerate(state.block_tables):
            for physical_id in table:
                heapq.heappush(self.layers[layer_idx].free_ids, physical_id)

    def _grow_table(self, state, request_id, layer_idx, n_pages, alloc=None):
        table = state.block_tables[layer_idx]
        if n_pages > self.max_blocks:
            raise ValueError("length exceeds fixed block-table capacity")
        if len(table) >= n_pages:
            return False
        new = alloc if alloc is not None else self.layers[layer_idx].alloc_pages(n_pages - len(table))
        lo = len(table)
        table.extend(new)
        self._cpu_block_table[layer_idx, request_id, lo:len(table)] = torch.tensor(new, dtype=torch.int32)
        return True

    def write_prefill(self, layer_idx, request_id, keys, values, physical_pages=None):
        """keys / values [1, Hkv, N, D]: scatter the prompt of one request into
        freshly allocated pages of this layer (``physical_pages`` forces the page
        ids, e.g. a shuffled free list)."""
        state = self.states[request_id]
        layer = self.layers[layer_idx]
        page = self.geometry.page
        if keys.ndim != 4 or keys.shape[0] != 1 or keys.shape[-2] < 1:
            raise ValueError("graph-ready prefill expects unpadded B1 KV")
        if keys.shape[1] != layer.num_kv_heads:
            raise ValueError("KV head count does not match arena")
        if keys.device != values.device or keys.dtype != values.dtype:
            raise ValueError("KV dtype/device mismatch")
        n = keys.shape[-2]
        required = (n + page - 1) // page
        if required > self.max_blocks:
            raise ValueError("prefill length exceeds fixed block-table capacity")
        if not state.block_tables[layer_idx]:
            if physical_pages is not None:
                physical_pages = [int(p) for p in physical_pages]
                if len(physical_pages) != required:
                    raise ValueError("physical_pages must cover the prompt exactly")
                taken = set(physical_pages)
                layer.free_ids = [p for p in layer.free_ids if p not in taken]
                heapq.heapify(layer.free_ids)
            self._grow_table(state, request_id, layer_idx, required, alloc=physical_pages)
            if state.prompt_length not in (0, n):
                raise ValueError("prefill length diverged across layers")
            state.prompt_length = n
            state.logical_length = n
        elif n != state.prompt_length:
            raise ValueError("prefill length diverged across layers")
        self.block_table_buf[layer_idx, request_id].copy_(self._cpu_block_table[layer_idx, request_id],
                                                          non_blocking=True)
        state.index_len[layer_idx] = 0
        state.index_live[layer_idx] = False
        from ..ops.paged_region_kernels import paged_write_prefill
        return paged_write_prefill(layer, keys, values, self.block_table_buf[layer_idx, request_id])

    def freeze(self, request_id, skip_far_list=None, skip_near_list=None):
        """End of prefill: the per-layer region-skip decisions of the request become fixed
        (reference: paged_region_cache.py:540-585; the gate policy that takes them is the caller's).
        A skipped region is neither scored nor selected from by that layer's selector."""
        state = self.states[request_id]
        skip_far_list = [False] * self.n_layers if skip_far_list is None else list(skip_far_list)
        skip_near_list = [False] * self.n_layers if skip_near_list is None else list(skip_near_list)
        if len(skip_far_list) != self.n_layers or len(skip_near_list) != self.n_layers:
            raise ValueError("freeze expects per-layer skip decisions")
        if state.logical_length == 0:
            raise ValueError("prefill before freeze")
        capacity_pages = (state.prompt_length + self.geometry.max_new_tokens
                          + self.geometry.page - 1) // self.geometry.page
        if capacity_pages > self.max_blocks:
            raise ValueError("prompt + max_new_tokens exceeds fixed block-table capacity")
        state.skip_far_by_layer = [bool(x) for x in skip_far_list]
        state.skip_near_by_layer = [bool(x) for x in skip_near_list]
        self.skip_far_layer_buf[:, request_id] = torch.tensor(state.skip_far_by_layer, dtype=torch.int32)
        self.skip_near_layer_buf[:, request_id] = torch.tensor(state.skip_near_by_layer, dtype=torch.int32)
        state.frozen = True

    # -- region helpers (reference: paged_region_cache.py:589-618) -------------
    def nfa_skip_signature(self, req_ids):
        """Per batch row the frozen (skip_far, skip_near) pairs of every layer; None for padding rows."""
        signature = []
        for request_id in req_ids:
            state = self.states.get(request_id) if request_id is not None and request_id >= 0 else None
            signature.append(None if state is None
                             else tuple(zip(state.skip_far_by_layer, state.skip_near_by_layer)))
        return tuple(signature)

    @staticmethod
    def nfa_region_mode(signature, layer_idx):
        """0 = mixed or nothing skipped, 1 = every live row skips far, 2 = near, 3 = both."""
        modes = [item[layer_idx] for item in signature if item is not None]
        if not modes or any(mode != modes[0] for mode in modes[1:]):
            return 0
        skip_far, skip_near = modes[0]
        if skip_far and skip_near:
            return 3
        return 1 if skip_far else 2 if skip_near else 0

    # -- per-step planning (reference: plan_common / commit_step) -------------
    def plan_common(self, active_req_ids, query_lengths=None):
        """Plan one decode token for every live row: allocate the page the new
        token falls in, refresh block tables, slot mappings and lengths on the
        device.  Request lengths only advance in ``commit_step``."""
        batch = len(active_req_ids)
        if batch > self.max_query_tokens:
            raise ValueError("batch exceeds fixed query metadata capacity")
        page = self.geometry.page
        self.active_req_ids = list(active_req_ids)
        self.pending_lengths.clear()
        act, val = self._np_meta64[0], self._np_meta64[1]
        lens, q2r = self._np_meta32[0], self._np_meta32[1]
        act[:batch] = self.INVALID_REQ_ID
        val[:batch] = 0
        lens[:batch] = 0
        q2r[:] = -1
        slots_np = self._np_slots
        slots_np[:, :batch] = PAD_SLOT
        for b, request_id in enumerate(active_req_ids):
            qlen = 1 if query_lengths is None else int(query_lengths[b])
            if request_id is None or request_id < 0 or request_id not in self.states or qlen == 0:
                continue
            if qlen != 1:
                raise ValueError("decode planning expects one query token per row")
            state = self.states[request_id]
            planned = state.logical_length + 1
            pos = planned - 1
            lp, off = divmod(pos, page)
            if min(map(len, state.block_tables)) <= lp:      # the token opens a page in some layer
                for layer_idx in range(self.n_layers):
                    if len(state.block_tables[layer_idx]) <= lp:
                        self._grow_table(state, request_id, layer_idx, lp + 1)
                        self.block_table_buf[layer_idx, request_id, lp:lp + 1].copy_(
                            self._cpu_block_table[layer_idx, request_id, lp:lp + 1], non_blocking=True)
            # the slot of the token in every layer at once (the pinned table mirrors the per-layer lists)
            slots_np[:, b] = self._np_block_table[:, request_id, lp] * page + off
            act[b] = request_id
            val[b] = request_id
            lens[b] = planned
            q2r[b] = b
            self.pending_lengths[request_id] = planned
        self._meta_dev.copy_(self._meta_cpu, non_blocking=True)      # one copy: slots, rows, lengths, ids

    def commit_step(self):
        for request_id, planned in self.pending_lengths.items():
            state = self.states[request_id]
            state.logical_length = planned
            for layer_idx in range(self.n_layers):
                if state.index_live[layer_idx]:
                    state.index_len[layer_idx] = planned
        self.pending_lengths.clear()

    def write_decode(self, layer_idx, key_states, value_states, slot_mapping):
        if key_states.ndim != 4 or key_states.shape[-2] != 1:
            raise ValueError("graph-ready decode KV must be one token per row")
        if key_states.shape[0] != slot_mapping.shape[0]:
            raise ValueError("request batch must match KV batch")
        from ..ops.paged_region_kernels import paged_write_decode
        return paged_write_decode(self.layers[layer_idx], key_states, value_states, slot_mapping)

    def get_seq_length(self, layer_idx=0):
        return max((s.logical_length for s in self.states.values()), default=0)

    def read_status(self):
        """Deferred device status word (host sync); clears it."""
        value = int(self.status_buf.item())
        self.status_buf.zero_()
        return value

    # -- selector runtime -----------------------------------------------------
    def ensure_index(self, indexer):
        """Allocate (once) the per-layer selector index, the scratch workspace and
        the C geometry for this cache + selector configuration."""
        lo0, lo1, dsub = indexer.subspace_ranges()
        key = (lo0, lo1, dsub, int(indexer.args.tia_block_size), int(indexer.args.tia_level1_topk),
               int(indexer.nt_near_pages), int(indexer.args.tia_level2_topk), indexer.sink_tokens,
               indexer.sliding_window_size, int(indexer.nt_near_len), indexer.nt_near_tokens,
               indexer.far_method, indexer.near_method)
        if self._runtime is not None:
            if self._runtime.key != key:
                raise ValueError("one cache serves one selector configuration")
            return self._runtime
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the selector index must be allocated before graph capture")
        self._runtime = SelectorRuntime(self, indexer, key)
        return self._runtime


def page_minmax_by_page(layer):
    """[max_requests, Hkv, pages, 2, d'] view-copy of a layer's page min / max statistics (min then max per
    logical page) out of the grouped device layout; for checks and diagnostics."""
    r, h, groups, cpr, gp, e = layer.page_mm.shape
    t = layer.page_mm.view(r, h, groups, 2, cpr // 2, gp, e).permute(0, 1, 2, 5, 3, 4, 6)
    return t.reshape(r, h, groups * gp, 2, (cpr // 2) * e)


def page_sum_by_page(layer):
    """[max_requests, Hkv, pages, d'] copy of a layer's page sums out of the grouped device layout."""
    r, h, groups, nc, gp, e = layer.page_sum.shape
    return layer.page_sum.permute(0, 1, 2, 4, 3, 5).reshape(r, h, groups * gp, nc * e)


class SelectorRuntime:
    """C structs and device buffers shared by every call on one cache."""

    def __init__(self, cache, indexer, key):
        indexer.require_supported()
        page = cache.geometry.page
        if int(indexer.args.tia_block_size) != page:
            raise FallbackRequired("selector block size must equal the cache page size")
        if cache.dtype != torch.bfloat16:
            raise FallbackRequired("only bf16 KV pools are implemented")
        if cache.geometry.sink != indexer.sink_tokens or cache.geometry.window != indexer.sliding_window_size:
            raise ValueError("cache geometry and selector disagree on sink / window")
        self.key = key
        lo0, lo1, dsub = indexer.subspace_ranges()
        layer0 = cache.layers[0]
        k1, nb_near = int(indexer.args.tia_level1_topk), int(indexer.nt_near_pages)
        g = _capi.Geometry(
            dtype=_capi.LODA_DTYPE_BF16, num_q_heads=cache.num_query_heads, num_kv_heads=cache.num_kv_heads,
            head_dim=layer0.head_dim_k, head_dim_v=layer0.head_dim_v, sub_dims=dsub, sub_lo0=lo0, sub_lo1=lo1,
            page=page, num_pages=layer0.max_physical_pages + 1, max_blocks=cache.max_blocks,
            max_requests=cache.max_requests, max_query_tokens=cache.max_query_tokens,
            max_visible=cache.max_visible_len, k_far=min(max(0, k1 - nb_near), cache.max_blocks),
            k_near=min(nb_near, cache.max_blocks), level2_topk=int(indexer.args.tia_level2_topk),
            sink=indexer.sink_tokens, swa=indexer.sliding_window_size, near_len=cache.geometry.near,
            pool_near_len=max(page, int(indexer.nt_near_len)),
            near_tokens_p1=0 if indexer.nt_near_tokens is None else int(indexer.nt_near_tokens) + 1,
            far_method={"minmax": _capi.FAR_MINMAX, "avg": _capi.FAR_AVG, "avg_top2": _capi.FAR_AVG_TOP2}[
                indexer.far_method],
            near_minmax=1 if indexer.near_method == "minmax" else 0)
        if indexer.nt_near_tokens is not None and int(indexer.nt_near_len) != cache.geometry.near:
            raise FallbackRequired("the numeric near-token quota needs nfa_near_len == RegionGeometry.near")
        self.geometry = g
        lib = _capi.lib()
        nbytes = lib.loda_workspace_bytes(C.byref(g))
        if nbytes == 0:
            _capi.check(_capi.LODA_ERR_UNSUPPORTED if "not" in lib.loda_last_error().decode()
                        else _capi.LODA_ERR_ARGUMENT)
        dev = cache.device
        self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        hkv, mq = cache.num_kv_heads, cache.max_query_tokens
        self.i_far = torch.zeros((mq, hkv, max(g.k_far, 1)), dtype=torch.int32, device=dev)
        self.i_near = torch.zeros((mq, hkv, max(g.k_near, 1)), dtype=torch.int32, device=dev)
        self.n_far = torch.zeros((mq, hkv), dtype=torch.int32, device=dev)
        self.n_near = torch.zeros((mq, hkv), dtype=torch.int32, device=dev)
        self.middle = torch.zeros((mq, hkv, g.level2_topk), dtype=torch.int32, device=dev)
        self.middle_counts = torch.zeros((mq, hkv), dtype=torch.int32, device=dev)
        self.layer_structs = []
        for li, layer in enumerate(cache.layers):
            # statistics in groups of 32 logical pages, chunk-major inside a group (include/loda_b200.h)
            groups = (cache.max_blocks + 31) // 32
            layer.page_mm = torch.zeros((cache.max_requests, hkv, groups, dsub // 4, 32, 8),
                                        dtype=cache.dtype, device=dev)
            layer.page_sum = torch.zeros((cache.max_requests, hkv, groups, dsub // 8, 32, 8),
                                         dtype=cache.dtype, device=dev)
            layer.tail_code = torch.zeros((g.num_pages, hkv, page, dsub // 2), dtype=torch.uint8, device=dev)
            layer.tail_sz = torch.zeros((g.num_pages, hkv, page, 2), dtype=cache.dtype, device=dev)
            self.layer_structs.append(_capi.Layer(
                pool_k=layer.kv_pool_k.data_ptr(), pool_v=layer.kv_pool_v.data_ptr(),
                page_mm=layer.page_mm.data_ptr(), page_sum=layer.page_sum.data_ptr(),
                tail_code=layer.tail_code.data_ptr(), tail_sz=layer.tail_sz.data_ptr(),
                block_table=cache.block_table_buf[li].data_ptr(),
                skip_far=cache.skip_far_layer_buf[li].data_ptr(),
                skip_near=cache.skip_near_layer_buf[li].data_ptr()))
        self.cache = cache

    def batch_struct(self, batch):
        c = self.cache
        return _capi.Batch(batch=batch, lengths=c.planned_lengths_buf.data_ptr(),
                           valid_req_ids=c.valid_req_ids_buf.data_ptr(),
                           active_req_ids=c.active_req_ids_buf.data_ptr())

    def selection_struct(self, gather, visible_lens, with_middle=True, with_page_lists=True, chained=False):
        """`with_page_lists` / `with_middle` add the optional diagnostic outputs
        (best-first page lists, L2 survivors before the union).  `chained`: the call directly follows
        a decode step of this library on the same batch metadata (LODA_SEL_CHAINED)."""
        pl = with_page_lists
        return _capi.Selection(
            flags=_capi.SEL_CHAINED if chained else 0,
            i_far=self.i_far.data_ptr() if pl else None, n_far=self.n_far.data_ptr() if pl else None,
            i_near=self.i_near.data_ptr() if pl else None, n_near=self.n_near.data_ptr() if pl else None,
            gather=gather.data_ptr(), visible_lens=visible_lens.data_ptr(),
            middle=self.middle.data_ptr() if with_middle else None,
            middle_counts=self.middle_counts.data_ptr() if with_middle else None)
