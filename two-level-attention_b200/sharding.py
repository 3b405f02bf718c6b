"""Multi-GPU partitioning of the decode path: one process per GPU.

Every stage of the path is independent per (request, KV head) row
(reference: ``row = m * HKV + kv`` throughout
sparse_attn/indexer/nfa_layer_batch_selector.py, ``kv_head = head // G`` in
sparse_attn/ops/paged_region_kernels.py:280), so two partitions need no
collective on the data path:

* by request: each rank owns whole requests (its own cache);
* by KV-head group: rank r owns KV heads [r * Hkv / n, (r + 1) * Hkv / n) and
  their query heads, i.e. a cache with Hkv / n heads; block tables and lengths
  are replicated.  A full-width output needs one all-gather of [B, Hq / n, Dv]
  (8 KB at batch 1) — or none when a row-parallel output projection follows.

The helpers below are backend-agnostic (``nccl`` on GPUs, ``gloo`` in the CPU
tests).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    kv_lo: int
    kv_hi: int
    q_lo: int
    q_hi: int

    @property
    def num_kv_heads(self):
        return self.kv_hi - self.kv_lo

    @property
    def num_q_heads(self):
        return self.q_hi - self.q_lo


def kv_head_shard(num_q_heads, num_kv_heads, world, rank):
    """Contiguous KV-head group of `rank` and the query heads that read it."""
    if num_q_heads % num_kv_heads:
        raise ValueError("GQA requires num_q_heads % num_kv_heads == 0")
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} KV heads cannot be split evenly over {world} ranks")
    if not 0 <= rank < world:
        raise ValueError("rank outside the world")
    g = num_q_heads // num_kv_heads
    per = num_kv_heads // world
    return HeadShard(rank, world, rank * per, (rank + 1) * per, rank * per * g, (rank + 1) * per * g)


def request_shard(num_requests, world, rank):
    """Requests owned by `rank` (round robin, so that ragged lengths balance)."""
    return list(range(rank, num_requests, world))


def gather_head_outputs(local_out, group=None):
    """All-gather of per-rank attention outputs [B, Hq / n, Dv] into [B, Hq, Dv]
    (ranks hold consecutive head groups)."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def max_over_ranks(value, device, group=None):
    """The slowest rank's time: multi-GPU numbers are the max of device timings."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def lse_merge(outs, ms, zs):
    """Fixed-order log-sum-exp merge of normalised partial attention outputs.

    outs [R, ..., Dv] (each partial already divided by its own z), ms [R, ...]
    row maxima in the exp2 domain, zs [R, ...] sums.  Partials over disjoint
    token sets of the same query merge to the attention over the union; an empty
    partial has z = 0.  The order of R is the merge order, so every rank that
    merges the same list gets the same bits."""
    m = ms.max(dim=0).values
    safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp2(ms - safe) * zs                      # weight of every partial
    z = torch.zeros_like(m)
    o = torch.zeros_like(outs[0], dtype=torch.float32)
    for r in range(outs.shape[0]):
        z = z + w[r]
        o = o + outs[r].float() * w[r].unsqueeze(-1)
    return torch.where(z.unsqueeze(-1) > 0, o / z.unsqueeze(-1).clamp_min(1e-38), torch.zeros_like(o))


# ---------------------------------------------------------------------------
# sequence sharding of one long request over the GPUs (batch-1 long context)
# ---------------------------------------------------------------------------
def combine_disjoint_scores(local, group=None):
    """All-gather of the ranks' uint16 score rows followed by a bitwise OR.  Every page (level 1)
    and every candidate slot (level 2) is scored by exactly one rank and is 0 on the others, so
    the OR is the single-GPU score row, identical on every rank.  The rows travel as bytes (NCCL
    has no 16-bit integer type; a bitwise OR does not care)."""
    world = dist.get_world_size(group)
    mine = local.contiguous().view(torch.uint8)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine, group=group)
    out = parts[0]
    for r in range(1, world):
        out = torch.bitwise_or(out, parts[r])
    return out.view(local.dtype).view(local.shape)


class SequenceShard:
    """One GPU's view of a paged cache under sequence sharding: logical page p belongs to rank
    p % world.  The view owns a copy of the block tables in which the other ranks' pages are -1
    (a deployment would simply never allocate them), a geometry carrying (rank, world), its own
    selector workspace and its own gather list; the pools and the page statistics are the
    cache's.  The selector runs in four stages (methods below); between them the score rows of
    the ranks are combined (`combine_disjoint_scores`)."""

    def __init__(self, cache, indexer, rank, world):
        import ctypes as C

        from . import _capi
        if world < 2 or not 0 <= rank < world:
            raise ValueError("sequence sharding needs world >= 2 and 0 <= rank < world")
        self.cache, self.rank, self.world = cache, rank, world
        rt = cache.ensure_index(indexer)
        self.rt = rt
        g = _capi.Geometry()
        C.memmove(C.byref(g), C.byref(rt.geometry), C.sizeof(g))
        g.shard_rank, g.shard_count = rank, world
        self.geometry = g
        regions = (C.c_int64 * 4)()
        _capi.check(_capi.lib().loda_shard_workspace_regions(C.byref(g), regions))
        self.workspace = torch.zeros_like(rt.workspace)
        ws = self.workspace
        self.l1_scores = ws[regions[0]:regions[0] + regions[1]].view(torch.int16)
        self.l2_scores = ws[regions[2]:regions[2] + regions[3]].view(torch.int16)
        self.gather = torch.full_like(cache.gather_indices_for_layer(0), -1)
        self.visible_lens = torch.zeros_like(cache.visible_lens_for_layer(0))
        self.block_tables = torch.empty_like(cache.block_table_buf)
        self.layers = []
        for li, st in enumerate(rt.layer_structs):
            layer = _capi.Layer()
            C.memmove(C.byref(layer), C.byref(st), C.sizeof(layer))
            layer.block_table = self.block_tables[li].data_ptr()
            self.layers.append(layer)
        self.refresh_block_tables()

    def refresh_block_tables(self):
        """Mask the other ranks' pages out of a fresh copy of the cache's block tables."""
        bt = self.cache.block_table_buf
        page_ids = torch.arange(bt.shape[-1], device=bt.device)
        mine = (page_ids % self.world) == self.rank
        self.block_tables.copy_(torch.where(mine, bt, torch.full_like(bt, -1)))

    def owns_token(self, position):
        return (position // self.cache.geometry.page) % self.world == self.rank

    def _call(self, fn, layer_idx, batch, q, scale, with_status, gathered=False):
        import ctypes as C

        from . import _capi
        rt, cache = self.rt, self.cache
        sel = rt.selection_struct(self.gather, self.visible_lens, with_middle=False, with_page_lists=False)
        args = [C.byref(self.geometry), C.byref(self.layers[layer_idx]), C.byref(rt.batch_struct(batch)),
                _capi.ptr(q), float(scale), C.byref(sel)]
        if with_status:
            args.append(C.c_void_p(cache.status_buf.data_ptr()))
        if gathered is not False:                      # the selection stages take the stacked rows of all ranks (or NULL)
            args.append(_capi.ptr(gathered))
        args += [_capi.ptr(self.workspace), _capi.current_stream()]
        _capi.check(fn(*args))

    def l1_scores_stage(self, layer_idx, batch, q, scale):
        from . import _capi
        self._call(_capi.lib().loda_shard_l1_scores, layer_idx, batch, q, scale, False)

    def l1_select_stage(self, layer_idx, batch, q, scale, gathered=None):
        from . import _capi
        self._call(_capi.lib().loda_shard_l1_select, layer_idx, batch, q, scale, False, gathered)

    def l2_scores_stage(self, layer_idx, batch, q, scale):
        from . import _capi
        self._call(_capi.lib().loda_shard_l2_scores, layer_idx, batch, q, scale, True)

    def l2_select_stage(self, layer_idx, batch, q, scale, gathered=None):
        from . import _capi
        self._call(_capi.lib().loda_shard_l2_select, layer_idx, batch, q, scale, True, gathered)

    def exchange_buffers(self, batch):
        """Fixed-address buffers of the collective exchanges (allocated once per batch size): the stacked
        score rows of all ranks for both levels, this rank's packed partial attention (out bf16, then the
        (max, sum) pairs) and the stacked partials of all ranks."""
        store = self.__dict__.setdefault("_exchange", {})
        buf = store.get(batch)
        if buf is None:
            cache, dev, world = self.cache, self.cache.device, self.world
            hq, dv = cache.num_query_heads, cache.layers[0].head_dim_v
            out_bytes = batch * hq * dv * 2
            lse_off = (out_bytes + 15) // 16 * 16
            part_bytes = (lse_off + batch * hq * 2 * 4 + 15) // 16 * 16
            part = torch.zeros(part_bytes, dtype=torch.uint8, device=dev)
            buf = dict(
                l1=torch.zeros((world,) + tuple(self.l1_scores.shape), dtype=torch.int16, device=dev),
                l2=torch.zeros((world,) + tuple(self.l2_scores.shape), dtype=torch.int16, device=dev),
                part=part, parts=torch.zeros((world, part_bytes), dtype=torch.uint8, device=dev),
                out=part[:out_bytes].view(torch.bfloat16).view(batch, hq, dv),
                lse=part[lse_off:lse_off + batch * hq * 8].view(torch.float32).view(batch, hq, 2),
                lse_off=lse_off, part_bytes=part_bytes,
                merged=torch.zeros((batch, hq, dv), dtype=torch.float32, device=dev))
            store[batch] = buf
        return buf

    def attend_stage(self, layer_idx, batch, q, scale, out=None, lse=None):
        """Attention over this rank's tokens of the selection: (out [B, Hq, Dv] bf16, lse [B, Hq, 2])."""
        import ctypes as C

        from . import _capi
        cache = self.cache
        hq, dv = cache.num_query_heads, cache.layers[layer_idx].head_dim_v
        out = q.new_empty((batch, hq, dv)) if out is None else out
        lse = torch.empty((batch, hq, 2), dtype=torch.float32, device=q.device) if lse is None else lse
        _capi.check(_capi.lib().loda_gather_attend_lse(
            C.byref(self.geometry), C.byref(self.layers[layer_idx]), _capi.ptr(q), _capi.ptr(self.gather),
            _capi.ptr(self.visible_lens), _capi.ptr(cache.query_to_req_buf), batch, cache.max_requests, float(scale),
            _capi.ptr(out), _capi.ptr(lse), _capi.ptr(self.workspace), _capi.current_stream()))
        return out, lse


def sequence_sharded_decode_step(shard, layer_idx, req_ids, query_states, attention, group=None):
    """Selector and attention of one layer with the request's pages dealt round robin over the
    ranks: level-1 scores of the own pages, all-gather + OR, page selection (identical on every
    rank); level-2 logits of the own pages' candidates, all-gather + OR, token selection
    (identical); attention over the own tokens; all-gather of (out, max, sum) and a fixed-order
    log-sum-exp merge.  Three collectives (one all_gather_into_tensor each, into fixed buffers) and seven
    kernels per layer: the selecting CTAs OR the gathered rows while they load them, one kernel merges.  Returns (out [B, Hq, Dv] fp32, gather, visible_lens); the index lists are
    those of the single-GPU path with -1 at the other ranks' tokens.  The cache must have been
    planned for the step (plan_common) and hold the step's token (the owner of its page appends)."""
    import ctypes as C

    from . import _capi
    b = len(req_ids)
    q = query_states.contiguous()
    scale = float(attention.scaling)
    x = shard.exchange_buffers(b)
    # level 1: own pages' scores -> one all-gather of the rows -> selection on the OR of the ranks' rows
    shard.l1_scores_stage(layer_idx, b, q, scale)
    # (16-bit integers are not a collective dtype of the NCCL process group: the rows travel as bytes)
    dist.all_gather_into_tensor(x["l1"].view(torch.uint8), shard.l1_scores.view(torch.uint8), group=group)
    shard.l1_select_stage(layer_idx, b, q, scale, gathered=x["l1"])
    # level 2: own candidates' logits -> all-gather -> quota selection, hole fill and union
    shard.l2_scores_stage(layer_idx, b, q, scale)
    dist.all_gather_into_tensor(x["l2"].view(torch.uint8), shard.l2_scores.view(torch.uint8), group=group)
    shard.l2_select_stage(layer_idx, b, q, scale, gathered=x["l2"])
    # attention over the own tokens -> all-gather of (out, max, sum) -> fixed-order merge (one kernel)
    shard.attend_stage(layer_idx, b, q, scale, out=x["out"], lse=x["lse"])
    dist.all_gather_into_tensor(x["parts"], x["part"], group=group)
    hq, dv = x["out"].shape[1], x["out"].shape[2]
    _capi.check(_capi.lib().loda_lse_merge(_capi.ptr(x["parts"]), x["part_bytes"], x["lse_off"], shard.world, b * hq, dv,
                                           _capi.ptr(x["merged"]), _capi.current_stream()))
    return x["merged"], shard.gather, shard.visible_lens
