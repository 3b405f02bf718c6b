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
