"""Dense decode attention over a contiguous KV cache (the prototype's dense arm).

Mirrors MHAInterface (reference: tls_attn/ops/mha.py:115-166): q [B, 1, Hq, D],
k / v [maxB, S, Hkv, D], lengths [maxB] int32; returns [B, 1, Hq, Dv] bf16.
Runs the gather-attention kernel over the identity token list.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _contiguous


class MHAInterface:
    def __init__(self, num_heads: int, num_kv_heads: int, dim_k: int, dim_v: int,
                 scaling: Optional[float] = None) -> None:
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.group_size = num_heads // num_kv_heads
        self.dim_k, self.dim_v = dim_k, dim_v
        self.scaling = dim_k ** -0.5 if scaling is None else scaling
        self._identity = {}

    def forward(self, q, k, v, lengths):
        o = torch.empty((q.shape[0], 1, self.num_heads, self.dim_v), dtype=torch.bfloat16, device=q.device)
        self.forward_with_buffer(q, k, v, lengths, o)
        return o

    def forward_with_buffer(self, q, k, v, lengths, o):
        batch, s = q.shape[0], k.shape[1]
        rt = _contiguous.runtime(q, k, v, self.num_heads, self.num_kv_heads, s)
        key = (batch, s, q.device.index)
        gather = self._identity.get(key)
        if gather is None:
            tok = torch.arange(s, dtype=torch.int32, device=q.device).view(1, 1, s)
            gather = (tok + rt["row_base"]).expand(batch, self.num_kv_heads, s).contiguous()
            self._identity = {key: gather}
        lens = lengths[:batch].to(torch.int32).view(batch, 1).expand(batch, self.num_kv_heads).contiguous()
        _contiguous.attend(rt, q, gather, lens, self.scaling, o.view(batch, self.num_heads, self.dim_v))
