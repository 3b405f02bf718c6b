"""Sparse gather attention over a contiguous KV cache.

Mirrors SparseMHAInterface (reference: tls_attn/ops/sparse_mha.py:128-180; its
PyTorch statement ``ref_attn`` :199-232): q [B, 1, Hq, D], k / v
[maxB, S, Hkv, D], token_indices [B, Hkv, topk] with -1 marking a hole;
returns [B, 1, Hq, Dv] bf16.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _contiguous


class SparseMHAInterface:
    def __init__(self, num_heads: int, num_kv_heads: int, dim_k: int, dim_v: int, topk: int,
                 scaling: Optional[float] = None) -> None:
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.group_size = num_heads // num_kv_heads
        self.dim_k, self.dim_v, self.topk = dim_k, dim_v, topk
        self.scaling = dim_k ** -0.5 if scaling is None else scaling

    def forward(self, q, k, v, token_indices):
        o = torch.empty((q.shape[0], 1, self.num_heads, self.dim_v), dtype=torch.bfloat16, device=q.device)
        self.forward_with_buffer(q, k, v, token_indices, o)
        return o

    def forward_with_buffer(self, q, k, v, token_indices, o):
        batch = q.shape[0]
        if token_indices.shape != (batch, self.num_kv_heads, self.topk):
            raise ValueError("token_indices must be [B, Hkv, topk]")
        rt = _contiguous.runtime(q, k, v, self.num_heads, self.num_kv_heads, self.topk)
        idx = token_indices.to(torch.int32)
        gather = torch.where(idx >= 0, idx + rt["row_base"], idx).contiguous()      # slot = b * S + token
        lens = torch.full((batch, self.num_kv_heads), self.topk, dtype=torch.int32, device=q.device)
        _contiguous.attend(rt, q, gather, lens, self.scaling, o.view(batch, self.num_heads, self.dim_v))
