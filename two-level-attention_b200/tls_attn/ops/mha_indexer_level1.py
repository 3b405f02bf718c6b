"""Level-1 indexer: bound score of every key block and the top-k blocks.

Mirrors MHAIndexerLevel1Interface (reference: tls_attn/ops/mha_indexer_level1.py:186-249; PyTorch
statement ``ref_indexer_topk`` :252-272): q [B, 1, Hq, D], k_min / k_max [maxB, S / block, Hkv, D],
lengths [maxB] int32 in blocks -> (scores fp32 [B, Hkv, max_len], topk_scores fp32 [B, Hkv, topk],
topk_indices int32 [B, Hkv, topk]).  The last ``sliding_blocks`` blocks of a sequence score -inf;
missing top-k entries are (-inf, -1); ties go to the lower block.
"""
from __future__ import annotations

from typing import Optional

import torch

from ... import _capi
from . import _checks


class MHAIndexerLevel1Interface:
    def __init__(self, num_heads: int, num_kv_heads: int, dim_k: int, topk: int, sliding_blocks: int,
                 scaling: Optional[float] = None) -> None:
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.group_size = num_heads // num_kv_heads
        self.dim_k, self.topk, self.sliding_blocks = dim_k, topk, sliding_blocks
        self.scaling = dim_k ** -0.5 if scaling is None else scaling

    def forward(self, q, k_min, k_max, lengths):
        batch = q.shape[0]
        max_length = max(int(lengths.amax().item()), 1)      # host read, as in the reference's forward
        dev = q.device
        scores = torch.full((batch, self.num_kv_heads, max_length), float("-inf"), dtype=torch.float32, device=dev)
        topk_scores = torch.zeros((batch, self.num_kv_heads, self.topk), dtype=torch.float32, device=dev)
        topk_indices = torch.zeros((batch, self.num_kv_heads, self.topk), dtype=torch.int32, device=dev)
        self.forward_with_buffer(q, k_min, k_max, lengths, scores, topk_scores, topk_indices)
        return scores, topk_scores, topk_indices

    def forward_with_buffer(self, q, k_min, k_max, lengths, scores, topk_scores, topk_indices):
        _checks.need_bf16_cuda(q=q, k_min=k_min, k_max=k_max)
        _checks.need_i32("lengths", lengths)
        batch = q.shape[0]
        if tuple(q.shape[-2:]) != (self.num_heads, self.dim_k):
            raise ValueError("q must be [B, 1, Hq, dim_k]")
        if k_min.shape != k_max.shape or tuple(k_min.shape[2:]) != (self.num_kv_heads, self.dim_k) or k_min.shape[0] < batch:
            raise ValueError("k_min / k_max must be [max_batch, blocks, Hkv, dim_k]")
        if scores.dim() != 3 or tuple(scores.shape[:2]) != (batch, self.num_kv_heads):
            raise ValueError("scores must be [B, Hkv, max_length]")
        _checks.need_f32("scores", scores, scores.shape)
        _checks.need_f32("topk_scores", topk_scores, (batch, self.num_kv_heads, self.topk))
        _checks.need_i32("topk_indices", topk_indices)
        _capi.check(_capi.lib().loda_tls_level1(
            _capi.ptr(q), _capi.ptr(k_min), _capi.ptr(k_max), _capi.ptr(lengths), _capi.ptr(scores),
            _capi.ptr(topk_scores), _capi.ptr(topk_indices), batch, self.num_heads, self.num_kv_heads, self.dim_k,
            k_min.shape[1], scores.shape[2], self.topk, self.sliding_blocks, float(self.scaling),
            _capi.current_stream()))
