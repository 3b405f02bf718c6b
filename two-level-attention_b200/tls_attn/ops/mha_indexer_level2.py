"""Level-2 indexer: softmax-mass score of every token of the chosen blocks and the top-k tokens.

Mirrors MHAIndexerLevel2Interface (reference: tls_attn/ops/mha_indexer_level2.py:217-290; PyTorch
statement ``ref_indexer_topk`` :293-395): q [B, 1, Hq, d'], k [maxB, S, Hkv, d'] (the tail
sub-dimensions), block_indices [B, Hkv, K1] int32 (-1 = hole), lengths [maxB] int32 in tokens ->
(scores fp32 [B, Hkv, K1 * block], indices int32 same shape, topk_scores fp32 [B, Hkv, K2],
topk_indices int32 [B, Hkv, K2]).  The tokens of the last ``sliding_blocks`` blocks come first
with score +inf; holes are (-inf, -1); ties go to the lower position.
"""
from __future__ import annotations

from typing import Optional

import torch

from ... import _capi
from . import _checks


class MHAIndexerLevel2Interface:
    def __init__(self, num_heads: int, num_kv_heads: int, dim_k: int, level1_topk: int, level2_topk: int,
                 block_size: int, sliding_blocks: int, scaling: Optional[float] = None) -> None:
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.group_size = num_heads // num_kv_heads
        self.dim_k, self.block_S = dim_k, block_size
        self.level1_topk, self.level2_topk, self.sliding_blocks = level1_topk, level2_topk, sliding_blocks
        self.scaling = dim_k ** -0.5 if scaling is None else scaling

    def forward(self, q, k, block_indices, lengths):
        batch, dev = q.shape[0], q.device
        n = self.level1_topk * self.block_S
        scores = torch.full((batch, self.num_kv_heads, n), float("-inf"), dtype=torch.float32, device=dev)
        indices = torch.full((batch, self.num_kv_heads, n), -1, dtype=torch.int32, device=dev)
        cummax = torch.full((batch, self.num_kv_heads, n), float("-inf"), dtype=torch.float32, device=dev)
        topk_scores = torch.zeros((batch, self.num_kv_heads, self.level2_topk), dtype=torch.float32, device=dev)
        topk_indices = torch.zeros((batch, self.num_kv_heads, self.level2_topk), dtype=torch.int32, device=dev)
        self.forward_with_buffer(q, k, block_indices, lengths, scores, indices, cummax, topk_scores, topk_indices)
        return scores, indices, topk_scores, topk_indices

    def forward_with_buffer(self, q, k, block_indices, lengths, scores, indices, cummax_scores, topk_scores,
                            topk_indices):
        _checks.need_bf16_cuda(q=q, k=k)
        _checks.need_i32("block_indices", block_indices)
        _checks.need_i32("lengths", lengths)
        _checks.need_i32("indices", indices)
        _checks.need_i32("topk_indices", topk_indices)
        batch = q.shape[0]
        n = self.level1_topk * self.block_S
        if tuple(q.shape[-2:]) != (self.num_heads, self.dim_k):
            raise ValueError("q must be [B, 1, Hq, dim_k]")
        if tuple(k.shape[2:]) != (self.num_kv_heads, self.dim_k) or k.shape[0] < batch:
            raise ValueError("k must be [max_batch, S, Hkv, dim_k]")
        if tuple(block_indices.shape) != (batch, self.num_kv_heads, self.level1_topk):
            raise ValueError("block_indices must be [B, Hkv, level1_topk]")
        _checks.need_f32("scores", scores, (batch, self.num_kv_heads, n))
        _checks.need_f32("cummax_scores", cummax_scores, (batch, self.num_kv_heads, n))
        _checks.need_f32("topk_scores", topk_scores, (batch, self.num_kv_heads, self.level2_topk))
        _capi.check(_capi.lib().loda_tls_level2(
            _capi.ptr(q), _capi.ptr(k), _capi.ptr(block_indices), _capi.ptr(lengths), _capi.ptr(scores),
            _capi.ptr(cummax_scores), _capi.ptr(indices), _capi.ptr(topk_scores), _capi.ptr(topk_indices), batch,
            self.num_heads, self.num_kv_heads, self.dim_k, k.shape[1], self.level1_topk, self.level2_topk,
            self.block_S, self.sliding_blocks, float(self.scaling), _capi.current_stream()))
