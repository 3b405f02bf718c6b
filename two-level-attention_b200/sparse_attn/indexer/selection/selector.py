"""Selection contract (reference: sparse_attn/indexer/selection/selector.py:6-38)."""
from dataclasses import dataclass

import torch


@dataclass
class TokenSelection:
    """``indices`` [..., K] ascending logical token ids, valid up to ``counts``."""
    indices: torch.Tensor
    counts: torch.Tensor

    def __post_init__(self):
        if self.indices.dtype != torch.int32 or self.counts.dtype != torch.int32:
            raise ValueError("TokenSelection expects int32 indices and counts")
        if self.indices.shape[:-1] != self.counts.shape:
            raise ValueError("counts must match the leading shape of indices")
