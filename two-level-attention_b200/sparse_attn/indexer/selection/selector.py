"""Selection contract of the selector: compact logical token ids and the canonical union.

Same types and functions as the reference (sparse_attn/indexer/selection/selector.py:6-66):
``TokenSelection`` is a NamedTuple (callers unpack it) with ``valid()`` and ``to_mask()``;
``canonical_selection`` sorts, de-duplicates and packs a padded id list.  Host-side helpers on
torch tensors: they run where the tensors live and launch no kernel of this package.
"""
from typing import NamedTuple

import torch


class TokenSelection(NamedTuple):
    """indices [B, Hkv, K] int32: ascending unique token ids in the first counts[b, h] places,
    0 in the rest; counts [B, Hkv] int32 (sink / window tokens are not part of it)."""
    indices: torch.Tensor
    counts: torch.Tensor

    def valid(self):
        """[B, Hkv, K] bool: place < counts."""
        return torch.arange(self.indices.shape[-1], device=self.indices.device) < self.counts[..., None]

    def to_mask(self, capacity):
        """[B, Hkv, capacity] bool mask of the selected ids (diagnostics, tests)."""
        result = torch.zeros((*self.indices.shape[:-1], capacity + 1), dtype=torch.bool, device=self.indices.device)
        ids = torch.where(self.valid(), self.indices.long(), capacity)
        result.scatter_(-1, ids, True)
        return result[..., :capacity]


def canonical_selection(ids, valid, capacity, width=None):
    """ids[valid & 0 <= ids < capacity], sorted and de-duplicated, the first ``width`` kept
    (selector.py:41-66).  The caller guarantees width >= the number of distinct valid ids."""
    if ids.ndim != 3 or valid.shape != ids.shape or capacity < 1:
        raise ValueError(
            f"selection requires [B,Hkv,K] IDs/valid and positive capacity, "
            f"got ids.shape={ids.shape} valid.shape={valid.shape} capacity={capacity}")
    width = ids.shape[-1] if width is None else min(width, ids.shape[-1])
    ordered = torch.where(valid & (ids >= 0) & (ids < capacity), ids, capacity).sort(-1).values
    previous = torch.cat((torch.full_like(ordered[..., :1], -1), ordered[..., :-1]), -1)
    unique = (ordered < capacity) & (ordered != previous)
    packed = torch.where(unique, ordered, capacity).sort(-1).values[..., :width]
    count = (packed < capacity).sum(-1, dtype=torch.int32)
    return TokenSelection(torch.where(packed < capacity, packed, 0).to(torch.int32).contiguous(), count.contiguous())
