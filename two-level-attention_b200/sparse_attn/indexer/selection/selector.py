"""What a selector hands to its consumers: per (request, kv head) a compact, ascending list of
logical token ids.

The type and the function have the names, fields and meaning of the reference's
(sparse_attn/indexer/selection/selector.py:6-66) so that callers written against it keep working:
``TokenSelection`` unpacks into ``(indices, counts)``, ``valid()`` marks the used places,
``to_mask()`` rebuilds a dense mask for checks, ``canonical_selection`` turns a padded id list with
repeats into that form.  They are host-side conveniences on torch tensors (parity checks, adapters);
the decode path itself reads the kernels' buffers and calls none of them.
"""
from __future__ import annotations

from typing import NamedTuple

import torch


class TokenSelection(NamedTuple):
    """indices [B, Hkv, K] int32: the selected token ids of a row, ascending and without repeats, in
    its first ``counts[b, h]`` places (0 behind them); counts [B, Hkv] int32.  Sink and window tokens
    are not listed: their consumers add them."""
    indices: torch.Tensor
    counts: torch.Tensor

    def valid(self):
        """[B, Hkv, K] bool: True in the used places of every row."""
        places = torch.arange(self.indices.size(-1), device=self.indices.device)
        return places.lt(self.counts.unsqueeze(-1))

    def to_mask(self, capacity):
        """[B, Hkv, capacity] bool: True at the listed token ids (for tests and diagnostics)."""
        mask = self.indices.new_zeros((*self.counts.shape, capacity), dtype=torch.bool)
        b, h, place = self.valid().nonzero(as_tuple=True)
        mask[b, h, self.indices[b, h, place].long()] = True
        return mask


def canonical_selection(ids, valid, capacity, width=None):
    """The ids of every row that are flagged valid and lie in [0, capacity), ascending, each once, as
    a ``TokenSelection`` of ``width`` places (default: as many as ``ids`` has).  A row with more
    distinct ids than places keeps its lowest ones: callers size ``width`` so that this never happens."""
    if ids.dim() != 3 or tuple(valid.shape) != tuple(ids.shape) or capacity < 1:
        raise ValueError(f"canonical_selection needs ids and valid of one shape [B, Hkv, K] and capacity >= 1 "
                         f"(ids {tuple(ids.shape)}, valid {tuple(valid.shape)}, capacity {capacity})")
    k = ids.size(-1)
    width = k if width is None else min(int(width), k)
    # one sort brings the usable ids to the front in ascending order (everything else becomes `capacity`);
    # an id is kept where it differs from its left neighbour; kept ids move to their rank by a scatter
    usable = valid & ids.ge(0) & ids.lt(capacity)
    ordered, _ = torch.where(usable, ids, torch.full_like(ids, capacity)).sort(dim=-1)
    first = ordered.lt(capacity)
    first[..., 1:] &= ordered[..., 1:].ne(ordered[..., :-1])
    rank = first.cumsum(-1) - 1
    keep = first & rank.lt(width)
    out = ordered.new_zeros((*ids.shape[:-1], width + 1))
    out.scatter_(-1, torch.where(keep, rank, torch.full_like(rank, width)), torch.where(keep, ordered, torch.zeros_like(ordered)))
    counts = keep.sum(-1, dtype=torch.int32)
    return TokenSelection(out[..., :width].to(torch.int32).contiguous(), counts.contiguous())
