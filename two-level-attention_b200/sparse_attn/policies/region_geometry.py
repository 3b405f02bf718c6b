"""Token regions of a request: sink | far | near | sliding window.

The cache and the selector agree on where the regions of a request of a given length begin and
end.  Same constructor fields, defaults and error behaviour as the reference's dataclass
(sparse_attn/policies/region_geometry.py:5-23), so code written against it runs unchanged; the
device code derives the same boundaries from the same five numbers (`make_regions`).
"""
from __future__ import annotations

from dataclasses import dataclass, fields

_MAY_BE_ZERO = frozenset({"sink"})


def _positive_int(name, value):
    """Plain ints only (a bool is not a size); `sink` may be 0, everything else starts at 1."""
    floor = 0 if name in _MAY_BE_ZERO else 1
    if type(value) is bool or not isinstance(value, int) or value < floor:
        raise ValueError(f"invalid {name}: {value}")


@dataclass(frozen=True)
class RegionGeometry:
    sink: int = 4                # leading tokens that are always attended
    near: int = 4096             # tokens before the window that form the near region
    window: int = 128            # trailing tokens that are always attended
    page: int = 64               # tokens per page
    max_new_tokens: int = 512    # decode tokens a request may add to its prompt

    def __post_init__(self):
        for f in fields(self):
            _positive_int(f.name, getattr(self, f.name))

    def bounds(self, length):
        """(sink_hi, far_hi, near_hi): ends of the sink, the far and the near region, as token
        positions, for a request that holds `length` tokens.  The far region ends on a page
        boundary; short requests collapse the regions onto the sink's end."""
        sink_hi = length if length < self.sink else self.sink
        window_lo = length - self.window
        near_hi = window_lo if window_lo > sink_hi else sink_hi
        far_hi = (window_lo - self.near) // self.page * self.page       # floor, also below zero
        if far_hi < sink_hi:
            far_hi = sink_hi
        if far_hi > near_hi:
            far_hi = near_hi
        return sink_hi, far_hi, near_hi

    def pages_for(self, tokens):
        """Pages that hold `tokens` tokens."""
        return -(-tokens // self.page)
