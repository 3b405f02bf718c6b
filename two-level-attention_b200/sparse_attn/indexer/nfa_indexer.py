"""Immutable selector configuration and subspace index ranges.

Mirrors NFAIndexer (reference: sparse_attn/indexer/nfa_indexer.py:22-145): the
same attribute names on ``args`` are read, the same constraints are enforced
with ValueError, and combinations that the CUDA path does not implement raise
FallbackRequired instead of silently changing behaviour.
"""
from __future__ import annotations

import operator

import torch

from ..._capi import FallbackRequired


class NFAIndexer:
    def __init__(self, args, snapshot=None) -> None:
        self.args = args
        self.layer_idx = None
        self.sliding_window_size = int(getattr(args, "nfa_swa_size", 128))
        self.cmp_ratio = int(args.tia_level2_cmp_ratio)
        self.subspace = getattr(args, "nfa_subspace", "full")
        if self.subspace not in ("full", "rope", "nope", "tail", "random", "highfreq", "mla_rope"):
            raise ValueError(f"nfa_subspace: illegal value {self.subspace}")
        self.enable_subspace = bool(getattr(args, "nfa_enable_subspace", True)) and self.subspace != "full"
        self.l2_subspace = getattr(args, "nfa_l2_subspace", "same")
        if self.l2_subspace not in ("same", "full"):
            raise ValueError(f"nfa_l2_subspace: illegal value {self.l2_subspace}")
        self.head_dim = int(getattr(args, "head_dim", 192 if self.subspace == "mla_rope" else 128))
        self.far_method = getattr(args, "nfa_far_method", "minmax")
        self.near_method = getattr(args, "nfa_near_method", "avg")
        self.sink_tokens = int(getattr(args, "nfa_sink_tokens", 128))
        if self.sink_tokens < 0:
            raise ValueError("nfa_sink_tokens must be >= 0")
        if self.sliding_window_size < 1:
            raise ValueError("nfa_swa_size must be >= 1")
        block_size = int(args.tia_block_size)
        if self.sliding_window_size % block_size:
            raise ValueError("nfa_swa_size must be a multiple of tia_block_size")

        def quota(name, value, allow_off=False):
            if allow_off and isinstance(value, str) and value.strip().lower() == "off":
                return None
            if value is None:
                return None
            if isinstance(value, bool):
                raise ValueError(f"{name} must be an integer count, got {value!r}")
            try:
                return int(value) if isinstance(value, str) else operator.index(value)
            except (TypeError, ValueError, OverflowError) as exc:
                raise ValueError(f"{name} must be an integer count, got {value!r}") from exc

        near_tokens_raw = getattr(args, "nfa_near_tokens", None)
        self.nt_near_pages = quota("nfa_near_pages", getattr(args, "nfa_near_pages", None))
        self.nt_near_tokens = quota("nfa_near_tokens", near_tokens_raw, allow_off=True)
        self.nt_near_len = quota("nfa_near_len", getattr(args, "nfa_near_len", None))
        near_tokens_off = isinstance(near_tokens_raw, str) and near_tokens_raw.strip().lower() == "off"
        if self.nt_near_pages is None or self.nt_near_len is None:
            raise ValueError("nfa_near_pages and nfa_near_len must be given")
        if self.nt_near_tokens is None and not near_tokens_off:
            raise ValueError("nfa_near_tokens must be a non-negative integer or 'off'")
        if self.nt_near_pages < 0 or self.nt_near_len < 0:
            raise ValueError("nfa_near_pages / nfa_near_len must be non-negative")
        if self.nt_near_pages > args.tia_level1_topk:
            raise ValueError("nfa_near_pages must not exceed tia_level1_topk")
        if self.nt_near_pages * block_size > self.nt_near_len:
            raise ValueError("nfa_near_pages * block_size must be <= nfa_near_len")
        k2 = int(args.tia_level2_topk)
        if k2 < self.sink_tokens + self.sliding_window_size:
            raise ValueError("tia_level2_topk must not be smaller than sink + swa")
        if not near_tokens_off:
            if self.nt_near_tokens < 0:
                raise ValueError("nfa_near_tokens must be non-negative")
            if self.nt_near_tokens > self.nt_near_pages * block_size:
                raise ValueError("nfa_near_tokens must be <= nfa_near_pages * block_size")

    # -- what the CUDA path implements -------------------------------------
    def require_supported(self):
        if self.far_method not in ("minmax", "avg", "avg_top2") or self.near_method not in ("avg", "minmax"):
            raise FallbackRequired("CUDA path implements far in {minmax, avg, avg_top2}, near in {avg, minmax}")
        if not self.enable_subspace or self.l2_subspace != "same":
            raise FallbackRequired("CUDA path scores L1 and L2 on the same proper subspace")
        self.subspace_ranges()

    @property
    def _sink_pool_lo_blk(self):
        return max(0, self.sink_tokens // int(self.args.tia_block_size))

    def subspace_ranges(self):
        """(lo0, lo1, d'): the subspace is [lo0, lo0 + d'/2) U [lo1, lo1 + d'/2)."""
        if self.subspace == "tail":
            if self.head_dim == 256:       # [NoPE192 | RoPE64]: 16 lowest-frequency dims of each RoPE half
                return 208, 240, 32
            if self.head_dim == 576:       # shared latent [compressed 512 | RoPE64]: the same 16 + 16 rotary dims
                return 528, 560, 32
            half = self.head_dim // 2
            delta = half // self.cmp_ratio
            return half - delta, self.head_dim - delta, 2 * delta
        if self.subspace == "rope":
            return 0, 32, 64
        if self.subspace == "nope":
            return (0, 32, 64) if self.head_dim == 256 else (64, 96, 64)
        if self.subspace == "mla_rope":
            return 128, 160, 64
        if self.subspace == "highfreq":
            delta = 64 // self.cmp_ratio
            return 0, 64, 2 * delta
        raise FallbackRequired(f"subspace {self.subspace!r} is not a pair of contiguous ranges")

    def _subspace_indices(self, device):
        lo0, lo1, d = self.subspace_ranges()
        return torch.cat((torch.arange(lo0, lo0 + d // 2, device=device),
                          torch.arange(lo1, lo1 + d // 2, device=device)))

    _tail_indices = _subspace_indices
