"""Seeded synthetic decode-step inputs with the shapes and value distributions
of the benchmark configurations (no dataset content).

Keys and values are N(0,1); RoPE (rotate-half layout, pairs (i, i + D/2)) is
applied by position to the keys and to the query; four fixed channels per KV
head are scaled by 8 as outliers; a few "needle" tokens in the far region get
keys aligned with the group-mean query so that recall of the selector can be
checked.  Generation is on the CPU generator when ``device`` is a CPU device
(bit-reproducible inputs for parity tests) and on the device generator
otherwise (full-size benchmark inputs).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class DecodeCase:
    q: torch.Tensor            # [Hq, D] post-RoPE query of the token being decoded
    k: torch.Tensor            # [L, Hkv, D] logical keys, current token included
    v: torch.Tensor            # [L, Hkv, Dv]
    length: int
    outlier_channels: torch.Tensor   # [Hkv, 4]
    needles: torch.Tensor            # [n_needles] token positions
    scale: float


def rope_tables(positions, head_dim, theta, device, llama3_scaling=False):
    half = head_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(half, device=device, dtype=torch.float32) / half))
    if llama3_scaling:
        # Llama-3.1 frequency rescaling: factor 8, low/high frequency factors
        # 1 and 4, original context 8192.
        factor, low, high, orig = 8.0, 1.0, 4.0, 8192.0
        wavelen = 2 * torch.pi / inv_freq
        smooth = ((orig / wavelen) - low) / (high - low)
        scaled = torch.where(wavelen > orig / low, inv_freq / factor, inv_freq)
        mid = (1 - smooth) * inv_freq / factor + smooth * inv_freq
        is_mid = (wavelen <= orig / low) & (wavelen >= orig / high)
        inv_freq = torch.where(is_mid, mid, scaled)
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x, cos, sin):
    """x [L, H, D]; cos/sin [L, D/2]; rotate-half layout."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


def make_decode_case(length, *, num_q_heads=32, num_kv_heads=8, head_dim=128,
                     seed=0, theta=1e6, n_needles=8, dtype=torch.float32,
                     device="cpu", swa=128, near_len=4096, sink=4,
                     llama3_scaling=False, chunk=16384):
    """One request of ``length`` tokens (the current token is the last one)."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    g = num_q_heads // num_kv_heads

    def randn(*shape):
        return torch.randn(*shape, generator=gen, device=device, dtype=torch.float32)

    q = randn(num_q_heads, head_dim)
    outliers = torch.stack([
        torch.randperm(head_dim, generator=gen, device=device)[:4]
        for _ in range(num_kv_heads)])
    far_hi = max(sink + 1, length - swa - near_len)
    needles = torch.randint(sink, far_hi, (n_needles,), generator=gen, device=device) \
        if far_hi > sink + 1 else torch.zeros(0, dtype=torch.long, device=device)

    cos_q, sin_q = rope_tables(torch.tensor([length - 1], device=device), head_dim, theta,
                               device, llama3_scaling)
    q = apply_rope(q[None], cos_q, sin_q)[0]
    q_bar = q.view(num_kv_heads, g, head_dim).mean(dim=1)
    q_bar = q_bar / q_bar.norm(dim=-1, keepdim=True)

    k = torch.empty(length, num_kv_heads, head_dim, dtype=dtype, device=device)
    v = torch.empty(length, num_kv_heads, head_dim, dtype=dtype, device=device)
    scale_vec = torch.ones(num_kv_heads, head_dim, device=device)
    scale_vec.scatter_(1, outliers, 8.0)
    for lo in range(0, length, chunk):
        hi = min(length, lo + chunk)
        kc = randn(hi - lo, num_kv_heads, head_dim) * scale_vec[None]
        cos, sin = rope_tables(torch.arange(lo, hi, device=device), head_dim, theta,
                               device, llama3_scaling)
        kc = apply_rope(kc, cos, sin)
        inside = needles[(needles >= lo) & (needles < hi)]
        for pos in inside.tolist():
            noise = randn(num_kv_heads, head_dim)
            # needle keys live in the post-RoPE space the query is compared in;
            # magnitude 24 makes them stand out against N(0,1) keys (|k| ~ 11).
            kc[pos - lo] = 24.0 * (0.9 * q_bar + 0.1 * noise / noise.norm(dim=-1, keepdim=True))
        k[lo:hi] = kc.to(dtype)
        v[lo:hi] = randn(hi - lo, num_kv_heads, head_dim).to(dtype)
    return DecodeCase(q.to(dtype), k, v, length, outliers, needles,
                      float(head_dim) ** -0.5)
