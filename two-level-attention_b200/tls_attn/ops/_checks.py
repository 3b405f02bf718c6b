"""Argument checks shared by the prototype-chain operators."""
from __future__ import annotations

import torch

from ... import _capi


def need_bf16_cuda(**tensors):
    for name, t in tensors.items():
        if not t.is_cuda:
            raise RuntimeError(f"{name}: tls_attn operators need CUDA tensors (no CPU path in this package)")
        if t.dtype != torch.bfloat16:
            raise _capi.FallbackRequired(f"{name}: tls_attn operators of this package take bf16 tensors")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")


def need_i32(name, t):
    if t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous int32 CUDA tensor")


def need_f32(name, t, shape):
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous() or tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must be a contiguous float32 CUDA tensor of shape {tuple(shape)}")
