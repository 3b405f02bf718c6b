"""TIA indexer: the reference's PyTorch method surface
(sparse_attn/indexer/tia_indexer.py:11-142, base class sparse_attn/indexer/base.py:36-95)
with its numeric primitives — the 4-bit per-token quantiser, the per-block
min / max index and the bound / fine scores — running as CUDA kernels through
the C ABI.  ``compute_mask`` keeps the reference's sequence of tensor ops
(GQA mean, top-k, masked softmax, top-k) on the device; it is the legacy
single-pool selection and not the decode hot path (that is NFAIndexer +
select_topk_for_layer_batched).  CUDA tensors only, bf16 or fp32.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ... import _capi

_DTYPES = {torch.bfloat16: _capi.LODA_DTYPE_BF16, torch.float32: _capi.LODA_DTYPE_FP32}


def _dtype_code(t):
    if not t.is_cuda:
        raise RuntimeError("TIAIndexer kernels need CUDA tensors (no CPU path in this package)")
    if t.dtype not in _DTYPES:
        raise _capi.FallbackRequired("TIA kernels support bf16 and fp32 tensors")
    return _DTYPES[t.dtype]


class TIAIndexer:
    def __init__(self, args) -> None:
        self.args = args
        self.group_size = None
        self.sliding_window_size = getattr(args, "nfa_swa_size", 128)
        self.cmp_ratio = args.tia_level2_cmp_ratio
        self.enable_async = bool(getattr(args, "tia_enable_async_topk", False))
        self.prev_mask = None

    def min_max_per_token_quant(self, x: torch.Tensor, num_bits: int = 4) -> torch.Tensor:
        if num_bits != 4:
            raise _capi.FallbackRequired("only 4-bit quantisation is implemented")
        if x.shape[-1] > 128:
            raise _capi.FallbackRequired("rows longer than 128 values are not supported")
        xc = x.contiguous()
        y = torch.empty_like(xc)
        dim = xc.shape[-1]
        _capi.check(_capi.lib().loda_tia_quant4(
            _capi.ptr(xc), _capi.ptr(y), xc.numel() // dim, dim, dim, dim, _dtype_code(xc), _capi.current_stream()))
        return y

    def prepare_index(self, k: torch.Tensor, cu_seqlens_k: torch.Tensor):
        assert k.shape[0] == 1
        if cu_seqlens_k.numel() != 2:
            raise _capi.FallbackRequired("one sequence per call")
        bs = int(self.args.tia_block_size)
        _, s, h, d = k.shape
        assert d == 128
        kc = k[0].contiguous()
        t = (s + bs - 1) // bs
        k_min = torch.empty((t, h, d), dtype=k.dtype, device=k.device)
        k_max = torch.empty_like(k_min)
        code = _dtype_code(kc)
        lib, stream = _capi.lib(), _capi.current_stream()
        _capi.check(lib.loda_tia_block_minmax(_capi.ptr(kc), _capi.ptr(k_min), _capi.ptr(k_max), s, h, d, bs, code, stream))
        delta = 64 // self.cmp_ratio
        k_qat = torch.zeros_like(kc)
        # the two halves of the tail subspace are quantised together as one row of 2 * delta values
        idx = torch.tensor(list(range(64 - delta, 64)) + list(range(128 - delta, 128)), device=k.device)
        tail = kc[..., idx].contiguous()
        k_qat[..., idx] = self.min_max_per_token_quant(tail)
        pad_total = t * bs
        return {
            "k_min": k_min.unsqueeze(0), "k_max": k_max.unsqueeze(0), "k_qat": k_qat.unsqueeze(0),
            "cu_seqlens_k_coarse": torch.tensor([0, pad_total // bs], device=k.device, dtype=cu_seqlens_k.dtype),
            "cu_seqlens_k_fine": cu_seqlens_k,
        }

    def compute_score(self, q: torch.Tensor, q_ids: torch.Tensor, index_dict, softmax_scale: float):
        assert q.shape[0] == 1 and q.shape[1] == 1
        k_min, k_max, k_qat = (index_dict[n][0].contiguous() for n in ("k_min", "k_max", "k_qat"))
        qc = q[0, 0].contiguous()
        hq, d = qc.shape
        t, hkv = k_min.shape[0], k_min.shape[1]
        s = k_qat.shape[0]
        self.group_size = hq // hkv
        coarse = torch.empty((hq, t), dtype=q.dtype, device=q.device)
        fine = torch.empty((hq, s), dtype=q.dtype, device=q.device)
        _capi.check(_capi.lib().loda_tia_scores(
            _capi.ptr(qc), _capi.ptr(k_min), _capi.ptr(k_max), _capi.ptr(k_qat), _capi.ptr(coarse), _capi.ptr(fine),
            hq, hkv, d, t, s, float(softmax_scale), _dtype_code(qc), _capi.current_stream()))
        return {"score_coarse": coarse[None, None], "score_fine": fine[None, None]}

    def compute_mask(self, q_ids: torch.Tensor, score_dict):
        g, bs = self.group_size, int(self.args.tia_block_size)
        coarse, fine = score_dict["score_coarse"], score_dict["score_fine"]
        b, qt, hq, kt = coarse.shape
        coarse = coarse.view(b, qt, hq // g, g, kt).mean(dim=-2)
        coarse[..., -1] = float("inf")
        idx = torch.topk(coarse, dim=-1, k=min(kt, int(self.args.tia_level1_topk))).indices
        blk = torch.zeros_like(coarse, dtype=torch.bool).scatter_(-1, idx, True)
        tok = blk[:, :, :, None, :, None].expand(b, qt, hq // g, g, kt, bs).reshape(b, qt, hq, kt * bs)
        tok = tok[..., :fine.shape[-1]]
        fine = torch.where(tok, fine, float("-inf"))
        p = F.softmax(fine, dim=-1).nan_to_num(nan=0)
        p = p.view(b, qt, hq // g, g, -1).mean(dim=-2)
        p[..., -self.sliding_window_size:] = 1.0
        idx = torch.topk(p, k=min(p.shape[-1], int(self.args.tia_level2_topk)), dim=-1).indices
        return torch.zeros_like(p, dtype=torch.bool).scatter_(-1, idx, True)

    def get_block_size(self):
        return 1

    def prepare_mask(self, q, q_ids, k, cu_seqlens_k, softmax_scale=None, valid_length=None):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** -0.5
        index_dict = self.prepare_index(k, cu_seqlens_k)
        score_dict = self.compute_score(q, q_ids, index_dict, softmax_scale)
        return self.compute_mask(q_ids, score_dict), self.get_block_size()

    def clear(self):
        self.prev_mask = None
