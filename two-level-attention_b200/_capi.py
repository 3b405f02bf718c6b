"""ctypes binding of the C-ABI CUDA library (include/loda_b200.h).

There is no fallback: if ``libloda_b200.so`` is missing the import of any
operator of this package raises.  Build it with ``python -m`` style call
``build.build()`` (see build.py) — it needs only nvcc.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("LODA_B200_LIBRARY") or os.path.join(HERE, "libloda_b200.so")

LODA_DTYPE_BF16 = 0
LODA_DTYPE_FP32 = 1
LODA_OK = 0
LODA_ERR_ARGUMENT = -1
LODA_ERR_UNSUPPORTED = -2
LODA_ERR_LAUNCH = -3
STATUS_BAD_SLOT, STATUS_BAD_PAGE, STATUS_TRUNCATED, STATUS_BAD_REQ, STATUS_TIMEOUT = 1, 2, 4, 8, 16
SEL_CHAINED = 1
FAR_MINMAX, FAR_AVG, FAR_AVG_TOP2 = 0, 1, 2


class FallbackRequired(Exception):
    """The geometry is outside what the CUDA path supports (same exception the
    reference selector raises, nfa_layer_batch_selector.py:21-22)."""


class Geometry(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "dtype", "num_q_heads", "num_kv_heads", "head_dim", "head_dim_v", "sub_dims",
        "sub_lo0", "sub_lo1", "page", "num_pages", "max_blocks", "max_requests",
        "max_query_tokens", "max_visible", "k_far", "k_near", "level2_topk", "sink", "swa",
        "near_len", "pool_near_len", "shard_rank", "shard_count", "near_tokens_p1", "far_method",
        "near_minmax", "reserved")]


class Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "pool_k", "pool_v", "page_mm", "page_sum", "tail_code", "tail_sz", "block_table", "skip_far", "skip_near")]


class Batch(C.Structure):
    _fields_ = [("batch", C.c_int32), ("lengths", C.c_void_p), ("valid_req_ids", C.c_void_p),
                ("active_req_ids", C.c_void_p)]


class Selection(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "i_far", "n_far", "i_near", "n_near", "gather", "visible_lens", "middle", "middle_counts")] + [
        ("middle_only", C.c_int32), ("flags", C.c_int32)]


EXPORTS = ("loda_version", "loda_last_error", "loda_workspace_bytes", "loda_append_decode",
           "loda_write_prefill", "loda_build_index", "loda_select_l1", "loda_select_l2",
           "loda_gather_attend", "loda_decode_step", "loda_gather_attend_static",
           "loda_select_step", "loda_tia_quant4", "loda_tia_block_minmax", "loda_tia_scores", "loda_gather_attend_lse",
           "loda_tls_store_kv", "loda_tls_store_k_index", "loda_tls_level1", "loda_tls_level2",
           "loda_shard_workspace_regions", "loda_shard_l1_scores", "loda_shard_l1_select", "loda_shard_l2_scores",
           "loda_shard_l2_select", "loda_protected_gather", "loda_last_decode_launches", "loda_last_decode_cluster", "loda_lse_merge")

_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run __graft_entry__.build() or two-level-attention_b200/build.py); "
            "this package has no CPU or PyTorch fallback")
    L = C.CDLL(LIB_PATH)
    P, I, F, V = C.c_void_p, C.c_int32, C.c_float, C.c_void_p
    G, LY, B, S = C.POINTER(Geometry), C.POINTER(Layer), C.POINTER(Batch), C.POINTER(Selection)
    L.loda_version.restype = C.c_char_p
    L.loda_last_error.restype = C.c_char_p
    L.loda_workspace_bytes.restype = C.c_size_t
    L.loda_workspace_bytes.argtypes = [G]
    L.loda_append_decode.argtypes = [G, LY, B, P, P, P, P, V]
    L.loda_write_prefill.argtypes = [G, LY, P, P, P, I, V]
    L.loda_build_index.argtypes = [G, LY, I, I, I, I, V]
    L.loda_select_l1.argtypes = [G, LY, B, P, F, S, P, V]
    L.loda_select_l2.argtypes = [G, LY, B, P, F, S, P, P, V]
    L.loda_gather_attend.argtypes = [G, LY, P, P, P, P, I, I, F, P, P, V]
    L.loda_gather_attend_lse.argtypes = [G, LY, P, P, P, P, I, I, F, P, P, P, V]
    L.loda_gather_attend_static.argtypes = [G, LY, P, P, P, P, I, I, F, P, V]
    L.loda_select_step.argtypes = [G, LY, B, P, P, P, P, F, S, P, P, V]
    I64 = C.c_int64
    L.loda_tia_quant4.argtypes = [P, P, I64, I, I64, I64, I, V]
    L.loda_tia_block_minmax.argtypes = [P, P, P, I, I, I, I, I, V]
    L.loda_tia_scores.argtypes = [P, P, P, P, P, P, I, I, I, I, I, F, I, V]
    L.loda_decode_step.argtypes = [G, LY, B, P, P, P, P, F, S, P, P, P, P, V]
    L.loda_tls_store_kv.argtypes = [P, P, P, P, P, I, I, I, I, I, I, I, V]
    L.loda_tls_store_k_index.argtypes = [P, P, P, P, P, I, I, I, I, I, I, I, I, I, V]
    L.loda_tls_level1.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, V]
    L.loda_tls_level2.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, V]
    L.loda_protected_gather.argtypes = [G, LY, B, P, P, P, V]
    L.loda_shard_workspace_regions.argtypes = [G, P]
    L.loda_shard_l1_scores.argtypes = [G, LY, B, P, F, S, P, V]
    L.loda_shard_l1_select.argtypes = [G, LY, B, P, F, S, P, P, V]
    L.loda_shard_l2_scores.argtypes = [G, LY, B, P, F, S, P, P, V]
    L.loda_shard_l2_select.argtypes = [G, LY, B, P, F, S, P, P, P, V]
    L.loda_lse_merge.argtypes = [P, C.c_int64, C.c_int64, I, I, I, P, V]
    for name in EXPORTS[3:]:
        getattr(L, name).restype = C.c_int
    _lib = L
    return L


def check(rc):
    if rc == LODA_OK:
        return
    msg = lib().loda_last_error().decode()
    if rc == LODA_ERR_ARGUMENT:
        raise ValueError(msg)
    if rc == LODA_ERR_UNSUPPORTED:
        raise FallbackRequired(msg)
    raise RuntimeError(msg)


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else C.c_void_p(t.data_ptr())


def current_stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)
