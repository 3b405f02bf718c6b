"""CPU oracle for the LoDA-SA (NFA) two-level select + gather-attend decode step.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is compared
against; nothing the library ships may import it.  It restates, in numpy, the
algorithm of the reference's production selector and gather attention:

  * subspace indices ............ sparse_attn/indexer/nfa_indexer.py:112-121
  * page statistics ............. sparse_attn/indexer/nfa_layer_batch_selector.py:87-131
  * region geometry and pools ... nfa_layer_batch_selector.py:209-262
  * query preparation ........... nfa_layer_batch_selector.py:943-1002
  * L1 bound / mean scores ...... nfa_layer_batch_selector.py:290-354
  * L1 packed-key top-k ......... nfa_layer_batch_selector.py:1473-1532, 1765-1793
  * candidates, bounds, quota ... nfa_layer_batch_selector.py:1116-1251, 1971-1986
  * L2 grouped-q logits ......... nfa_layer_batch_selector.py:422-516
  * L2 top-k, quota, hole fill .. nfa_layer_batch_selector.py:518-605
  * final union + slot mapping .. nfa_layer_batch_selector.py:1336-1437
  * 4-bit per-token quantiser ... sparse_attn/indexer/tia_indexer.py:22-31
  * paged write (CPU branch) .... sparse_attn/ops/paged_region_kernels.py:653-662, 716-724
  * gather attention (CPU) ...... sparse_attn/ops/paged_region_kernels.py:1008-1041

Parity pinning.  The reference ships no golden vectors for this path; its own
tests generate their comparisons at test time on a GPU.  The primitives that
the reference implements in plain PyTorch are pinned here against outputs of
the reference itself, generated on CPU by tests/golden/make_golden.py and
committed as fixtures: the 4-bit quantiser (bit exact, bf16 and fp32), the
page min/max index (bit exact), the min/max bound score (fp32 tolerance: the
reference leaves the reduction order to the BLAS), L1 page sets against the
archived PyTorch pipeline, the paged write (bit exact) and the gather
attention (fp32 tolerance).  The production selector itself only exists as
GPU Triton code, so the packed-key ordering, quota, hole-fill and union rules
are restated from its source and checked only against its documented
formulas; for those stages, for the packed 4-bit key store, and for every
multi-GPU mode, parity is UNPINNED by the reference.

Canonical arithmetic.  The reference leaves the fp32 summation order inside a
dot product to the compiler.  Selection compares rounded scores, so this
oracle fixes one order that a GPU kernel reproduces exactly; every product and
sum below is a separate IEEE fp32 operation (no fused multiply-add):

  * a length-d' dot is split into chunks of 8 consecutive subspace dims; each
    chunk is summed left to right starting from 0.0f; chunk sums are combined
    by a balanced pairwise tree of adjacent chunks;
  * the min/max bound adds (tree over the min chunks) + (tree over the max
    chunks);
  * the L2 logit is one left-to-right chain over all d' dims;
  * a page sum is accumulated in ascending token order starting from 0.0f;
  * sums over the GQA group run over heads in ascending order from 0.0f.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

F32 = np.float32
NEG_INF = F32(-np.inf)


# --------------------------------------------------------------------------
# bf16 helpers (values are carried as float32 holding bf16-representable data)
# --------------------------------------------------------------------------
def bf16_rn(x):
    """Round float32 to the nearest bf16 (ties to even); result as float32."""
    x = np.ascontiguousarray(x, dtype=F32)
    u = x.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32)
    r = np.where(np.isnan(x), np.uint32(0x7FC00000), r).astype(np.uint32)
    return r.view(F32).reshape(x.shape)


def bf16_bits(x):
    """uint16 bit pattern of bf16-representable float32 values."""
    x = np.ascontiguousarray(x, dtype=F32)
    return (x.view(np.uint32) >> 16).astype(np.uint16).reshape(x.shape)


def bits_to_f32(bits):
    """float32 values of bf16 bit patterns."""
    b = np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16
    return b.view(F32).reshape(np.shape(bits))


def act(x, mode):
    """Round to the activation dtype: bf16 in 'bf16' mode, identity in 'fp32'."""
    return bf16_rn(x) if mode == "bf16" else np.asarray(x, dtype=F32)


def ordered_key(score, mode):
    """Monotone unsigned key of a score; NaN (canonicalised) sorts highest.

    bf16 mode: 16-bit key of the bf16 pattern (nfa_layer_batch_selector.py:
    1482-1485); fp32 mode: the same construction on the 32-bit pattern.
    """
    score = np.ascontiguousarray(score, dtype=F32)
    if mode == "bf16":
        bits = bf16_bits(score).astype(np.int64)
        bits = np.where(np.isnan(score), 0x7FC0, bits)
        return np.where(bits & 0x8000, (~bits) & 0xFFFF, bits | 0x8000)
    bits = score.view(np.uint32).astype(np.int64).reshape(score.shape)
    bits = np.where(np.isnan(score), 0x7FC00000, bits)
    return np.where(bits & 0x80000000, (~bits) & 0xFFFFFFFF, bits | 0x80000000)


# --------------------------------------------------------------------------
# configuration
# --------------------------------------------------------------------------
@dataclass
class SelectorConfig:
    """Selector constants; defaults are the production values
    (sparse_attn/ops/paged_region_kernels_nfa.py:10-20) at 16-token pages."""
    head_dim: int = 128
    num_q_heads: int = 32
    num_kv_heads: int = 8
    block_size: int = 16          # tia_block_size == cache page
    max_blocks: int = 2112        # KT: block-table capacity per request
    level1_topk: int = 128        # K1
    near_pages: int = 32          # nb_near
    near_len: int = 4096          # geometry.near and POOL_NEAR_LEN
    level2_topk: int = 1024       # K2
    cmp_ratio: int = 4
    sink: int = 4
    swa: int = 128
    max_visible: int = 1024
    mode: str = "bf16"            # 'bf16' | 'fp32'
    l2_quant: bool = True         # 4-bit tail keys (build) vs raw keys (live reference)
    l2_metric: str = "grouped_logit"   # | 'softmax_prob_mean'
    q_round: bool = True          # bf16-round the scaled query (live selector: always)
    near_tokens: int = None       # numeric near-token quota (nfa_near_tokens); None = 'off'
    far_method: str = "minmax"    # | 'avg' | 'avg_top2'  (nfa_far_method)
    near_method: str = "avg"      # | 'minmax'            (nfa_near_method)
    geometry_near: int = None     # RegionGeometry.near where it differs from near_len (L1 region bounds)
    dims: np.ndarray = field(default=None, repr=False)

    def __post_init__(self):
        if self.dims is None:
            self.dims = tail_dims(self.head_dim, self.cmp_ratio)
        self.dims = np.asarray(self.dims, dtype=np.int64)
        if self.swa % self.block_size:
            raise ValueError("swa must be a multiple of the block size")
        if self.near_pages > self.level1_topk:
            raise ValueError("near_pages must not exceed level1_topk")
        if self.near_pages * self.block_size > self.near_len:
            raise ValueError("near_pages * block_size must be <= near_len")
        if self.level2_topk < self.sink + self.swa:
            raise ValueError("level2_topk must be >= sink + swa")
        if self.geometry_near is None:
            self.geometry_near = self.near_len

    @property
    def group(self):
        return self.num_q_heads // self.num_kv_heads

    @property
    def k_far(self):
        return min(max(0, self.level1_topk - self.near_pages), self.max_blocks)

    @property
    def k_near(self):
        return min(max(0, self.near_pages), self.max_blocks)

    @property
    def sink_pool_lo(self):
        return max(0, self.sink // self.block_size)

    @property
    def pool_near_len(self):
        return max(self.block_size, self.near_len)

    @property
    def s_cap(self):
        return self.max_blocks * self.block_size


def tail_dims(head_dim=128, cmp_ratio=4):
    """Lowest-frequency RoPE dims of both halves (nfa_indexer.py:117-121)."""
    half = head_dim // 2
    delta = half // cmp_ratio
    return np.concatenate((np.arange(half - delta, half),
                           np.arange(head_dim - delta, head_dim))).astype(np.int64)


# --------------------------------------------------------------------------
# 4-bit per-token quantiser (tia_indexer.py:22-31)
# --------------------------------------------------------------------------
def quant4(x, mode):
    """Per-token asymmetric 16-level quantisation over the last axis.

    Returns (code uint8, scale, zero, dequantised) where every torch op of the
    reference is one rounding to the tensor dtype.
    """
    x = act(x, mode)
    r = (lambda v: bf16_rn(v)) if mode == "bf16" else (lambda v: np.asarray(v, F32))
    mx = x.max(axis=-1, keepdims=True)
    mn = x.min(axis=-1, keepdims=True)
    floor = r(np.asarray(1e-9, dtype=F32))
    rng = r(mx - mn)
    rng = np.where(rng < floor, floor, rng).astype(F32)
    scale = r(rng / F32(15.0))
    zero = (-mn).astype(F32)
    with np.errstate(all="ignore"):
        t = r(r(x + zero) / scale)
        code_f = np.clip(np.rint(t), F32(0), F32(15)).astype(F32)
    deq = r(r(code_f * scale) - zero)
    code = np.nan_to_num(code_f, nan=0.0).astype(np.uint8)
    return code, scale[..., 0], zero[..., 0], deq


def dequant4(code, scale, zero, mode):
    r = (lambda v: bf16_rn(v)) if mode == "bf16" else (lambda v: np.asarray(v, F32))
    return r(r(code.astype(F32) * scale[..., None]) - zero[..., None])


# --------------------------------------------------------------------------
# page statistics (nfa_layer_batch_selector.py:87-131)
# --------------------------------------------------------------------------
def page_stats(k_sub, length, block_size, mode):
    """min / max / sum over the visible tokens of every logical block.

    k_sub: [S, Hkv, d'] subspace keys (S >= length).  Returns arrays
    [kt_eff, Hkv, d'] in the pool dtype.  Invalid lanes are excluded from
    min/max and contribute 0 to the sum; the sum runs in ascending token order.
    """
    kt_eff = (length + block_size - 1) // block_size
    hkv, dsub = k_sub.shape[1], k_sub.shape[2]
    pad = kt_eff * block_size
    buf = np.zeros((pad, hkv, dsub), dtype=F32)
    buf[:length] = act(k_sub[:length], mode)
    blk = buf.reshape(kt_eff, block_size, hkv, dsub)
    tok = np.arange(pad).reshape(kt_eff, block_size)
    vis = (tok < length)[:, :, None, None]
    vmin = np.where(vis, blk, F32(np.inf)).min(axis=1)
    vmax = np.where(vis, blk, F32(-np.inf)).max(axis=1)
    vsum = np.zeros((kt_eff, hkv, dsub), dtype=F32)
    for i in range(block_size):
        vsum = (vsum + np.where(vis[:, i], blk[:, i], F32(0))).astype(F32)
    return act(vmin, mode), act(vmax, mode), act(vsum, mode)


# --------------------------------------------------------------------------
# region geometry (nfa_layer_batch_selector.py:209-262, 1136-1163)
# --------------------------------------------------------------------------
@dataclass
class Regions:
    length: int
    kt_eff: int
    near_blks: int
    sink_hi: int
    swa_hi: int
    orig_far_hi: int
    swa_lo_blk: int
    swa_lo_tok: int
    swa_byp_blk: int
    swa_byp: bool
    sink_byp: bool
    lower: int
    upper: int
    quota: int
    skip_far: bool = False
    skip_near: bool = False
    far_hi_tok: int = 0       # token bound between the far and the near region of level 2
    lower0: int = 0           # [lower0, upper0): the middle range before any region is skipped
    upper0: int = 0
    base_quota: int = 0


def regions(length, cfg: SelectorConfig, skip_far=False, skip_near=False) -> Regions:
    """Region geometry of one request.  skip_far / skip_near: the frozen per-layer decisions of
    the request (paged_region_cache.py:540-559); a skipped region is neither scored
    (nfa_layer_batch_selector.py:223-226, 241-267) nor part of the middle range (:1151-1163)."""
    bs, w, spl = cfg.block_size, cfg.swa, cfg.sink_pool_lo
    kt_eff = (length + bs - 1) // bs
    near_blks = max(_cdiv(length - w - cfg.pool_near_len, bs), spl)
    sink_hi = min(cfg.sink, length)
    swa_hi = max(sink_hi, length - w)
    far_blk = _cdiv(length - w - cfg.geometry_near, bs)
    orig_far_hi = min(swa_hi, max(sink_hi, far_blk * bs))
    swa_lo_blk = max(near_blks, kt_eff - max(1, w // bs))
    swa_lo_tok = max(length - w, 0)
    swa_byp_blk = swa_lo_tok // bs
    swa_byp = (swa_lo_tok % bs != 0) and (swa_byp_blk >= spl)
    sink_byp = cfg.sink % bs != 0
    if sink_byp:
        swa_byp = swa_byp and swa_byp_blk != spl
    lower0 = spl * bs
    upper0 = max(lower0, swa_lo_tok)
    # level-2 region bound (nfa_layer_batch_selector.py:1155-1163)
    far_hi_tok = min(swa_hi, max(sink_hi, (max(length - w - cfg.geometry_near, 0) // bs) * bs))
    lower = far_hi_tok if skip_far else lower0
    upper = far_hi_tok if skip_near else upper0
    upper = max(lower, upper)
    base_quota = max(min(length, cfg.level2_topk) - cfg.sink - (length - swa_lo_tok), 0)
    quota = min(base_quota, upper - lower)
    return Regions(length, kt_eff, near_blks, sink_hi, swa_hi, orig_far_hi,
                   swa_lo_blk, swa_lo_tok, swa_byp_blk, swa_byp, sink_byp,
                   lower, upper, quota, bool(skip_far), bool(skip_near), far_hi_tok,
                   lower0, upper0, base_quota)


def _cdiv(a, b):
    """C-style truncating division (what the Triton kernels compute)."""
    q = abs(a) // b
    return q if a >= 0 else -q


def pools(rg: Regions, cfg: SelectorConfig):
    """Boolean far/near pool membership per block index [kt_eff]."""
    bs, spl = cfg.block_size, cfg.sink_pool_lo
    t = np.arange(rg.kt_eff)
    lo, hi = t * bs, t * bs + bs
    far_on, near_on = not rg.skip_far, not rg.skip_near
    has_sink = lo < rg.sink_hi
    has_far = far_on & (hi > rg.sink_hi) & (lo < rg.orig_far_hi)
    has_near = near_on & (hi > rg.orig_far_hi) & (lo < rg.swa_hi)
    has_swa = (hi > rg.swa_hi) & (lo < rg.length)
    valid = (lo < rg.length) & (has_sink | has_far | has_near | has_swa)
    far = (t >= spl) & (t < rg.near_blks) & far_on
    near = (t >= rg.near_blks) & (t < rg.swa_lo_blk) & ~((t == rg.swa_byp_blk) & rg.swa_byp) & near_on
    if rg.sink_byp:
        far &= t != spl
        near &= t != spl
    return far & valid, near & valid


# --------------------------------------------------------------------------
# query preparation (nfa_layer_batch_selector.py:943-1002)
# --------------------------------------------------------------------------
def prepare_q_unrounded(q, cfg: SelectorConfig, scale):
    """fp32 scaled query on the subspace without the bf16 rounding: what the avg_top2 far score
    is computed from (nfa_layer_batch_selector.py:2936-2938, 2412-2427)."""
    qs = act(np.asarray(q, dtype=F32), cfg.mode)[:, cfg.dims]
    return (qs * F32(scale)).astype(F32)


def prepare_q(q, cfg: SelectorConfig, scale):
    """q [Hq, D] -> (q_hat [Hq, d'] bf16-rounded scaled query on the subspace,
    q_fine [Hkv, d'] fp32 sum of q_hat over each GQA group)."""
    q_hat = prepare_q_unrounded(q, cfg, scale)
    if cfg.q_round:
        q_hat = bf16_rn(q_hat)
    g = cfg.group
    q_fine = np.zeros((cfg.num_kv_heads, q_hat.shape[1]), dtype=F32)
    for j in range(g):
        q_fine = (q_fine + q_hat.reshape(cfg.num_kv_heads, g, -1)[:, j]).astype(F32)
    return q_hat, q_fine


# --------------------------------------------------------------------------
# canonical dot products
# --------------------------------------------------------------------------
def _chunk_tree_dot(k, q):
    """k [..., d'], q [d'] -> [...]: chunks of 8 summed left to right, then a
    balanced pairwise tree over adjacent chunks."""
    d = k.shape[-1]
    assert d % 8 == 0 and (d // 8) & (d // 8 - 1) == 0
    c = d // 8
    kk = k.reshape(k.shape[:-1] + (c, 8))
    qq = q.reshape(c, 8)
    acc = np.zeros(kk.shape[:-1], dtype=F32)
    for i in range(8):
        acc = (acc + (kk[..., i] * qq[:, i]).astype(F32)).astype(F32)
    while acc.shape[-1] > 1:
        acc = (acc[..., 0::2] + acc[..., 1::2]).astype(F32)
    return acc[..., 0]


def _chain_dot(k, q):
    """k [..., d'], q [d'] -> [...]: one left-to-right chain from 0.0f."""
    acc = np.zeros(k.shape[:-1], dtype=F32)
    for i in range(k.shape[-1]):
        acc = (acc + (k[..., i] * q[i]).astype(F32)).astype(F32)
    return acc


# --------------------------------------------------------------------------
# L1 scores (nfa_layer_batch_selector.py:290-354)
# --------------------------------------------------------------------------
def l1_scores(vmin, vmax, vsum, q_hat, rg: Regions, cfg: SelectorConfig, q_raw=None):
    """far / near page scores [Hkv, kt_eff]; -inf outside the pools.

    Each pool is scored by its method: 'minmax' = the min/max upper bound, 'avg' = the page
    mean, both averaged over the GQA group of per-head bf16 scores; far 'avg_top2' = the mean of
    the two best per-head page-mean scores of the group, computed from the unrounded scaled
    query q_raw (nfa_layer_batch_selector.py:2412-2427)."""
    g, hkv, mode = cfg.group, cfg.num_kv_heads, cfg.mode
    far_pool, near_pool = pools(rg, cfg)
    far = np.full((hkv, rg.kt_eff), NEG_INF, dtype=F32)
    near = np.full((hkv, rg.kt_eff), NEG_INF, dtype=F32)
    with np.errstate(all="ignore"):
        kavg = act((vsum / F32(cfg.block_size)).astype(F32), mode)
        for kv in range(hkv):
            mm_acc = np.zeros(rg.kt_eff, dtype=F32)
            av_acc = np.zeros(rg.kt_eff, dtype=F32)
            per_head = []
            for j in range(g):
                qh = q_hat[kv * g + j]
                q_lo, q_hi = np.minimum(qh, F32(0)), np.maximum(qh, F32(0))
                mm = (_chunk_tree_dot(vmin[:, kv], q_lo)
                      + _chunk_tree_dot(vmax[:, kv], q_hi)).astype(F32)
                mm_acc = (mm_acc + act(mm, mode)).astype(F32)
                av = _chunk_tree_dot(kavg[:, kv], qh)
                av_acc = (av_acc + act(av, mode)).astype(F32)
                if cfg.far_method == "avg_top2":
                    per_head.append(act(_chunk_tree_dot(kavg[:, kv], q_raw[kv * g + j]), mode))
            mm_score = act((mm_acc / F32(g)).astype(F32), mode)
            av_score = act((av_acc / F32(g)).astype(F32), mode)
            if cfg.far_method == "minmax":
                far_score = mm_score
            elif cfg.far_method == "avg":
                far_score = av_score
            else:
                top = np.sort(np.stack(per_head), axis=0)[::-1]
                far_score = act(((top[0] + top[1]) / F32(2)).astype(F32), mode)
            near_score = mm_score if cfg.near_method == "minmax" else av_score
            far[kv] = np.where(far_pool, far_score, NEG_INF)
            near[kv] = np.where(near_pool, near_score, NEG_INF)
    return far, near


# --------------------------------------------------------------------------
# L1 top-k (nfa_layer_batch_selector.py:1473-1532, 1765-1793)
# --------------------------------------------------------------------------
def topk_pages(scores, k, kt_cap, mode):
    """Best k page ids by (score descending in key order, lower id first).

    Positions without a score count as -inf and act as fillers.  Returns
    (ids [k], n_valid) where the first n_valid ids have a score != -inf.
    """
    full = np.full(kt_cap, NEG_INF, dtype=F32)
    n = min(len(scores), kt_cap)
    full[:n] = scores[:n]
    key = ordered_key(full, mode)
    order = np.lexsort((np.arange(kt_cap), -key))[:k]
    neg_inf_key = ordered_key(np.array([NEG_INF]), mode)[0]
    n_valid = int(np.sum(key[order] != neg_inf_key))
    return order.astype(np.int32), n_valid


def l1_select(far, near, cfg: SelectorConfig):
    """I_F [Hkv, K_F], I_N [Hkv, K_N] and the number of non-filler entries."""
    hkv = cfg.num_kv_heads
    i_f = np.zeros((hkv, cfg.k_far), np.int32)
    i_n = np.zeros((hkv, cfg.k_near), np.int32)
    n_f = np.zeros(hkv, np.int32)
    n_n = np.zeros(hkv, np.int32)
    for kv in range(hkv):
        i_f[kv], n_f[kv] = topk_pages(far[kv], cfg.k_far, cfg.max_blocks, cfg.mode)
        i_n[kv], n_n[kv] = topk_pages(near[kv], cfg.k_near, cfg.max_blocks, cfg.mode)
    return i_f, n_f, i_n, n_n


# --------------------------------------------------------------------------
# L2 (nfa_layer_batch_selector.py:422-605, 1194-1251)
# --------------------------------------------------------------------------
def candidate_tokens(pages_f, pages_n, rg: Regions, cfg: SelectorConfig):
    """Ascending token ids that compete for the middle quota."""
    bs = cfg.block_size
    pages = [int(p) for p in pages_f] + [int(p) for p in pages_n]
    if rg.sink_byp:
        pages.append(cfg.sink_pool_lo)
    if rg.swa_byp:
        pages.append(rg.swa_byp_blk)
    pages = sorted(set(p for p in pages if p < cfg.max_blocks))
    if not pages:
        return np.zeros(0, np.int64)
    tok = (np.asarray(pages, np.int64)[:, None] * bs + np.arange(bs)[None, :]).reshape(-1)
    keep = ((tok >= cfg.sink) & (tok < rg.swa_lo_tok) & (tok < rg.length)
            & (tok >= rg.lower) & (tok < rg.upper))
    return tok[keep]


def l2_logits(k_tail, q_fine_kv, mode):
    """Grouped-q logit per candidate: fp32 chain dot rounded to bf16
    (nfa_layer_batch_selector.py:505-516; logits are bf16 in every mode)."""
    with np.errstate(all="ignore"):
        return bf16_rn(_chain_dot(np.asarray(k_tail, F32), q_fine_kv))


def filtered_topk(tokens, logits, low, high, q, cfg: SelectorConfig):
    """Best q candidates of [low, high) by (logit descending, lower token first); missing
    entries are filled with the first ids of [low, high) not chosen; ids below the sink are
    dropped; ascending (nfa_layer_batch_selector.py:518-605)."""
    if q <= 0:
        return np.zeros(0, np.int32)
    good = ~np.isnan(logits) & (logits != NEG_INF) & (tokens >= low) & (tokens < high)
    tok, lg = tokens[good], logits[good]
    key = ordered_key(lg, "bf16")
    order = np.lexsort((tok, -key))
    take = min(q, cfg.level2_topk, len(order))
    chosen = np.sort(tok[order[:take]])
    if len(chosen) < q:
        need = q - len(chosen)
        span = np.arange(low, min(high, low + len(chosen) + need), dtype=np.int64)
        holes = np.setdiff1d(span, chosen, assume_unique=True)[:need]
        chosen = np.sort(np.concatenate((chosen, holes)))
    chosen = chosen[chosen >= cfg.sink]
    return chosen[:cfg.level2_topk].astype(np.int32)


def fixed_quota_regions(rg: Regions, cfg: SelectorConfig):
    """(far_low, far_high, far_quota, near_low, near_high, near_quota) of the numeric
    near-token quota (nfa_layer_batch_selector.py:872-920): the near region reserves
    near_tokens of the middle budget; what the far region cannot use goes to the near
    region, never the other way."""
    base = rg.base_quota
    far_quota = max(base - min(int(cfg.near_tokens), base), 0)
    far_low = rg.far_hi_tok if rg.skip_far else rg.lower0
    far_high = rg.far_hi_tok
    far_quota = min(far_quota, max(far_high - far_low, 0))
    near_quota = max(base - far_quota, 0)
    near_low = rg.far_hi_tok
    near_high = rg.far_hi_tok if rg.skip_near else rg.upper0
    near_quota = min(near_quota, max(near_high - near_low, 0))
    return far_low, far_high, far_quota, near_low, near_high, near_quota


def l2_select(tokens, logits, rg: Regions, cfg: SelectorConfig):
    """The middle tokens: one quota over [lower, upper) ('off'), or, with a numeric near-token
    quota, the far and the near region selected separately and concatenated
    (nfa_layer_batch_selector.py:2274-2332, 922-943)."""
    if cfg.near_tokens is None:
        return filtered_topk(tokens, logits, rg.lower, rg.upper, rg.quota, cfg)
    fl, fh, fq, nl, nh, nq = fixed_quota_regions(rg, cfg)
    far = filtered_topk(tokens, logits, fl, fh, fq, cfg)
    near = filtered_topk(tokens, logits, nl, nh, nq, cfg)
    return np.concatenate((far, near)).astype(np.int32)[:cfg.level2_topk]


def l2_select_softmax_prob(tokens, k_tail, q_hat_group, rg, cfg):
    """Alternative ranking of the PyTorch indexers (tia_indexer.py:116-135):
    per-head softmax over the candidates, GQA mean of probabilities."""
    q = rg.quota
    if q == 0 or len(tokens) == 0:
        return l2_select(tokens, np.full(len(tokens), NEG_INF, F32), rg, cfg)
    probs = np.zeros(len(tokens), dtype=np.float64)
    for qh in q_hat_group:
        s = act(_chain_dot(np.asarray(k_tail, F32), qh), cfg.mode).astype(np.float64)
        e = np.exp(s - s.max())
        probs += e / e.sum()
    probs /= len(q_hat_group)
    order = np.lexsort((tokens, -probs))
    chosen = np.sort(tokens[order[:min(q, len(order))]])
    if len(chosen) < q:
        need = q - len(chosen)
        span = np.arange(rg.lower, min(rg.upper, rg.lower + len(chosen) + need), dtype=np.int64)
        chosen = np.sort(np.concatenate((chosen, np.setdiff1d(span, chosen)[:need])))
    return chosen[chosen >= cfg.sink].astype(np.int32)


# --------------------------------------------------------------------------
# final union (nfa_layer_batch_selector.py:1336-1437)
# --------------------------------------------------------------------------
def protected_ids(length, cfg: SelectorConfig):
    sink_count = min(length, cfg.sink)
    total = min(length, cfg.sink + cfg.swa)
    ids = list(range(sink_count))
    ids += [length - cfg.swa + i for i in range(total - sink_count)]
    return np.array([i for i in ids if 0 <= i < cfg.s_cap], dtype=np.int64)


def final_union(middle, length, cfg: SelectorConfig):
    out = np.union1d(np.asarray(middle, np.int64), protected_ids(length, cfg))
    return out[:cfg.max_visible].astype(np.int32)


def to_slots(ids, block_table_row, page):
    ids = np.asarray(ids, np.int64)
    return (np.asarray(block_table_row, np.int64)[ids // page] * page + ids % page).astype(np.int32)


# --------------------------------------------------------------------------
# one request, end to end
# --------------------------------------------------------------------------
@dataclass
class RequestIndex:
    """What the append-time kernel maintains for one request: page statistics
    on the subspace and the packed 4-bit tail keys."""
    vmin: np.ndarray
    vmax: np.ndarray
    vsum: np.ndarray
    code: np.ndarray      # [S, Hkv, d'] uint8 in 0..15
    scale: np.ndarray     # [S, Hkv]
    zero: np.ndarray      # [S, Hkv]


def build_index(k, length, cfg: SelectorConfig) -> RequestIndex:
    """k [S, Hkv, D] logical keys of one request (S >= length)."""
    k_sub = act(np.asarray(k[:length], F32), cfg.mode)[:, :, cfg.dims]
    vmin, vmax, vsum = page_stats(k_sub, length, cfg.block_size, cfg.mode)
    code, scale, zero, _ = quant4(k_sub, cfg.mode)
    return RequestIndex(vmin, vmax, vsum, code, scale, zero)


@dataclass
class Selection:
    far_scores: np.ndarray
    near_scores: np.ndarray
    i_far: np.ndarray
    n_far: np.ndarray
    i_near: np.ndarray
    n_near: np.ndarray
    middle: list          # per kv head: ascending logical ids
    logical: list         # per kv head: ascending logical ids after the union
    regions: Regions


def select_request(q, k, length, cfg: SelectorConfig, scale, index: RequestIndex = None,
                   skip_far=False, skip_near=False) -> Selection:
    """Two-level selection for one request and its current query.

    q [Hq, D] post-RoPE query of the token being decoded; k [S, Hkv, D] logical
    keys with the current token already appended (length counts it).
    """
    if index is None:
        index = build_index(k, length, cfg)
    rg = regions(length, cfg, skip_far, skip_near)
    q_hat, q_fine = prepare_q(q, cfg, scale)
    q_raw = prepare_q_unrounded(q, cfg, scale) if cfg.far_method == "avg_top2" else None
    far, near = l1_scores(index.vmin, index.vmax, index.vsum, q_hat, rg, cfg, q_raw)
    i_f, n_f, i_n, n_n = l1_select(far, near, cfg)
    middle, logical = [], []
    g = cfg.group
    for kv in range(cfg.num_kv_heads):
        tok = candidate_tokens(i_f[kv, :n_f[kv]], i_n[kv, :n_n[kv]], rg, cfg)
        if cfg.l2_quant:
            k_tail = dequant4(index.code[tok, kv], index.scale[tok, kv], index.zero[tok, kv], cfg.mode)
        else:
            k_tail = act(np.asarray(k[tok, kv], F32), cfg.mode)[:, cfg.dims]
        if cfg.l2_metric == "grouped_logit":
            mid = l2_select(tok, l2_logits(k_tail, q_fine[kv], cfg.mode), rg, cfg)
        else:
            mid = l2_select_softmax_prob(tok, k_tail, q_hat[kv * g:(kv + 1) * g], rg, cfg)
        middle.append(mid)
        logical.append(final_union(mid, length, cfg))
    return Selection(far, near, i_f, n_f, i_n, n_n, middle, logical, rg)


# --------------------------------------------------------------------------
# paged pool helpers and the CPU branches of the paged ops
# --------------------------------------------------------------------------
def paged_write_prefill(pool_k, pool_v, k, v, block_table_row):
    """k [Hkv, N, D] -> pool [pages+1, Hkv, PAGE, D] through one block-table
    row (paged_region_kernels.py:653-662)."""
    page = pool_k.shape[2]
    n = k.shape[1]
    for lp in range((n + page - 1) // page):
        phys = int(block_table_row[lp])
        lo, hi = lp * page, min(lp * page + page, n)
        pool_k[phys, :, :hi - lo] = k[:, lo:hi]
        pool_v[phys, :, :hi - lo] = v[:, lo:hi]


def paged_write_decode(pool_k, pool_v, k, v, slots):
    """k [B, Hkv, D]; slot -1 goes to the PAD page (paged_region_kernels.py:716-724)."""
    page = pool_k.shape[2]
    pad_slot = (pool_k.shape[0] - 1) * page
    for b in range(k.shape[0]):
        slot = int(slots[b])
        if slot < 0:
            slot = pad_slot
        phys, off = divmod(slot, page)
        pool_k[phys, :, off] = k[b]
        pool_v[phys, :, off] = v[b]


def logical_keys(pool, block_table_row, length):
    """[length, Hkv, D] logical view of a request's rows in a pool."""
    page = pool.shape[2]
    nblk = (length + page - 1) // page
    rows = pool[np.asarray(block_table_row[:nblk], np.int64)]       # [nblk, Hkv, PAGE, D]
    return rows.transpose(0, 2, 1, 3).reshape(nblk * page, pool.shape[1], pool.shape[3])[:length]


def gather_attention(q, pool_k, pool_v, gather, vis_lens, query_to_req, scale, mode):
    """Exact softmax attention over the gathered slots
    (paged_region_kernels.py:1008-1041).  q [T, Hq, D]; pools
    [pages+1, Hkv, PAGE, D]; gather [B, Hkv, MAX_VIS] physical slots."""
    t_total, hq, _ = q.shape
    hkv, page = pool_k.shape[1], pool_k.shape[2]
    g = hq // hkv
    out = np.zeros((t_total, hq, pool_v.shape[3]), dtype=F32)
    qf = act(np.asarray(q, F32), mode).astype(np.float64)
    for t in range(t_total):
        req = int(query_to_req[t])
        if req < 0:
            continue
        for kv in range(hkv):
            n = int(vis_lens[req, kv])
            slots = np.asarray(gather[req, kv, :n], np.int64)
            slots = slots[slots >= 0]
            if len(slots) == 0:
                continue
            kk = pool_k[slots // page, kv, slots % page].astype(np.float64)
            vv = pool_v[slots // page, kv, slots % page].astype(np.float64)
            s = (qf[t, kv * g:(kv + 1) * g] @ kk.T) * float(scale)
            m = s.max(axis=1, keepdims=True)
            p = np.exp(s - m)
            z = p.sum(axis=1, keepdims=True)
            out[t, kv * g:(kv + 1) * g] = ((p @ vv) / z).astype(F32)
    return act(out, mode)
