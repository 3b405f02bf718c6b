// The prototype chain on a contiguous KV cache (reference: tls_attn/ops).
//
//   store KV        tls_attn/ops/mha_store_kv.py:10-141        (prefill copy, decode append)
//   store K index   tls_attn/ops/mha_store_k_index.py:10-185   (per-block min / max of the full key,
//                                                               tail sub-dimensions of every token)
//   level-1 indexer tls_attn/ops/mha_indexer_level1.py:11-249  (block bound scores, top-k blocks)
//   level-2 indexer tls_attn/ops/mha_indexer_level2.py:11-290  (token scores inside the chosen blocks,
//                                                               top-k tokens + forced sliding blocks)
//
// Layouts are the reference's: caches [maxB, S, Hkv, D] token-major, bf16; scores fp32.
// Scores accumulate in fp32 from bf16 operands like the reference kernels (q is scaled and
// rounded to bf16 first); the order of the fp32 sums differs, so scores agree to rounding,
// not bit for bit.  Top-k order is (score descending, then position ascending); entries that
// do not exist are (-inf, -1), as in the reference's buffers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "loda_common.cuh"

namespace loda {

using bf16 = __nv_bfloat16;

// ---------------------------------------------------------------------------
// store KV
// ---------------------------------------------------------------------------
// cache[b, s] = x[b, offsets[b] + s] for s < seqlen - offsets[b]; rows of row_bytes (multiple of 16)
__global__ void __launch_bounds__(256) tls_copy_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ offsets,
                                                            uint4* __restrict__ cache, int seqlen, int max_seqlen,
                                                            int row_vecs) {
  const int b = blockIdx.y;
  const int off = max(offsets[b], 0);
  const int n = min(max(seqlen - off, 0), max_seqlen);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int s = blockIdx.x * 8 + warp; s < n; s += gridDim.x * 8) {
    const uint4* src = x + ((size_t)b * seqlen + off + s) * row_vecs;
    uint4* dst = cache + ((size_t)b * max_seqlen + s) * row_vecs;
    for (int i = lane; i < row_vecs; i += 32) dst[i] = src[i];
  }
}

// cache[b, lengths[b] - 1] = x[b, 0]
__global__ void __launch_bounds__(128) tls_append_row_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ lengths,
                                                             uint4* __restrict__ cache, int max_seqlen, int row_vecs) {
  const int b = blockIdx.x;
  const int idx = lengths[b] - 1;
  if (idx < 0 || idx >= max_seqlen) return;
  const uint4* src = x + (size_t)b * row_vecs;
  uint4* dst = cache + ((size_t)b * max_seqlen + idx) * row_vecs;
  for (int i = threadIdx.x; i < row_vecs; i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------------------
// store K index
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }

// One warp per (b, block j, head): min / max over the block's tokens (a ragged last block is
// padded with zeros, as the reference pads), and the tail sub-dimensions of each token.
// Source rows are k[b, t0 + s, h, :] of a [*, src_len, Hkv, D] tensor; j0 / nblk select the blocks.
__global__ void __launch_bounds__(256) tls_k_index_kernel(const bf16* __restrict__ k, const int32_t* __restrict__ offsets,
                                                          const int32_t* __restrict__ lengths, bf16* __restrict__ l1min,
                                                          bf16* __restrict__ l1max, bf16* __restrict__ l2k, int src_len,
                                                          int hkv, int d, int bs, int cmp, int l1_len, int l2_len,
                                                          int decode) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int half = d / 2, hc = half / cmp, dc = 2 * hc;
  int t0, ntok, j_first, nblk;
  bool do_l1 = true;
  if (decode) {
    // the newest token (index = lengths[b] - 1) of a cache that already holds it
    const int index = lengths[b] - 1;
    if (index < 0 || index >= src_len) return;
    j_first = index / bs;
    nblk = 1;
    t0 = 0;
    ntok = index + 1;
    do_l1 = (index + 1) % bs == 0;
  } else {
    t0 = max(offsets[b], 0);
    ntok = max(src_len - t0, 0);
    j_first = 0;
    nblk = (ntok + bs - 1) / bs;
  }
  for (int jj = blockIdx.x * 8 + warp; jj < nblk; jj += gridDim.x * 8) {
    const int j = j_first + jj;
    const int s_lo = decode ? (do_l1 ? j * bs : ntok - 1) : j * bs;
    const int s_hi = min(j * bs + bs, ntok);
    // lanes over pairs of dims
    for (int p = lane; p < d / 2; p += 32) {
      float mn0 = INFINITY, mn1 = INFINITY, mx0 = -INFINITY, mx1 = -INFINITY;
      for (int s = s_lo; s < s_hi; ++s) {
        const uint32_t u = *(const uint32_t*)(k + (((size_t)b * src_len + t0 + s) * hkv + h) * d + 2 * p);
        const float x0 = bf16_lo(u), x1 = bf16_hi(u);
        mn0 = fminf(mn0, x0); mx0 = fmaxf(mx0, x0);
        mn1 = fminf(mn1, x1); mx1 = fmaxf(mx1, x1);
      }
      if (s_hi - j * bs < bs) {       // zero padding takes part in min / max
        mn0 = fminf(mn0, 0.0f); mx0 = fmaxf(mx0, 0.0f);
        mn1 = fminf(mn1, 0.0f); mx1 = fmaxf(mx1, 0.0f);
      }
      if (do_l1 && j < l1_len) {
        const size_t o = (((size_t)b * l1_len + j) * hkv + h) * d + 2 * p;
        *(__nv_bfloat162*)(l1min + o) = __floats2bfloat162_rn(mn0, mn1);
        *(__nv_bfloat162*)(l1max + o) = __floats2bfloat162_rn(mx0, mx1);
      }
    }
    // tail sub-dimensions [half - hc, half) and [d - hc, d) of every token of the block
    const int c_lo = decode ? ntok - 1 : j * bs;
    for (int e = lane; e < (s_hi - c_lo) * dc; e += 32) {
      const int s = c_lo + e / dc, c = e % dc;
      const int src = c < hc ? half - hc + c : d - hc + (c - hc);
      if (s < l2_len) l2k[(((size_t)b * l2_len + s) * hkv + h) * dc + c] = k[(((size_t)b * src_len + t0 + s) * hkv + h) * d + src];
    }
  }
}

// ---------------------------------------------------------------------------
// level 1: block bound scores
// ---------------------------------------------------------------------------
// score[b, h, s] = sum_g sum_d ( max(q,0)_gd * kmax_sd + min(q,0)_gd * kmin_sd ), q scaled and
// rounded to bf16 first; -inf at and beyond lengths[b] - sliding_blocks.  Eight lanes per block
// row (each lane 16-byte chunks of the row), the group's positive and negative parts summed
// over the heads beforehand (the sum over heads commutes with the dot).
template <int D>
__global__ void __launch_bounds__(256) tls_l1_scores_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kmin,
                                                            const bf16* __restrict__ kmax, const int32_t* __restrict__ lengths,
                                                            float* __restrict__ scores, int hq, int hkv, int l1_len,
                                                            int max_length, float scaling, int sliding_blocks,
                                                            int rows_per_cta) {
  constexpr int CH = D / 64;                     // 16-byte chunks per lane
  __shared__ float qpos[D], qneg[D];
  const int h = blockIdx.y, b = blockIdx.z, G = hq / hkv;
  for (int dd = threadIdx.x; dd < D; dd += blockDim.x) {
    float p = 0.0f, n = 0.0f;
    for (int g = 0; g < G; ++g) {
      const float x = __bfloat162float(q[((size_t)b * hq + h * G + g) * D + dd]);
      p += bf16r(fmaxf(x, 0.0f) * scaling);
      n += bf16r(fminf(x, 0.0f) * scaling);
    }
    qpos[dd] = p;
    qneg[dd] = n;
  }
  __syncthreads();
  const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;       // 32 rows per pass
  float qp[CH][8], qn[CH][8];
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) { qp[c][i] = qpos[(c * 8 + sub) * 8 + i]; qn[c][i] = qneg[(c * 8 + sub) * 8 + i]; }
  const int seqlen = lengths[b];
  const int s_end = min((int)(blockIdx.x + 1) * rows_per_cta, max_length);
  for (int s0 = blockIdx.x * rows_per_cta; s0 < s_end; s0 += 32) {       // uniform trip count: the shuffles need all lanes
    const int s = s0 + grp;
    const bool live = s < s_end && s < seqlen - sliding_blocks && s < l1_len;
    float acc = 0.0f;
    if (live) {
      const size_t row = (((size_t)b * l1_len + s) * hkv + h) * D;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const uint4 a = *(const uint4*)(kmax + row + (c * 8 + sub) * 8);
        const uint4 m = *(const uint4*)(kmin + row + (c * 8 + sub) * 8);
        const uint32_t av[4] = {a.x, a.y, a.z, a.w}, mv[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc = fmaf(bf16_lo(av[i]), qp[c][2 * i], acc);
          acc = fmaf(bf16_hi(av[i]), qp[c][2 * i + 1], acc);
          acc = fmaf(bf16_lo(mv[i]), qn[c][2 * i], acc);
          acc = fmaf(bf16_hi(mv[i]), qn[c][2 * i + 1], acc);
        }
      }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (sub == 0 && s < s_end) scores[((size_t)b * hkv + h) * max_length + s] = live ? acc : -INFINITY;
  }
}

// ---------------------------------------------------------------------------
// level 2: token scores inside the chosen blocks
// ---------------------------------------------------------------------------
// For slot t = i * bs + o of block_indices[b, h, i] = blk >= 0: token = blk * bs + o,
// s_g = (q_g * scaling rounded to bf16) . k[b, token, h, :], M = max over all slots and heads,
// score = sum_g exp(s_g - M).  Holes: (-inf, -1).  One CTA per (b, h); the dots are computed
// twice (maximum, then sums) instead of being kept.
__global__ void __launch_bounds__(256) tls_l2_scores_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                            const int32_t* __restrict__ block_indices,
                                                            float* __restrict__ scores, float* __restrict__ cummax,
                                                            int32_t* __restrict__ indices, int hq, int hkv, int dk,
                                                            int k_len, int k1, int bs, float scaling) {
  extern __shared__ __align__(16) unsigned char smem[];
  float* qs = (float*)smem;                      // [G][dk]
  float* red = qs + (hq / hkv) * dk;             // 8 warp maxima
  const int h = blockIdx.x, b = blockIdx.y, G = hq / hkv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < G * dk; i += blockDim.x)
    qs[i] = bf16r(__bfloat162float(q[((size_t)b * hq + h * G + i / dk) * dk + i % dk]) * scaling);
  __syncthreads();
  const int nslots = k1 * bs;
  const int32_t* bi = block_indices + ((size_t)b * hkv + h) * k1;
  auto dots = [&](int t, auto&& visit) {
    const int blk = bi[t / bs];
    if (blk < 0 || (size_t)blk * bs + bs > (size_t)k_len) return false;
    const bf16* row = k + (((size_t)b * k_len + (size_t)blk * bs + t % bs) * hkv + h) * dk;
    for (int g = 0; g < G; ++g) {
      float acc = 0.0f;
      for (int c = 0; c < dk; c += 8) {
        const uint4 u = *(const uint4*)(row + c);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc = fmaf(bf16_lo(w[i]), qs[g * dk + c + 2 * i], acc);
          acc = fmaf(bf16_hi(w[i]), qs[g * dk + c + 2 * i + 1], acc);
        }
      }
      visit(acc);
    }
    return true;
  };
  float m = -INFINITY;
  for (int t = tid; t < nslots; t += blockDim.x) dots(t, [&](float s) { m = fmaxf(m, s); });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) red[warp] = m;
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < (int)blockDim.x / 32; ++w) M = fmaxf(M, red[w]);
  const size_t base = ((size_t)b * hkv + h) * nslots;
  for (int t = tid; t < nslots; t += blockDim.x) {
    float sum = 0.0f;
    const bool ok = dots(t, [&](float s) { sum += expf(s - M); });
    scores[base + t] = ok ? sum : -INFINITY;
    if (cummax) cummax[base + t] = M;
    indices[base + t] = ok ? bi[t / bs] * bs + t % bs : -1;
  }
}

// The same in two launches when the caller provides the cummax buffer (it serves as scratch):
// (a) many CTAs per row: per slot m_t = max_g s_g into cummax, z_t = sum_g exp(s_g - m_t) into
// scores; (b) one CTA per row: M = max_t m_t, scores = z_t exp(m_t - M), cummax = M.
__global__ void __launch_bounds__(256) tls_l2_partial_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                             const int32_t* __restrict__ block_indices,
                                                             float* __restrict__ scores, float* __restrict__ cummax,
                                                             int32_t* __restrict__ indices, int hq, int hkv, int dk,
                                                             int k_len, int k1, int bs, float scaling) {
  extern __shared__ __align__(16) unsigned char smem[];
  float* qs = (float*)smem;                      // [G][dk]
  const int h = blockIdx.y, b = blockIdx.z, G = hq / hkv;
  for (int i = threadIdx.x; i < G * dk; i += blockDim.x)
    qs[i] = bf16r(__bfloat162float(q[((size_t)b * hq + h * G + i / dk) * dk + i % dk]) * scaling);
  __syncthreads();
  const int nslots = k1 * bs;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nslots) return;
  const size_t base = ((size_t)b * hkv + h) * nslots;
  const int blk = block_indices[((size_t)b * hkv + h) * k1 + t / bs];
  if (blk < 0 || (size_t)blk * bs + bs > (size_t)k_len) {
    scores[base + t] = -INFINITY;
    cummax[base + t] = -INFINITY;
    indices[base + t] = -1;
    return;
  }
  const bf16* row = k + (((size_t)b * k_len + (size_t)blk * bs + t % bs) * hkv + h) * dk;
  float m = -INFINITY, z = 0.0f;
  for (int g = 0; g < G; ++g) {
    float acc = 0.0f;
    for (int c = 0; c < dk; c += 8) {
      const uint4 u = *(const uint4*)(row + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc = fmaf(bf16_lo(w[i]), qs[g * dk + c + 2 * i], acc);
        acc = fmaf(bf16_hi(w[i]), qs[g * dk + c + 2 * i + 1], acc);
      }
    }
    const float mn = fmaxf(m, acc);
    z = z * expf(m - mn) + expf(acc - mn);       // m = -inf at g = 0: z * 0
    m = mn;
  }
  scores[base + t] = z;
  cummax[base + t] = m;
  indices[base + t] = blk * bs + t % bs;
}

__global__ void __launch_bounds__(512) tls_l2_rescale_kernel(float* __restrict__ scores, float* __restrict__ cummax, int nslots) {
  __shared__ float red[16];
  const size_t base = (size_t)blockIdx.x * nslots;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float m = -INFINITY;
  for (int t = tid; t < nslots; t += 512) m = fmaxf(m, cummax[base + t]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) red[warp] = m;
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < 16; ++w) M = fmaxf(M, red[w]);
  for (int t = tid; t < nslots; t += 512) {
    const float mt = cummax[base + t];
    if (mt != -INFINITY) scores[base + t] *= expf(mt - M);
    cummax[base + t] = M;
  }
}

// ---------------------------------------------------------------------------
// top-k of a row of fp32 scores, sorted (score descending, position ascending)
// ---------------------------------------------------------------------------
// Optional forced window: tokens [fw_lo, fw_hi) come first with score +inf (the sliding blocks
// of level 2).  Elements at -inf are not candidates; missing entries are (-inf, -1).
// One CTA per row: 4 x 8-bit radix select over the ordered keys (shared histogram), survivors
// gathered as 64-bit (key, ~position) words, bitonic sort of at most kpad words.
constexpr int TLS_TOPK_NT = 512;

__device__ __forceinline__ uint32_t f32_ordered(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float f32_from_ordered(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

__global__ void __launch_bounds__(TLS_TOPK_NT) tls_topk_kernel(const float* __restrict__ scores,
                                                               const int32_t* __restrict__ indices,
                                                               const int32_t* __restrict__ lengths, float* __restrict__ topk_scores,
                                                               int32_t* __restrict__ topk_indices, int hkv, int n, int k,
                                                               int kpad, int window_block, int window_blocks) {
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned long long* items = (unsigned long long*)smem;        // [kpad]
  int* hist = (int*)(items + kpad);                             // 256
  int* sh = hist + 256;                                         // 8
  int* wtot = sh + 8;                                           // 64
  const int tid = threadIdx.x;
  const int row = blockIdx.x, b = row / hkv;
  const float* sc = scores + (size_t)row * n;
  const int32_t* idx = indices ? indices + (size_t)row * n : nullptr;
  float* out_s = topk_scores + (size_t)row * k;
  int32_t* out_i = topk_indices + (size_t)row * k;
  const uint32_t NEG_INF_KEY = f32_ordered(-INFINITY);

  // forced window (level 2): the last window_blocks blocks of the sequence
  int nforced = 0;
  if (window_blocks > 0) {
    const int seqlen = lengths[b];
    if (seqlen > 0) {
      const int start = ((seqlen - 1) / window_block - window_blocks + 1) * window_block;
      const int lo = max(start, 0), hi = min(start + window_blocks * window_block, seqlen);
      nforced = min(max(hi - lo, 0), k);
      for (int i = tid; i < nforced; i += TLS_TOPK_NT) { out_s[i] = INFINITY; out_i[i] = lo + i; }
    }
  }
  const int want = k - nforced;

  // radix select of the want-th largest candidate key
  uint32_t prefix = 0, mask = 0;
  int remaining = want, ncand = 0;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += TLS_TOPK_NT) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += TLS_TOPK_NT) {
      const uint32_t key = f32_ordered(sc[i]);
      if (key != NEG_INF_KEY && (key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    // thread d < 256 owns digit d: number of matching keys with a larger digit, by a reversed scan
    {
      const int lane = tid & 31, warp = tid >> 5;
      const int mine = tid < 256 ? hist[255 - tid] : 0;          // reversed: position p holds digit 255 - p
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int nb = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += nb;
      }
      if (lane == 31 && warp < 8) wtot[warp] = incl;
      __syncthreads();
      int before = 0, total = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) { const int x = wtot[w]; total += x; before += w < warp ? x : 0; }
      const int above = before + incl - mine;                    // keys with a digit larger than this thread's
      if (tid == 0) { sh[2] = total; sh[0] = -1; }
      __syncthreads();
      if (tid < 256 && mine > 0 && above < remaining && remaining <= above + mine) { sh[0] = 255 - tid; sh[1] = remaining - above; }
    }
    __syncthreads();
    if (pass == 0) ncand = sh[2];        // (later passes count only the keys that match the prefix)
    if (ncand <= want || want <= 0) break;     // everything scored is kept
    prefix |= (uint32_t)sh[0] << shift;
    mask |= 255u << shift;
    remaining = sh[1];
    __syncthreads();
  }
  const bool all = ncand <= want;
  const int take = want <= 0 ? 0 : (all ? ncand : want);
  const uint32_t thr = prefix;                   // keep key > thr and the first `remaining` keys == thr
  // gather: strictly above in any order, ties in position order
  if (tid == 0) sh[3] = 0;
  for (int i = tid; i < kpad; i += TLS_TOPK_NT) items[i] = 0ull;
  __syncthreads();
  if (take > 0) {
    for (int i = tid; i < n; i += TLS_TOPK_NT) {
      const uint32_t key = f32_ordered(sc[i]);
      if (key != NEG_INF_KEY && (all || key > thr)) {
        const int p = atomicAdd(&sh[3], 1);
        if (p < kpad) items[p] = ((unsigned long long)key << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)i);
      }
    }
    __syncthreads();
    if (!all) {
      int base = sh[3], seen = 0;
      __syncthreads();
      for (int i0 = 0; i0 < n && seen < remaining; i0 += TLS_TOPK_NT) {
        const int i = i0 + tid;
        const bool tie = i < n && f32_ordered(sc[i]) == thr;
        int total;
        const int r = block_flag_scan<TLS_TOPK_NT>(tie, wtot, (i0 / TLS_TOPK_NT) & 1, &total);
        if (tie && seen + r < remaining && base + seen + r < kpad)
          items[base + seen + r] = ((unsigned long long)thr << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)i);
        seen += total;
      }
    }
    __syncthreads();
    // bitonic sort, descending
    for (int size = 2; size <= kpad; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int t = tid; t < kpad / 2; t += TLS_TOPK_NT) {
          const int lo = 2 * t - (t & (stride - 1));
          const int hi = lo + stride;
          const bool desc = (lo & size) == 0;
          const unsigned long long a = items[lo], c = items[hi];
          if ((a < c) == desc) { items[lo] = c; items[hi] = a; }
        }
        __syncthreads();
      }
    }
    for (int i = tid; i < take; i += TLS_TOPK_NT) {
      const unsigned long long it = items[i];
      const int pos = (int)(0xFFFFFFFFu - (uint32_t)(it & 0xFFFFFFFFull));
      out_s[nforced + i] = f32_from_ordered((uint32_t)(it >> 32));
      out_i[nforced + i] = idx ? idx[pos] : pos;
    }
  }
  for (int i = nforced + take + tid; i < k; i += TLS_TOPK_NT) { out_s[i] = -INFINITY; out_i[i] = -1; }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
cudaError_t tls_store_kv(const void* x, const int32_t* offsets_or_lengths, void* cache, int batch, int seqlen, int max_seqlen,
                         int row_bytes, bool decode, cudaStream_t st) {
  if (batch <= 0) return cudaSuccess;
  const int row_vecs = row_bytes / 16;
  if (decode) {
    tls_append_row_kernel<<<batch, 128, 0, st>>>((const uint4*)x, offsets_or_lengths, (uint4*)cache, max_seqlen, row_vecs);
  } else {
    const int gx = min(max((seqlen + 7) / 8, 1), 1024);
    tls_copy_rows_kernel<<<dim3(gx, batch), 256, 0, st>>>((const uint4*)x, offsets_or_lengths, (uint4*)cache, seqlen,
                                                         max_seqlen, row_vecs);
  }
  return cudaGetLastError();
}

cudaError_t tls_store_k_index(const void* k, const int32_t* offsets, const int32_t* lengths, void* l1min, void* l1max,
                              void* l2k, int batch, int src_len, int hkv, int d, int bs, int cmp, int l1_len, int l2_len,
                              bool decode, cudaStream_t st) {
  if (batch <= 0) return cudaSuccess;
  const int nblk = decode ? 1 : (src_len + bs - 1) / bs;
  const int gx = min(max((nblk + 7) / 8, 1), 2048);
  tls_k_index_kernel<<<dim3(gx, hkv, batch), 256, 0, st>>>((const bf16*)k, offsets, lengths, (bf16*)l1min, (bf16*)l1max,
                                                         (bf16*)l2k, src_len, hkv, d, bs, cmp, l1_len, l2_len,
                                                         decode ? 1 : 0);
  return cudaGetLastError();
}

cudaError_t tls_l1_scores(const void* q, const void* kmin, const void* kmax, const int32_t* lengths, float* scores,
                          int batch, int hq, int hkv, int d, int l1_len, int max_length, float scaling,
                          int sliding_blocks, cudaStream_t st) {
  if (batch <= 0 || max_length <= 0) return cudaSuccess;
  const int rows_per_cta = 256;
  const dim3 grid((max_length + rows_per_cta - 1) / rows_per_cta, hkv, batch);
  switch (d) {
    case 64:
      tls_l1_scores_kernel<64><<<grid, 256, 0, st>>>((const bf16*)q, (const bf16*)kmin, (const bf16*)kmax, lengths, scores,
                                                    hq, hkv, l1_len, max_length, scaling, sliding_blocks, rows_per_cta);
      break;
    case 128:
      tls_l1_scores_kernel<128><<<grid, 256, 0, st>>>((const bf16*)q, (const bf16*)kmin, (const bf16*)kmax, lengths, scores,
                                                     hq, hkv, l1_len, max_length, scaling, sliding_blocks, rows_per_cta);
      break;
    case 256:
      tls_l1_scores_kernel<256><<<grid, 256, 0, st>>>((const bf16*)q, (const bf16*)kmin, (const bf16*)kmax, lengths, scores,
                                                     hq, hkv, l1_len, max_length, scaling, sliding_blocks, rows_per_cta);
      break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t tls_l2_scores(const void* q, const void* k, const int32_t* block_indices, float* scores, float* cummax,
                          int32_t* indices, int batch, int hq, int hkv, int dk, int k_len, int k1, int bs, float scaling,
                          cudaStream_t st) {
  if (batch <= 0) return cudaSuccess;
  const size_t smem = (size_t)(hq / hkv) * dk * 4 + 64;
  if (cummax != nullptr) {
    const int nslots = k1 * bs;
    tls_l2_partial_kernel<<<dim3((nslots + 255) / 256, hkv, batch), 256, smem, st>>>(
        (const bf16*)q, (const bf16*)k, block_indices, scores, cummax, indices, hq, hkv, dk, k_len, k1, bs, scaling);
    tls_l2_rescale_kernel<<<batch * hkv, 512, 0, st>>>(scores, cummax, nslots);
    return cudaGetLastError();
  }
  tls_l2_scores_kernel<<<dim3(hkv, batch), 256, smem, st>>>((const bf16*)q, (const bf16*)k, block_indices, scores, cummax,
                                                          indices, hq, hkv, dk, k_len, k1, bs, scaling);
  return cudaGetLastError();
}

size_t tls_topk_smem(int kpad) { return (size_t)kpad * 8 + (256 + 8 + 64) * 4; }

cudaError_t tls_topk(const float* scores, const int32_t* indices, const int32_t* lengths, float* topk_scores,
                     int32_t* topk_indices, int rows, int hkv, int n, int k, int window_block, int window_blocks,
                     cudaStream_t st) {
  if (rows <= 0 || k <= 0) return cudaSuccess;
  int kpad = 2;
  while (kpad < k) kpad <<= 1;
  const size_t smem = tls_topk_smem(kpad);
  cudaError_t e = cudaFuncSetAttribute(tls_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  tls_topk_kernel<<<rows, TLS_TOPK_NT, smem, st>>>(scores, indices, lengths, topk_scores, topk_indices, hkv, n, k, kpad,
                                                  window_block, window_blocks);
  return cudaGetLastError();
}

int report_error(int code, const char* message);

}  // namespace loda

using namespace loda;

extern "C" {

static int tls_done(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return LODA_OK;
  char msg[160];
  snprintf(msg, sizeof(msg), "%s: %s", what, cudaGetErrorString(e));
  return report_error(LODA_ERR_LAUNCH, msg);
}

int loda_tls_store_kv(const void* k, const void* v, const int32_t* offsets_or_lengths, void* k_cache, void* v_cache,
                      int32_t batch, int32_t seqlen, int32_t max_seqlen, int32_t num_kv_heads, int32_t dim_k,
                      int32_t dim_v, int32_t decode, void* stream) {
  if (!k || !v || !offsets_or_lengths || !k_cache || !v_cache || batch < 0 || seqlen < 1 || max_seqlen < 1 ||
      num_kv_heads < 1 || dim_k < 1 || dim_v < 1)
    return report_error(LODA_ERR_ARGUMENT, "tls_store_kv: bad arguments");
  if ((num_kv_heads * dim_k) % 8 || (num_kv_heads * dim_v) % 8)
    return report_error(LODA_ERR_UNSUPPORTED, "tls_store_kv: a token row must be a multiple of 16 bytes");
  cudaError_t e = tls_store_kv(k, offsets_or_lengths, k_cache, batch, seqlen, max_seqlen, num_kv_heads * dim_k * 2,
                               decode != 0, (cudaStream_t)stream);
  if (e == cudaSuccess)
    e = tls_store_kv(v, offsets_or_lengths, v_cache, batch, seqlen, max_seqlen, num_kv_heads * dim_v * 2, decode != 0,
                     (cudaStream_t)stream);
  return tls_done(e, "tls_store_kv");
}

int loda_tls_store_k_index(const void* k, const int32_t* offsets_or_lengths, void* l1_min, void* l1_max, void* l2_k,
                           int32_t batch, int32_t src_len, int32_t num_kv_heads, int32_t dim_k, int32_t block,
                           int32_t cmp_ratio, int32_t l1_len, int32_t l2_len, int32_t decode, void* stream) {
  if (!k || !offsets_or_lengths || !l1_min || !l1_max || !l2_k || batch < 0 || src_len < 1 || num_kv_heads < 1 ||
      block < 1 || cmp_ratio < 1 || l1_len < 1 || l2_len < 1)
    return report_error(LODA_ERR_ARGUMENT, "tls_store_k_index: bad arguments");
  if (dim_k < 2 || dim_k % 2 || (dim_k / 2) % cmp_ratio)
    return report_error(LODA_ERR_ARGUMENT, "tls_store_k_index: dim_k / 2 must be a multiple of the compression ratio");
  return tls_done(tls_store_k_index(k, offsets_or_lengths, offsets_or_lengths, l1_min, l1_max, l2_k, batch, src_len,
                                    num_kv_heads, dim_k, block, cmp_ratio, l1_len, l2_len, decode != 0,
                                    (cudaStream_t)stream),
                  "tls_store_k_index");
}

int loda_tls_level1(const void* q, const void* k_min, const void* k_max, const int32_t* lengths, float* scores,
                    float* topk_scores, int32_t* topk_indices, int32_t batch, int32_t num_heads, int32_t num_kv_heads,
                    int32_t dim_k, int32_t l1_len, int32_t max_length, int32_t topk, int32_t sliding_blocks, float scaling,
                    void* stream) {
  if (!q || !k_min || !k_max || !lengths || !scores || !topk_scores || !topk_indices || batch < 0 || num_kv_heads < 1 ||
      num_heads < num_kv_heads || num_heads % num_kv_heads || l1_len < 1 || max_length < 1 || topk < 1 || sliding_blocks < 0)
    return report_error(LODA_ERR_ARGUMENT, "tls_level1: bad arguments");
  if (dim_k != 64 && dim_k != 128 && dim_k != 256) return report_error(LODA_ERR_UNSUPPORTED, "tls_level1: dim_k must be 64, 128 or 256");
  if (topk > 4096) return report_error(LODA_ERR_UNSUPPORTED, "tls_level1: topk > 4096");
  cudaError_t e = tls_l1_scores(q, k_min, k_max, lengths, scores, batch, num_heads, num_kv_heads, dim_k, l1_len, max_length,
                                scaling, sliding_blocks, (cudaStream_t)stream);
  if (e == cudaSuccess)
    e = tls_topk(scores, nullptr, lengths, topk_scores, topk_indices, batch * num_kv_heads, num_kv_heads, max_length, topk,
                 1, 0, (cudaStream_t)stream);
  return tls_done(e, "tls_level1");
}

int loda_tls_level2(const void* q, const void* k, const int32_t* block_indices, const int32_t* lengths, float* scores,
                    float* cummax_scores, int32_t* indices, float* topk_scores, int32_t* topk_indices, int32_t batch,
                    int32_t num_heads, int32_t num_kv_heads, int32_t dim_k, int32_t k_len, int32_t level1_topk,
                    int32_t level2_topk, int32_t block, int32_t sliding_blocks, float scaling, void* stream) {
  if (!q || !k || !block_indices || !lengths || !scores || !indices || !topk_scores || !topk_indices || batch < 0 ||
      num_kv_heads < 1 || num_heads < num_kv_heads || num_heads % num_kv_heads || k_len < 1 || level1_topk < 1 ||
      level2_topk < 1 || block < 1 || sliding_blocks < 0)
    return report_error(LODA_ERR_ARGUMENT, "tls_level2: bad arguments");
  if (dim_k < 8 || dim_k % 8) return report_error(LODA_ERR_UNSUPPORTED, "tls_level2: dim_k must be a multiple of 8");
  if (level2_topk > 4096) return report_error(LODA_ERR_UNSUPPORTED, "tls_level2: level2_topk > 4096");
  if ((size_t)(num_heads / num_kv_heads) * dim_k * 4 > 40 * 1024) return report_error(LODA_ERR_UNSUPPORTED, "tls_level2: group x dim_k too large");
  cudaError_t e = tls_l2_scores(q, k, block_indices, scores, cummax_scores, indices, batch, num_heads, num_kv_heads, dim_k,
                                k_len, level1_topk, block, scaling, (cudaStream_t)stream);
  if (e == cudaSuccess)
    e = tls_topk(scores, indices, lengths, topk_scores, topk_indices, batch * num_kv_heads, num_kv_heads,
                 level1_topk * block, level2_topk, block, sliding_blocks, (cudaStream_t)stream);
  return tls_done(e, "tls_level2");
}

}  // extern "C"

