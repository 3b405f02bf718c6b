// Shared device helpers of the loda_b200 kernels: bf16 rounding, ordered score
// keys, region geometry, block-wide radix select and scans.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "loda_b200.h"

// optional sub-phase timestamps inside the block routines (compile with -DLODA_PHASES):
// thread 0 of the CTAs with blockIdx.y == 0 records clock64() at numbered points
#ifdef LODA_PHASES
static __device__ long long g_subphase[64];
#ifdef LODA_SUB_X0      // one-dimensional grids: the first CTA only
#define LODA_SUB(i) do { if (threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.x == 0) g_subphase[(i)] = clock64(); } while (0)
#else
#define LODA_SUB(i) do { if (threadIdx.x == 0 && blockIdx.y == 0) g_subphase[(i)] = clock64(); } while (0)
#endif
#define LODA_SUB0(i) do { if (threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.x == 0) g_subphase[(i)] = clock64(); } while (0)
#define LODA_SUB_READER(name) extern "C" int loda_phase_read_sub_##name(long long* host) { \
    return (int)cudaMemcpyFromSymbol(host, g_subphase, sizeof(long long) * 64); }
#else
#define LODA_SUB(i)
#define LODA_SUB0(i)
#define LODA_SUB_READER(name)
#endif

namespace loda {

// ---------------------------------------------------------------------------
// numerics
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16r(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

// Monotone 16-bit key of a bf16-representable score: larger score -> larger
// key; NaN is canonicalised to the positive quiet NaN and sorts highest; -inf
// maps to ORD16_NEG_INF.  Same construction as the packed keys of
// nfa_layer_batch_selector.py:1482-1485.
__device__ __forceinline__ uint32_t ord16(float r) {
  uint32_t b = __float_as_uint(r) >> 16;
  if (r != r) b = 0x7FC0u;
  return (b & 0x8000u) ? ((~b) & 0xFFFFu) : (b | 0x8000u);
}
constexpr uint32_t ORD16_NEG_INF = 0x007Fu;

// index of subspace dim d inside the head: two contiguous halves
__device__ __forceinline__ int sub_dim(const loda_geometry& g, int d) {
  const int half = g.sub_dims >> 1;
  return d < half ? g.sub_lo0 + d : g.sub_lo1 + d - half;
}

// ---------------------------------------------------------------------------
// region geometry of one request (nfa_layer_batch_selector.py:209-262,
// 1136-1163, 1971-1986), with the frozen region-skip decisions of the request's
// layer (:223-226 pools, :1151-1163 middle range) and the numeric near-token
// quota (:872-920)
// ---------------------------------------------------------------------------
struct Regions {
  int length, kt_eff, near_blks, spl;
  int far_lo, far_hi;       // far pool = pages [far_lo, far_hi)
  int swa_lo_blk, swa_lo_tok, swa_byp_blk;
  bool swa_byp, sink_byp;
  int lower, upper, quota, kt_cap;   // quota: tokens the middle receives (both regions together under a numeric quota)
  int shard_rank, shard_count;   // sequence sharding: logical page p is scored here iff p % count == rank
  bool near_on;             // the near pool is scored (its region is not skipped)
  int near_lo_valid;        // with the far region skipped, near-pool pages below this one are invalid
  // numeric near-token quota: the far region [fq_lo, fq_hi) receives fq tokens, the near region
  // [nq_lo, nq_hi) nq; numeric == false: one quota over [lower, upper)
  bool numeric;
  int fq_lo, fq_hi, fq, nq_lo, nq_hi, nq;
};

__device__ __forceinline__ int cdiv_trunc(int a, int b) { return a / b; }  // C division truncates

__device__ __forceinline__ Regions make_regions(const loda_geometry& g, int length, bool skip_far = false,
                                                bool skip_near = false) {
  Regions r;
  const int bs = g.page, w = g.swa;
  r.length = length;
  r.kt_cap = g.max_blocks;
  r.spl = g.sink / bs;
  r.kt_eff = (length + bs - 1) / bs;
  r.near_blks = max(cdiv_trunc(length - w - g.pool_near_len, bs), r.spl);
  r.sink_byp = (g.sink % bs) != 0;
  r.far_lo = r.spl + (r.sink_byp ? 1 : 0);
  r.far_hi = min(min(r.near_blks, r.kt_eff), g.max_blocks);
  r.swa_lo_blk = max(r.near_blks, r.kt_eff - max(1, w / bs));
  r.swa_lo_tok = max(length - w, 0);
  r.swa_byp_blk = r.swa_lo_tok / bs;
  r.swa_byp = (r.swa_lo_tok % bs != 0) && (r.swa_byp_blk >= r.spl);
  if (r.sink_byp) r.swa_byp = r.swa_byp && (r.swa_byp_blk != r.spl);
  // token bound between the far and the near region
  const int sink_hi = min(g.sink, length);
  const int swa_hi = max(sink_hi, length - w);
  const int far_hi_tok = min(swa_hi, max(sink_hi, (max(length - w - g.near_len, 0) / bs) * bs));
  const int lower0 = r.spl * bs;
  const int upper0 = max(lower0, r.swa_lo_tok);
  r.lower = skip_far ? far_hi_tok : lower0;
  r.upper = max(r.lower, skip_near ? far_hi_tok : upper0);
  const int base_quota = max(min(length, g.level2_topk) - g.sink - (length - r.swa_lo_tok), 0);
  r.quota = min(base_quota, r.upper - r.lower);
  // pools of a row with a skipped region: the region's pool is empty, and a page of the other pool
  // counts only where it reaches into a region that is still on (block_valid of the reference)
  r.near_on = !skip_near;
  r.near_lo_valid = skip_far ? far_hi_tok / bs : 0;
  if (skip_far) r.far_hi = min(r.far_hi, r.far_lo);
  else if (skip_near) r.far_hi = min(r.far_hi, (far_hi_tok + bs - 1) / bs);
  r.numeric = g.near_tokens_p1 > 0;
  r.fq_lo = r.fq_hi = r.fq = r.nq_lo = r.nq_hi = r.nq = 0;
  if (r.numeric) {
    const int reserve = min(g.near_tokens_p1 - 1, base_quota);
    r.fq_lo = skip_far ? far_hi_tok : lower0;
    r.fq_hi = far_hi_tok;
    r.fq = min(max(base_quota - reserve, 0), max(r.fq_hi - r.fq_lo, 0));
    r.nq_lo = far_hi_tok;
    r.nq_hi = skip_near ? far_hi_tok : upper0;
    r.nq = min(max(base_quota - r.fq, 0), max(r.nq_hi - r.nq_lo, 0));
    r.quota = r.fq + r.nq;
  }
  r.shard_rank = g.shard_rank;
  r.shard_count = g.shard_count;
  return r;
}

// the skip decisions of request slot `req` in this layer (NULL arrays: nothing skipped)
__device__ __forceinline__ void load_skip_flags(const loda_layer& L, int req, bool* skip_far, bool* skip_near) {
  *skip_far = L.skip_far != nullptr && L.skip_far[req] != 0;
  *skip_near = L.skip_near != nullptr && L.skip_near[req] != 0;
}

// Request slot of an active batch row, checked: a slot outside [0, max_requests) makes the row a
// padding row (length 0, slot 0) and raises LODA_STATUS_BAD_REQ instead of addressing memory with it.
__device__ __forceinline__ int checked_request(const loda_geometry& g, long long act, long long val, int* length,
                                               uint32_t* status) {
  if (act < 0) { *length = 0; return (val >= 0 && val < g.max_requests) ? (int)val : 0; }
  if (val < 0 || val >= g.max_requests) {
    *length = 0;
    if (status && threadIdx.x == 0) atomicOr(status, LODA_STATUS_BAD_REQ);
    return 0;
  }
  return (int)val;
}

__device__ __forceinline__ bool page_owned(const Regions& r, int t) {
  return r.shard_count <= 1 || t % r.shard_count == r.shard_rank;
}

// (pool membership as this GPU scores it: under sequence sharding only the pages it owns)
__device__ __forceinline__ bool in_far_pool(const Regions& r, int t) {
  return t >= r.far_lo && t < r.far_hi && page_owned(r, t);
}

__device__ __forceinline__ bool in_near_pool(const Regions& r, int t) {
  if (t < r.near_blks || t >= r.swa_lo_blk || t >= r.kt_eff || t >= r.kt_cap) return false;
  if (!r.near_on || t < r.near_lo_valid) return false;
  if (r.swa_byp && t == r.swa_byp_blk) return false;
  if (r.sink_byp && t == r.spl) return false;
  return page_owned(r, t);
}

// First page behind both level-1 pools: tiles from there on hold no page that is scored (the sliding
// window's pages), so they are neither staged nor written.
__device__ __forceinline__ int pools_end(const Regions& r) {
  const int far_end = r.far_hi > r.far_lo ? r.far_hi : 0;
  const int near_end = r.near_on ? min(min(r.swa_lo_blk, r.kt_eff), r.kt_cap) : 0;
  return max(far_end, near_end);
}

#ifndef LODA_BISECT_INLINE
#define LODA_BISECT_INLINE __forceinline__
#endif

// Barrier of a thread group: BAR = 0 is the whole CTA (__syncthreads); BAR > 0 is the named
// barrier BAR over the CTA's first NT threads, for routines that run on a part of a larger CTA.
template <int NT, int BAR>
__device__ __forceinline__ void group_sync() {
  if constexpr (BAR == 0) __syncthreads();
  else asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(NT) : "memory");
}

// ---------------------------------------------------------------------------
// block-wide primitives (NT threads, all must call; BAR as in group_sync; TBASE = first thread of the group)
// ---------------------------------------------------------------------------

// Exclusive prefix sum of one int per thread; *total gets the block sum.
// scratch: 33 ints of shared memory.
template <int NT, int BAR = 0, int TBASE = 0>
__device__ __forceinline__ int block_exclusive_scan(int v, int* scratch, int* total) {
  const int lane = ((int)threadIdx.x - TBASE) & 31, warp = ((int)threadIdx.x - TBASE) >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  group_sync<NT, BAR>();
  if (lane == 31) scratch[warp] = incl;
  group_sync<NT, BAR>();
  if (warp == 0) {
    int w = lane < NT / 32 ? scratch[lane] : 0;
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    scratch[lane] = wi - w;
    if (lane == 31) scratch[32] = wi;
  }
  group_sync<NT, BAR>();
  *total = scratch[32];
  return scratch[warp] + incl - v;
}

// k-th largest of n unique non-zero 32-bit keys held in shared memory (zeros
// are "no key" and must number at most n - k).  Four 8-bit radix passes from
// the most significant byte.  hist: 258 ints of shared memory.
template <int NT>
__device__ __forceinline__ uint32_t block_kth_largest(const uint32_t* keys, int n, int k, int* hist) {
  uint32_t prefix = 0, mask = 0;
#pragma unroll 1
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += NT) hist[i] = 0;
    __syncthreads();
    // warp-aggregated histogram: lanes holding the same digit elect one lane to
    // add their count (scores share their leading bits, so un-aggregated atomics
    // would serialise 32-way on one shared-memory word)
    for (int base = 0; base < n; base += NT) {
      const int i = base + threadIdx.x;
      const uint32_t key = i < n ? keys[i] : 0u;
      const bool live = i < n && (key & mask) == prefix;
      const unsigned active = __ballot_sync(0xffffffffu, live);
      if (live) {
        const uint32_t digit = (key >> shift) & 255u;
        const unsigned peers = __match_any_sync(active, digit);
        if ((threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[digit], __popc(peers));
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      int c[8], s = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) { c[i] = hist[lane * 8 + i]; s += c[i]; }
      int above = 0;  // sum over the lanes holding larger digits
      int acc = s;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int nb = __shfl_down_sync(0xffffffffu, acc, o);
        if (lane + o < 32) acc += nb;
      }
      above = acc - s;
      if (above < k && k <= above + s) {
        int run = above;
#pragma unroll
        for (int i = 7; i >= 0; --i) {
          if (run < k && k <= run + c[i]) { hist[256] = lane * 8 + i; hist[257] = k - run; }
          run += c[i];
        }
      }
    }
    __syncthreads();
    prefix |= (uint32_t)hist[256] << shift;
    mask |= 255u << shift;
    k = hist[257];
    __syncthreads();
  }
  return prefix;
}

// ---------------------------------------------------------------------------
// Exact top-k over a row of 16-bit ordered scores in shared memory (0 = no
// score), ties toward the lower index, kept indices written in ASCENDING order.
// Three routines for three regimes; all return the number kept
// (min(k, #scored)).  A single CTA runs them, so what costs is latency, not
// throughput: the loops are written for instruction-level parallelism, block
// sums go through per-warp columns and one barrier (contended shared atomics
// serialise at ~65 cycles each), 1-bit flags are scanned with ballots, and the
// packed 16x2 compare intrinsics (emulated on this architecture) are avoided.
// The row must be 16-byte aligned and readable (zero) up to a multiple of 8.
// ---------------------------------------------------------------------------

// key that orders by (score descending, index ascending); 0 = no score
__device__ __forceinline__ uint32_t rank_key(uint32_t score, int idx) {
  return score ? (score << 16) | (uint32_t)(0xFFFF - idx) : 0u;
}

// how many of the n4 * 4 keys are greater than `key` (four independent chains)
__device__ __forceinline__ int count_greater(const uint32_t* keys, int n4, uint32_t key) {
  int r0 = 0, r1 = 0, r2 = 0, r3 = 0;
#pragma unroll 4
  for (int j = 0; j < n4; ++j) {
    const uint4 o = ((const uint4*)keys)[j];
    r0 += o.x > key; r1 += o.y > key; r2 += o.z > key; r3 += o.w > key;
  }
  return (r0 + r1) + (r2 + r3);
}

// exclusive scan of one flag per thread: ballot inside the warp, per-warp totals
// through shared memory, one barrier.  wtot: 2 x 32 ints (16-byte aligned), the
// caller alternates `buf` between back-to-back calls.
template <int NT, int BAR = 0, int TBASE = 0>
__device__ __forceinline__ int block_flag_scan(bool flag, int* wtot, int buf, int* total) {
  constexpr int NW = NT / 32;
  const int lane = ((int)threadIdx.x - TBASE) & 31, warp = ((int)threadIdx.x - TBASE) >> 5;
  const unsigned bal = __ballot_sync(0xffffffffu, flag);
  if (lane == 0) wtot[buf * 32 + warp] = __popc(bal);
  group_sync<NT, BAR>();
  int before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    const int c = wtot[buf * 32 + w];
    all += c;
    before += w < warp ? c : 0;
  }
  *total = all;
  return before + __popc(bal & ((1u << lane) - 1u));
}

// sum of one int per thread: redux, per-warp column, one barrier (same buffers)
template <int NT, int BAR = 0, int TBASE = 0>
__device__ __forceinline__ int block_sum_cols(int v, int* wtot, int buf) {
  constexpr int NW = NT / 32;
  const int r = __reduce_add_sync(0xffffffffu, v);
  if ((((int)threadIdx.x - TBASE) & 31) == 0) wtot[buf * 32 + (((int)threadIdx.x - TBASE) >> 5)] = r;
  group_sync<NT, BAR>();
  const int4* col = (const int4*)(wtot + buf * 32);
  int s = 0;
#pragma unroll
  for (int w4 = 0; w4 < (NW + 3) / 4; ++w4) {
    const int4 x = col[w4];
    s += (x.x + x.y) + (x.z + x.w);
  }
  return s;
}

__device__ __forceinline__ void unpack_u16x8(const uint4& u, uint32_t (&v)[8]) {
  v[0] = u.x & 0xFFFFu; v[1] = u.x >> 16; v[2] = u.y & 0xFFFFu; v[3] = u.y >> 16;
  v[4] = u.z & 0xFFFFu; v[5] = u.z >> 16; v[6] = u.w & 0xFFFFu; v[7] = u.w >> 16;
}

// (1) n <= NT scores: every thread ranks its own element against all others.
// keys: NT words (16-byte aligned); wtot: 64 ints.
template <int NT, int BAR = 0, int TBASE = 0>
__device__ __forceinline__ int block_rank_topk_small(const uint16_t* sc, int n, int k, int* out, uint32_t* keys,
                                                     int* wtot) {
  const int tid = ((int)threadIdx.x - TBASE);
  const uint32_t key = tid < n ? rank_key(sc[tid], tid) : 0u;
  keys[tid] = key;
  group_sync<NT, BAR>();
  const int rank = key ? count_greater(keys, (n + 3) >> 2, key) : 0;
  const bool sel = key != 0 && rank < k;
  int total;
  const int pos = block_flag_scan<NT, BAR, TBASE>(sel, wtot, 0, &total);
  if (sel) out[pos] = tid;
  group_sync<NT, BAR>();
  return total;
}

// (1b) NT < n <= 2 NT scores: the same with two elements per thread (tid, tid + NT).
// keys: 2 NT words (16-byte aligned); wtot: 64 ints.
template <int NT, int BAR = 0, int TBASE = 0>
__device__ __forceinline__ int block_rank_topk_pair(const uint16_t* sc, int n, int k, int* out, uint32_t* keys,
                                                    int* wtot) {
  const int tid = ((int)threadIdx.x - TBASE), hi = tid + NT;
  const uint32_t k0 = tid < n ? rank_key(sc[tid], tid) : 0u;
  const uint32_t k1 = hi < n ? rank_key(sc[hi], hi) : 0u;
  keys[tid] = k0;
  keys[hi] = k1;
  group_sync<NT, BAR>();
  int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
  const int n4 = (n + 3) >> 2;
#pragma unroll 4
  for (int j = 0; j < n4; ++j) {
    const uint4 o = ((const uint4*)keys)[j];
    a0 += (o.x > k0) + (o.y > k0); a1 += (o.z > k0) + (o.w > k0);
    b0 += (o.x > k1) + (o.y > k1); b1 += (o.z > k1) + (o.w > k1);
  }
  const bool s0 = k0 != 0 && a0 + a1 < k, s1 = k1 != 0 && b0 + b1 < k;
  int t0, t1;
  const int p0 = block_flag_scan<NT, BAR, TBASE>(s0, wtot, 0, &t0);
  const int p1 = block_flag_scan<NT, BAR, TBASE>(s1, wtot, 1, &t1);
  if (s0) out[p0] = tid;
  if (s1) out[t0 + p1] = hi;
  group_sync<NT, BAR>();
  return t0 + t1;
}

// Shared last step of the threshold selections: keep, in index order, the scores
// strictly above `thr` and the first `rem` scores equal to it (`all`: every scored
// element).  Blocked layout (ept consecutive scores per thread), one shuffle scan.
// wtot: 32 ints.  Returns all ? nvalid : k.
template <int NT, int BAR = 0, int TBASE = 0>
__device__ __forceinline__ int block_compact_threshold(const uint16_t* sc, int n, int k, uint32_t thr, int rem, bool all,
                                                       int nvalid, int* out, int* wtot) {
  constexpr int NW = NT / 32;
  const int tid = ((int)threadIdx.x - TBASE), lane = tid & 31, warp = tid >> 5;
  const int ept = (((n + NT - 1) / NT) + 7) & ~7;
  const int base = tid * ept;
  const int nch = base < n ? min(ept, ((n - base + 7) & ~7)) >> 3 : 0;
  const uint4* blk = (const uint4*)(sc + base);
  int gt = 0, tie = 0;
  for (int ch = 0; ch < nch; ++ch) {
    uint32_t v[8];
    unpack_u16x8(blk[ch], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) { gt += all ? v[j] != 0 : v[j] > thr; tie += (!all) && v[j] == thr; }
  }
  // exclusive scan of (gt | tie << 16): shuffles inside the warp, columns across warps
  int incl = gt | (tie << 16);
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int nb = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += nb;
  }
  group_sync<NT, BAR>();                             // the columns may still be read by slower warps
  if (lane == 31) wtot[warp] = incl;
  group_sync<NT, BAR>();
  int before = 0;
#pragma unroll
  for (int w = 0; w < NW; ++w) before += w < warp ? wtot[w] : 0;
  const int excl = before + incl - (gt | (tie << 16));
  int tb = excl >> 16;
  int pos = (excl & 0xFFFF) + min(tb, rem);
  for (int ch = 0; ch < nch; ++ch) {
    uint32_t v[8];
    unpack_u16x8(blk[ch], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = base + ch * 8 + j;
      if (all ? v[j] != 0 : v[j] > thr) out[pos++] = i;
      else if (!all && v[j] == thr) { if (tb < rem) out[pos++] = i; ++tb; }
    }
  }
  group_sync<NT, BAR>();
  return all ? nvalid : k;
}

// Bin of the k-th largest element in a histogram over the top 12 bits of 16-bit scores: 4096
// counters of 16 bits, two per word (bin b in word b >> 1, half b & 1; at most 65535 elements).
// Thread t covers the words [2048 - (t + 1) W, 2048 - t W), so the running sum over the threads
// counts from the largest bin down.  *nvalid receives the number of elements; the result is
// meaningful only when *nvalid > k > 0; *above (optional) receives the number of elements in the
// bins above it.  wtot: 64 ints, zero in the columns of absent warps.
template <int NT, int BAR = 0, int TBASE = 0>
__device__ __forceinline__ uint32_t block_hist_kth_bin(const uint32_t* hist, int k, int* wtot, int* nvalid,
                                                       int* above = nullptr) {
  static_assert(2048 % NT == 0 && (2048 / NT) % 4 == 0, "whole 16-byte vectors per thread");
  constexpr int NW = NT / 32, WPT = 2048 / NT;
  const int tid = ((int)threadIdx.x - TBASE), lane = tid & 31, warp = tid >> 5;
  const int w0 = 2048 - (tid + 1) * WPT;
  uint32_t w[WPT];
#pragma unroll
  for (int i = 0; i < WPT; i += 4) {
    const uint4 u = *(const uint4*)(hist + w0 + i);
    w[i] = u.x; w[i + 1] = u.y; w[i + 2] = u.z; w[i + 3] = u.w;
  }
  int own = 0;                         // elements in this thread's bins
#pragma unroll
  for (int i = 0; i < WPT; ++i) own += (int)((w[i] & 0xFFFFu) + (w[i] >> 16));
  int incl = own;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int nb = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += nb;
  }
  if (lane == 31) wtot[warp] = incl;
  group_sync<NT, BAR>();
  int before = 0, tot = 0;
#pragma unroll
  for (int w4 = 0; w4 < (NW + 3) / 4; ++w4) {
    const int4 x = ((const int4*)wtot)[w4];
    tot += (x.x + x.y) + (x.z + x.w);
    before += (w4 * 4 + 0 < warp ? x.x : 0) + (w4 * 4 + 1 < warp ? x.y : 0) + (w4 * 4 + 2 < warp ? x.z : 0) +
              (w4 * 4 + 3 < warp ? x.w : 0);
  }
  int c = before + incl - own;         // elements in bins above this thread's
  if (c < k && k <= c + own) {         // exactly one thread when tot >= k > 0
    int bin = 0, over = 0;               // over: elements in the bins above the chosen one
#pragma unroll
    for (int i = WPT - 1; i >= 0; --i) {
      const int hi = (int)(w[i] >> 16), lo = (int)(w[i] & 0xFFFFu);
      if (c < k && k <= c + hi) { bin = 2 * (w0 + i) + 1; over = c; }
      c += hi;
      if (c < k && k <= c + lo) { bin = 2 * (w0 + i); over = c; }
      c += lo;
    }
    wtot[32] = bin;
    wtot[33] = over;
  }
  group_sync<NT, BAR>();
  *nvalid = tot;
  if (above) *above = wtot[33];
  return (uint32_t)wtot[32];
}

// (2) any n < 65536, any k: bisection over the 16 score bits, two bits per round.
// The row is cut into chunks of 8 scores dealt round-robin to the threads (kept in
// registers); a last partial round of chunks that holds at most NT scores is dealt
// one score per thread instead, so that no thread pays for a whole chunk slot that
// only a few threads fill.  A first pass finds the number of scored elements and
// their minimum and maximum: the bits above the highest bit in which the two differ
// are those of the k-th largest score too, and their rounds are skipped.  Per round
// every thread counts its scores at or above three candidate thresholds (independent
// chains), one barrier publishes the block sums.
// wtot: 6 x 32 ints (16-byte aligned).
// With HIST the caller hands in a histogram of the scored elements by the top 12 bits of their
// score (block_hist_kth_bin): it replaces the first pass and the six rounds above the last four bits.
template <int NT, int BAR = 0, int TBASE = 0, int MAXC = 4, bool HIST = false>   // MAXC: chunks a thread keeps in registers
__device__ LODA_BISECT_INLINE int block_bisect_topk(const uint16_t* sc, int n, int k, int* out, int* wtot,
                                                    const uint32_t* hist = nullptr) {
  constexpr int NW = NT / 32;
  const int tid = ((int)threadIdx.x - TBASE), lane = tid & 31, warp = tid >> 5;
  const int nchunks = (n + 7) >> 3;
  const int full = nchunks / NT, remc = nchunks - full * NT;     // whole rounds of chunks, chunks left
  const bool single = remc > 0 && remc * 8 <= NT;                // the rest as one score per thread
  const int nslots = full + ((remc > 0 && !single) ? 1 : 0);
  // MAXC == 1: the caller guarantees n <= 9 NT (one chunk and one single score per thread at most)
  const bool in_regs = MAXC == 1 || nslots <= MAXC;
  uint4 mine[MAXC];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = tid + c * NT;
    mine[c] = (in_regs && c < nslots && ch < nchunks) ? ((const uint4*)sc)[ch] : make_uint4(0, 0, 0, 0);
  }
  const uint32_t xtra = (in_regs && single && tid < remc * 8) ? sc[full * NT * 8 + tid] : 0u;
  auto count3 = [&](uint32_t t1, uint32_t t2, uint32_t t3, int& c1, int& c2, int& c3) {
    c1 = xtra >= t1; c2 = xtra >= t2; c3 = xtra >= t3;           // thresholds are >= 1
    if (in_regs) {
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        if (c < nslots) {                        // uniform: skip register slots no thread uses
          uint32_t v[8];
          unpack_u16x8(mine[c], v);
#pragma unroll
          for (int j = 0; j < 8; ++j) { c1 += v[j] >= t1; c2 += v[j] >= t2; c3 += v[j] >= t3; }
        }
      }
    } else {
      for (int ch = tid; ch < nchunks; ch += NT) {
        uint32_t v[8];
        unpack_u16x8(((const uint4*)sc)[ch], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) { c1 += v[j] >= t1; c2 += v[j] >= t2; c3 += v[j] >= t3; }
      }
    }
  };
  // three sums with one barrier: columns [buf][counter][warp]
  auto sum3 = [&](int buf, int& c1, int& c2, int& c3) {
    c1 = __reduce_add_sync(0xffffffffu, c1);
    c2 = __reduce_add_sync(0xffffffffu, c2);
    c3 = __reduce_add_sync(0xffffffffu, c3);
    if (lane == 0) {
      wtot[(buf * 3 + 0) * 32 + warp] = c1;
      wtot[(buf * 3 + 1) * 32 + warp] = c2;
      wtot[(buf * 3 + 2) * 32 + warp] = c3;
    }
    group_sync<NT, BAR>();
    int s[3] = {0, 0, 0};
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const int4* col = (const int4*)(wtot + (buf * 3 + q) * 32);
#pragma unroll
      for (int w4 = 0; w4 < (NW + 3) / 4; ++w4) {
        const int4 x = col[w4];
        s[q] += (x.x + x.y) + (x.z + x.w);
      }
    }
    c1 = s[0]; c2 = s[1]; c3 = s[2];
  };
  LODA_SUB(0);
  for (int i = tid; i < 6 * 32; i += NT) wtot[i] = 0;      // columns of absent warps stay 0
  group_sync<NT, BAR>();
  LODA_SUB(1);
  // scored elements, their maximum, and 0xFFFF - their minimum (so that empty columns, 0, are neutral)
  int nvalid;
  uint32_t smax = 0, smin = 0, hist_bin = 0;
  int above = 0;         // scores at or above the upper end of the interval the threshold is known to lie in
  if constexpr (HIST) {
    hist_bin = block_hist_kth_bin<NT, BAR, TBASE>(hist, k, wtot, &nvalid, &above);
  } else {
    int nz = xtra != 0u;
    uint32_t mx = xtra, mi = xtra ? 0xFFFFu - xtra : 0u;
    auto visit = [&](const uint4& u) {
      uint32_t v[8];
      unpack_u16x8(u, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        nz += v[j] != 0u;
        mx = max(mx, v[j]);
        mi = max(mi, v[j] ? 0xFFFFu - v[j] : 0u);
      }
    };
    if (in_regs) {
#pragma unroll
      for (int c = 0; c < MAXC; ++c)
        if (c < nslots) visit(mine[c]);
    } else {
      for (int ch = tid; ch < nchunks; ch += NT) visit(((const uint4*)sc)[ch]);
    }
    nz = __reduce_add_sync(0xffffffffu, nz);
    mx = __reduce_max_sync(0xffffffffu, mx);
    mi = __reduce_max_sync(0xffffffffu, mi);
    if (lane == 0) {
      wtot[0 * 32 + warp] = nz;
      wtot[1 * 32 + warp] = (int)mx;
      wtot[2 * 32 + warp] = (int)mi;
    }
    group_sync<NT, BAR>();
    int a = 0, b = 0, c = 0;
#pragma unroll
    for (int w4 = 0; w4 < (NW + 3) / 4; ++w4) {
      const int4 x = ((const int4*)(wtot + 0 * 32))[w4];
      const int4 y = ((const int4*)(wtot + 1 * 32))[w4];
      const int4 z = ((const int4*)(wtot + 2 * 32))[w4];
      a += (x.x + x.y) + (x.z + x.w);
      b = max(max(b, max(y.x, y.y)), max(y.z, y.w));
      c = max(max(c, max(z.x, z.y)), max(z.z, z.w));
    }
    nvalid = a;
    smax = (uint32_t)b;
    smin = 0xFFFFu - (uint32_t)c;
  }
  LODA_SUB(2);
  if (k <= 0 || nvalid == 0) { group_sync<NT, BAR>(); return 0; }
  const bool all = nvalid <= k;
  uint32_t thr = 1u;     // keep v >= thr ...
  int rem = 0;           // ... but of those equal to thr only the first `rem` (all == true: everything scored)
  if (!all) {
    // rounds whose two bits lie above the highest bit in which minimum and maximum differ are decided
    const uint32_t diff = smax ^ smin;
    int first_round = 8;
    int buf = 1;           // the first pass used the columns of buffer 0; the buffers alternate from here
    thr = smax;
    if constexpr (HIST) {
      first_round = 6;     // the histogram decided the top 12 bits
      thr = hist_bin << 4;
    } else if (diff != 0u) {
      const int shift0 = (31 - __clz(diff)) & ~1;
      first_round = (14 - shift0) >> 1;
      thr = smax & ~((4u << shift0) - 1u);
    }
    // rounds 0..7 decide two bits each.  `above` follows the count at the upper end of the
    // threshold's interval (the next candidate above the chosen one), so that after the last
    // round it is the number of scores strictly above the threshold without a counting round
    // of its own.  (One rolled loop body: this code runs once per launch, and fetching it costs
    // as much as executing it.)
#pragma unroll 1
    for (int round = first_round; round < 8; ++round) {
      const int shift = 14 - 2 * round;
      int c1, c2, c3;
      count3(thr | (1u << shift), thr | (2u << shift), thr | (3u << shift), c1, c2, c3);
      sum3(buf, c1, c2, c3);
      buf ^= 1;
      const uint32_t d = c3 >= k ? 3u : c2 >= k ? 2u : c1 >= k ? 1u : 0u;   // largest candidate with >= k at or above
      above = d == 3u ? above : d == 2u ? c3 : d == 1u ? c2 : c1;
      thr |= d << shift;
      LODA_SUB(3 + round);
    }
    rem = k - above;
  }
  if constexpr (MAXC > 1) {
    if (!in_regs) return block_compact_threshold<NT, BAR, TBASE>(sc, n, k, thr, rem, all, nvalid, out, wtot);
  }
  // Compaction from the registers, in index order: consecutive threads hold consecutive
  // chunks of a slot, so one scan over the threads per slot places its survivors (strictly
  // above the threshold, then the first `rem` scores equal to it).  The single scores follow
  // every chunk in index order: they ride with the last slot's scan (two counters per thread,
  // one barrier), x is the thread's single score there and 0 in the slots before.
  int base_gt = 0, base_tie = 0, cbuf = 0;
  auto place = [&](const uint32_t (&v)[8], int idx0, uint32_t x) {
    // bit j of gm / tm: score j is above / equal to the threshold
    uint32_t gm = 0, tm = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      gm |= (uint32_t)(all ? v[j] != 0u : v[j] > thr) << j;
      tm |= (uint32_t)((!all) && v[j] == thr) << j;
    }
    const bool xg = all ? x != 0u : x > thr, xt = (!all) && x == thr;
    const int own = __popc(gm) | (__popc(tm) << 16), ownx = (int)xg | ((int)xt << 16);
    int incl = own, inclx = ownx;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int nb = __shfl_up_sync(0xffffffffu, incl, o), nx = __shfl_up_sync(0xffffffffu, inclx, o);
      if (lane >= o) { incl += nb; inclx += nx; }
    }
    if (lane == 31) { wtot[cbuf * 32 + warp] = incl; wtot[64 + cbuf * 32 + warp] = inclx; }
    group_sync<NT, BAR>();
    int before = 0, tot = 0, beforex = 0, totx = 0;
#pragma unroll
    for (int w4 = 0; w4 < (NW + 3) / 4; ++w4) {
      const int4 x4 = ((const int4*)(wtot + cbuf * 32))[w4];
      const int4 y4 = ((const int4*)(wtot + 64 + cbuf * 32))[w4];
      tot += (x4.x + x4.y) + (x4.z + x4.w);
      totx += (y4.x + y4.y) + (y4.z + y4.w);
      before += (w4 * 4 + 0 < warp ? x4.x : 0) + (w4 * 4 + 1 < warp ? x4.y : 0) + (w4 * 4 + 2 < warp ? x4.z : 0) +
                (w4 * 4 + 3 < warp ? x4.w : 0);
      beforex += (w4 * 4 + 0 < warp ? y4.x : 0) + (w4 * 4 + 1 < warp ? y4.y : 0) + (w4 * 4 + 2 < warp ? y4.z : 0) +
                 (w4 * 4 + 3 < warp ? y4.w : 0);
    }
    cbuf ^= 1;
    const int excl = before + incl - own;
    const int tb = base_tie + (excl >> 16);              // ties before this thread's scores
    const int pos = base_gt + (excl & 0xFFFF) + min(tb, rem);
    // of this thread's ties only the first rem - tb survive; every survivor's place follows
    // from the bits below it, so the eight stores are independent and predicated
    const int allowed = max(rem - tb, 0);
    uint32_t m = gm;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if ((tm >> j) & 1u) m |= (uint32_t)(__popc(tm & ((1u << j) - 1u)) < allowed) << j;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if ((m >> j) & 1u) out[pos + __popc(m & ((1u << j) - 1u))] = idx0 + j;
    }
    base_gt += tot & 0xFFFF;
    base_tie += tot >> 16;
    const int exclx = beforex + inclx - ownx;
    const int tbx = base_tie + (exclx >> 16);
    const int posx = base_gt + (exclx & 0xFFFF) + min(tbx, rem);
    if (xg || (xt && tbx < rem)) out[posx] = full * NT * 8 + tid;
    base_gt += totx & 0xFFFF;
    base_tie += totx >> 16;
  };
  group_sync<NT, BAR>();                               // the columns may still be read by slower warps
  if (tid < 128) wtot[tid] = 0;                  // rows of per-warp totals; absent warps stay 0
  group_sync<NT, BAR>();
  // one loop body for all slots (the registers rotate); a row of single scores alone takes one pass
  const int ns = min(nslots, MAXC);
#pragma unroll 1
  for (int c = 0; c < max(ns, 1); ++c) {
    uint32_t v[8];
    unpack_u16x8(c < ns ? mine[0] : make_uint4(0, 0, 0, 0), v);
    place(v, (tid + c * NT) * 8, c >= ns - 1 ? xtra : 0u);
#pragma unroll
    for (int r = 0; r + 1 < MAXC; ++r) mine[r] = mine[r + 1];
  }
  LODA_SUB(12);
  group_sync<NT, BAR>();
  LODA_SUB(13);
  return all ? nvalid : k;
}

// (3) large n, small k (k <= 128): a cheap lower bound on the k-th largest score
// discards almost everything, the survivors are ranked exactly.  The scores of
// the row are dealt round-robin to the threads, the threads form 256 groups;
// the k-th largest of the 256 group maxima is a lower bound of the k-th largest
// score (k groups each hold a score at or above it).  Scores at or above the
// bound (about 1.5 k of them for unclustered scores) are compacted in index
// order and ranked against each other.  Returns -1 without writing anything
// when more than 2 NT survive (heavily tied or sorted scores): the caller then
// bisects.  keys: 2 NT + 8 words (16-byte aligned); wtot: 64 ints; sh: 2 ints.
// With HIST the caller hands in a histogram of the row's scored elements by the top 12 bits of
// their score (block_hist_kth_bin): the bin of the k-th largest is the bound, and the survivors
// are the k best and the scores that share its bin.
template <int NT, int BAR = 0, int TBASE = 0, bool HIST = false>
__device__ __forceinline__ int block_prefilter_topk(const uint16_t* sc, int n, int k, int* out, uint32_t* keys,
                                                    int* wtot, int* sh, const uint32_t* hist = nullptr) {
  static_assert(NT % 256 == 0 && NT / 256 <= 32, "group layout");
  // The k-th largest of the group maxima is the tighter a bound the more groups there are: the g-th
  // largest group maximum is about the score of rank -NG ln(1 - g / NG), so k = 96 leaves ~120 survivors
  // with 256 groups and ~180 with 128 (whatever the row's length) — but ranking the maxima costs NG / 4
  // vector compares per thread.  Two threads share a maximum's ranking, so a CTA of 512 threads takes 256
  // groups and one of 256 threads 128: 16 + 45 compare rounds there instead of 64 + 30.
  constexpr int NG = NT >= 512 ? 256 : 128;      // groups
  constexpr int GS = NT / NG;                    // threads per group
  constexpr int NW = NT / 32;
  const int tid = ((int)threadIdx.x - TBASE), lane = tid & 31, warp = tid >> 5;
  const int nchunks = (n + 7) >> 3;
  LODA_SUB(16);
  uint32_t bound;
  if constexpr (HIST) {
    static_assert(NW % 4 == 0, "every column of the histogram scan is written");
    int nvalid;
    const uint32_t bin = block_hist_kth_bin<NT, BAR, TBASE>(hist, k, wtot, &nvalid);
    bound = nvalid > k ? max(bin << 4, 1u) : 1u;
  } else {
    // thread maximum over the scores tid, tid + NT, ...: a thread's scores lie NT positions apart, so a run of
    // neighbouring high scores (page scores vary slowly with position) spreads over as many groups as it is
    // long and the bound stays tight; dealt in chunks of 8 neighbours, such a run fed few groups and left
    // ten times as many survivors (two independent chains)
    uint32_t m0 = 0, m1 = 0;
#pragma unroll 1                                 // (the loops of this routine run once per launch: fetching an
    for (int i = tid; i < n; i += 2 * NT) {      //  unrolled copy costs more than the loop overhead it saves)
      m0 = max(m0, (uint32_t)sc[i]);
      if (i + NT < n) m1 = max(m1, (uint32_t)sc[i + NT]);
    }
    uint32_t m = max(m0, m1);
#pragma unroll
    for (int o = 1; o < GS; o <<= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & (GS - 1)) == 0) keys[tid / GS] = rank_key(m, tid / GS);
    if (tid == 0) sh[1] = 0;
    group_sync<NT, BAR>();
    LODA_SUB(17);
    int is_kth = 0;
    uint32_t gkey = 0;
    if constexpr (GS >= 2) {
      // two threads per maximum (tid and tid + NG, in different warps), each against half of the maxima;
      // the counts meet behind the maxima in `keys`
      const int part = tid / NG;
      gkey = keys[tid % NG];
      int cnt = 0;
      if (part < 2 && gkey != 0) cnt = count_greater(keys + part * (NG / 2), NG / 8, gkey);
      if (part < 2) keys[NG + tid] = (uint32_t)cnt;
      group_sync<NT, BAR>();
      if (tid < NG) {
        is_kth = gkey != 0 && (int)(keys[NG + tid] + keys[2 * NG + tid]) == k - 1;
        if (is_kth) sh[0] = (int)(gkey >> 16);
      }
    } else if (tid < NG) {
      gkey = keys[tid];
      is_kth = gkey != 0 && count_greater(keys, NG / 4, gkey) == k - 1;
      if (is_kth) sh[0] = (int)(gkey >> 16);
    }
    // fewer than k non-empty groups: nothing can be discarded
    if (is_kth) sh[1] = 1;                         // sh[1] was cleared before the barrier above
    group_sync<NT, BAR>();
    bound = sh[1] ? (uint32_t)sh[0] : 1u;
  }
  LODA_SUB(18);
  // survivors: every thread owns `cpt` consecutive chunks, so one scan over the thread counts places
  // them in index order (and yields the total)
  const int cpt = (nchunks + NT - 1) / NT;
  const int ch0 = tid * cpt, ch1 = min(ch0 + cpt, nchunks);
  int cnt = 0;
#pragma unroll 1
  for (int ch = ch0; ch < ch1; ++ch) {
    uint32_t v[8];
    unpack_u16x8(((const uint4*)sc)[ch], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) cnt += v[j] >= bound;
  }
  int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int nb = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += nb;
  }
  if (lane == 31) wtot[warp] = incl;
  group_sync<NT, BAR>();
  int before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    const int x = wtot[w];
    total += x;
    before += w < warp ? x : 0;
  }
  if (total > 2 * NT) return -1;
  LODA_SUB(19);
  {
    int pos = before + incl - cnt;
#pragma unroll 1
    for (int ch = ch0; ch < ch1 && cnt > 0; ++ch) {
      uint32_t v[8];
      unpack_u16x8(((const uint4*)sc)[ch], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (v[j] >= bound) keys[pos++] = rank_key(v[j], ch * 8 + j);
      }
    }
  }
  int buf = 1;
  if (tid < 4) keys[total + tid] = 0;            // pad the last vector of keys
  group_sync<NT, BAR>();
  LODA_SUB(20);
  // exact ranking of the survivors (already in ascending index order), up to two per thread
  const int n4 = (total + 3) >> 2;
  const uint32_t key0 = tid < total ? keys[tid] : 0u;
  if (total <= NT) {                             // uniform
    const bool sel0 = key0 != 0 && count_greater(keys, n4, key0) < k;
    int kept0;
    const int pos0 = block_flag_scan<NT, BAR, TBASE>(sel0, wtot, buf, &kept0);
    if (sel0) out[pos0] = 0xFFFF - (int)(key0 & 0xFFFFu);
    group_sync<NT, BAR>();
    LODA_SUB(21);
    return kept0;
  }
  // more survivors than threads: both keys of a thread are ranked in one pass over the keys
  const uint32_t key1 = tid + NT < total ? keys[tid + NT] : 0u;
  int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
#pragma unroll 2
  for (int j = 0; j < n4; ++j) {
    const uint4 o = ((const uint4*)keys)[j];
    a0 += (o.x > key0) + (o.y > key0); a1 += (o.z > key0) + (o.w > key0);
    b0 += (o.x > key1) + (o.y > key1); b1 += (o.z > key1) + (o.w > key1);
  }
  const bool sel0 = key0 != 0 && a0 + a1 < k, sel1 = key1 != 0 && b0 + b1 < k;
  int kept0, kept1;
  const int pos0 = block_flag_scan<NT, BAR, TBASE>(sel0, wtot, buf, &kept0);
  const int pos1 = block_flag_scan<NT, BAR, TBASE>(sel1, wtot, buf ^ 1, &kept1);
  if (sel0) out[pos0] = 0xFFFF - (int)(key0 & 0xFFFFu);
  if (sel1) out[kept0 + pos1] = 0xFFFF - (int)(key1 & 0xFFFFu);
  group_sync<NT, BAR>();
  LODA_SUB(21);
  return kept0 + kept1;
}

// ---------------------------------------------------------------------------
// Layout of the page statistics (page_mm, page_sum) of one (request, kv head) row: the logical
// pages are taken in groups of 32; inside a group the 16-byte chunks of the pages are stored chunk
// by chunk — chunk c of the 32 pages, then chunk c + 1 — so that 32 threads reading chunk c of 32
// consecutive pages touch one contiguous 512-byte run (coalesced in global memory, conflict-free in
// shared memory), and any run of whole groups is one contiguous block that a single bulk copy moves.
// CH = chunks per page: d' / 4 for page_mm (min then max), d' / 8 for page_sum.
// ---------------------------------------------------------------------------
constexpr int STAT_GROUP = 32;
__host__ __device__ __forceinline__ size_t stat_group_bytes(int CH) { return (size_t)STAT_GROUP * CH * 16; }
__host__ __device__ __forceinline__ size_t stat_row_bytes(int max_blocks, int CH) {
  return (size_t)((max_blocks + STAT_GROUP - 1) / STAT_GROUP) * stat_group_bytes(CH);
}
__host__ __device__ __forceinline__ size_t stat_chunk_offset(int page, int c, int CH) {
  return ((size_t)(page / STAT_GROUP) * CH + c) * (STAT_GROUP * 16) + (size_t)(page % STAT_GROUP) * 16;
}

// ---------------------------------------------------------------------------
// async copy
// ---------------------------------------------------------------------------
// Bulk asynchronous copy global -> shared memory of this CTA, completion counted in bytes on an
// mbarrier (both addresses and the size are multiples of 16 bytes).  Plain copies of this GPU's own
// memory into the issuing CTA's shared memory only.
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n.reg .b64 t;\nmbarrier.arrive.shared::cta.b64 t, [%0];\n}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Wait for a phase of the barrier, bounded: every try_wait suspends the thread for a while, and
// after MBAR_WAIT_LIMIT tries the wait gives up and returns false (the caller raises a status bit
// and carries on with whatever the buffer holds) — a copy that never lands cannot hang the GPU.
constexpr int MBAR_WAIT_LIMIT = 1 << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
#pragma unroll 1
  for (int i = 0; i < MBAR_WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool valid) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// ---------------------------------------------------------------------------
// programmatic dependent launch: a kernel of the chain may be scheduled while
// its predecessor in the stream still runs; it must not touch memory before
// pdl_wait(), which returns once the predecessor has completed and flushed.
// Both are no-ops for a kernel launched without the attribute.
// LODA_PDL_TRIGGER chooses where a kernel releases its dependent launch: 1 (default) =
// when its long phase is over (after the row's selection, after the attention tiles), so
// that the dependent's launch latency and prologue hide behind the closing phase only;
// 0 = at once.  Released at once, the dependent's CTAs sit on the SMs waiting while the
// single selecting CTA of a row still works, and slow it down: measured 4.4 us per
// layer-step (of 48.7) at batch 1.
// ---------------------------------------------------------------------------
#ifndef LODA_PDL_TRIGGER
#define LODA_PDL_TRIGGER 1
#endif
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// host: ordinal (-1 on failure) and multiprocessor count of the current device, looked up once per device
int device_ordinal();
int device_sm_count();

// decode append carried by extra CTAs of the L1 launch (enabled == 0: none)
struct AppendArgs {
  const __nv_bfloat16* k_new;   // NULL with enabled != 0: refresh the index only
  const __nv_bfloat16* v_new;
  const int32_t* slots;
  uint32_t* status;
  int enabled;
};

// ---------------------------------------------------------------------------
// Shared-memory carve-out asked for every kernel of the chain (percent of the maximum).
// All kernels ask for the same one: an SM has to drain before its L1/shared split can
// change, which would keep a dependent launch from starting beside its predecessor.
#ifndef LODA_CARVEOUT
#define LODA_CARVEOUT 100
#endif
template <typename K>
inline cudaError_t set_kernel_smem(K kernel, size_t smem) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess && LODA_CARVEOUT >= 0)
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, LODA_CARVEOUT);
  return e;
}

// optional phase timestamps (compile with -DLODA_PHASES): thread 0 of each CTA
// records clock64() at numbered points; LODA_PHASE_STORAGE defines the per-file
// array and a C reader.  Compiled out of the shipped library.
// ---------------------------------------------------------------------------
#ifdef LODA_PHASES
#define LODA_PHASE_CTAS 2048
#define LODA_PHASE_STORAGE(name)                                                        \
  static __device__ long long g_phase_##name[LODA_PHASE_CTAS][16];                      \
  extern "C" int loda_phase_read_##name(long long* host) {                              \
    return (int)cudaMemcpyFromSymbol(host, g_phase_##name, sizeof(long long) * LODA_PHASE_CTAS * 16); \
  }
// phase 0 also stores the global timer (ns) in slot 15 and the SM id in slot 14; slot 13
// holds the global timer of the latest phase >= 8 (the kernels' closing phases)
#define LODA_PHASE(name, cta, i)                                                        \
  do {                                                                                  \
    if (threadIdx.x == 0 && (cta) < LODA_PHASE_CTAS) {                                  \
      g_phase_##name[(cta)][(i)] = clock64();                                           \
      if ((i) == 0 || (i) >= 8) {                                                       \
        unsigned long long gt_;                                                         \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));                         \
        if ((i) == 0) {                                                                 \
          unsigned sm_;                                                                 \
          asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_));                              \
          g_phase_##name[(cta)][15] = (long long)gt_;                                   \
          g_phase_##name[(cta)][14] = sm_;                                              \
        }                                                                               \
        g_phase_##name[(cta)][13] = (long long)gt_;                                     \
      }                                                                                 \
    }                                                                                   \
  } while (0)
#else
#define LODA_PHASE_STORAGE(name)
#define LODA_PHASE(name, cta, i)
#endif

// scratch views handed to the kernels (carved out of the caller's workspace)
struct SelectWorkspace {
  int* l1_ticket;        // [ticket_rows + 2], zero between launches: a ticket per row, then the row queue
                         // and the exit count of the streaming level-1 kernel
  int ticket_rows;
  int* l2_ticket;        // [rows], zero between launches
  uint16_t* l1_scores;   // [rows, score_stride]: ordered bf16 score of every logical page (0 = not in a pool)
  int score_stride;
  int* pages;            // [rows, k_far + k_near + 2]: surviving pages, ascending, bypass pages included
  int* phys;             // [rows, k_far + k_near + 2]: their physical page ids (-1 = invalid)
  int* np;               // [rows]
  uint16_t* l2_scores;   // [rows, (k_far + k_near + 2) * page]: ordered bf16 logit per candidate slot
  // sequence sharding, selection phases: the score rows of all GPUs after an all-gather, [n_gathered] blocks
  // of the same shape as l1_scores (level 1) or l2_scores (level 2), gathered_stride elements apart; the
  // selecting CTA ORs them while loading (every page / slot is scored by exactly one GPU, the others hold 0).
  // NULL: the rows in l1_scores / l2_scores are already combined.
  const uint16_t* gathered = nullptr;
  int n_gathered = 0;
  size_t gathered_stride = 0;
};
struct AttnWorkspace {
  int* ticket;    // [n_query * Hkv], zero between launches
  float* part_m;  // [n_query * Hkv, nsplit, G]
  float* part_z;  // [n_query * Hkv, nsplit, G]
  float* part_o;  // [n_query * Hkv, nsplit, G, DV]
};

}  // namespace loda
