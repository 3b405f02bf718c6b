// Device pieces shared by the selector kernels: the canonical L1 page score, the L1 page
// selection of the selecting CTA, the L2 logit on the packed 4-bit tail keys.
#pragma once

#include "loda_common.cuh"

namespace loda {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xFFFF0000u);
  f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xFFFF0000u);
  f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xFFFF0000u);
  f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xFFFF0000u);
}

// tree over NC chunk sums (NC a power of two), adjacent pairs first
template <int NC>
__device__ __forceinline__ float chunk_tree(float (&p)[NC]) {
#pragma unroll
  for (int w = 1; w < NC; w <<= 1) {
#pragma unroll
    for (int i = 0; i + w < NC; i += 2 * w) p[i] = __fadd_rn(p[i], p[i + w]);
  }
  return p[0];
}

// canonical dot of DSUB register values with DSUB floats in shared memory
template <int DSUB>
__device__ __forceinline__ float dot_chunks(const float (&k)[DSUB], const float* qv) {
  constexpr int NC = DSUB / 8;
  float p[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const float4 q0 = *(const float4*)(qv + c * 8);
    const float4 q1 = *(const float4*)(qv + c * 8 + 4);
    float a = 0.0f;
    a = fmaf(k[8 * c + 0], q0.x, a); a = fmaf(k[8 * c + 1], q0.y, a);
    a = fmaf(k[8 * c + 2], q0.z, a); a = fmaf(k[8 * c + 3], q0.w, a);
    a = fmaf(k[8 * c + 4], q1.x, a); a = fmaf(k[8 * c + 5], q1.y, a);
    a = fmaf(k[8 * c + 6], q1.z, a); a = fmaf(k[8 * c + 7], q1.w, a);
    p[c] = a;
  }
  return chunk_tree<NC>(p);
}

// Packed fp32 arithmetic (two independent IEEE fp32 operations per instruction, sm_100): the low lane
// carries the min . min(q, 0) dot of the bound, the high lane the max . max(q, 0) dot, each in the
// canonical order — the same roundings as two scalar chains at half the instructions.
__device__ __forceinline__ unsigned long long pack_u32x2(uint32_t lo, uint32_t hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ unsigned long long ffma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long fadd2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// min/max bound of one head: kp[d] = (min_d, max_d) as packed fp32, qmm = (min(q_d, 0), max(q_d, 0)) interleaved
// in shared memory.  Chunks of 8 dims summed left to right from 0, chunk sums by the balanced tree, then the
// two lanes added: bit for bit dot_chunks(min, qlow) + dot_chunks(max, qhigh).
template <int DSUB>
__device__ __forceinline__ float bound_pair(const unsigned long long (&kp)[DSUB], const float* qmm) {
  constexpr int NC = DSUB / 8;
  unsigned long long p[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    unsigned long long a = 0ull;                       // (0.0f, 0.0f)
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const ulonglong2 q2 = *(const ulonglong2*)(qmm + (8 * c + i) * 2);
      a = ffma2(kp[8 * c + i], q2.x, a);
      a = ffma2(kp[8 * c + i + 1], q2.y, a);
    }
    p[c] = a;
  }
#pragma unroll
  for (int w = 1; w < NC; w <<= 1) {
#pragma unroll
    for (int i = 0; i + w < NC; i += 2 * w) p[i] = fadd2(p[i], p[i + w]);
  }
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p[0]));
  return __fadd_rn(lo, hi);
}

// Which statistic a pool's pages are scored on, and therefore staged: the min/max rows (true) or
// the sum row (false).  GENERIC == false fixes the default methods at compile time (far pool by
// the min/max bound, near pool by the page mean); GENERIC == true reads them from the geometry.
template <bool GENERIC>
__device__ __forceinline__ bool l1_far_uses_minmax(const loda_geometry& g) {
  return GENERIC ? g.far_method == LODA_FAR_MINMAX : true;
}
template <bool GENERIC>
__device__ __forceinline__ bool l1_near_uses_minmax(const loda_geometry& g) {
  return GENERIC ? g.near_minmax != 0 : false;
}

// ---------------------------------------------------------------------------
// Level-1 tiles.  A tile is TP consecutive logical pages of one (request, kv head) row = TP / 32
// groups of the interleaved statistics layout (STAT_GROUP).  A stage of shared memory holds one
// tile: a slot of SLOT bytes per group, byte-identical to the group in global memory (the group's
// min/max rows, or its sum rows in the first half of the slot), plus one spill slot of SUMG bytes
// for the sums of the one group of a row that holds pages of both pools (the far / near boundary).
// One bulk asynchronous copy per group and statistic fills it; an mbarrier counts the bytes.
// ---------------------------------------------------------------------------
template <int DSUB, int TP>
struct L1Tile {
  static constexpr int NC = DSUB / 8, CPR = 2 * NC, GROUPS = TP / STAT_GROUP;
  static constexpr int SLOT = STAT_GROUP * CPR * 16;      // one group of min/max rows
  static constexpr int SUMG = STAT_GROUP * NC * 16;       // one group of sum rows
  static constexpr int STAGE = GROUPS * SLOT + SUMG;      // bytes of one stage
};

// Does the group of 32 pages starting at page g0 hold pages scored on the min/max rows / on the sums?
template <bool GENERIC>
__device__ __forceinline__ void l1_group_needs(const loda_geometry& g, const Regions& rg, int g0, int page_end,
                                               bool* need_mm, bool* need_sum) {
  const int lo = g0, hi = min(g0 + STAT_GROUP, page_end);
  const bool has_far = rg.far_hi > rg.far_lo && lo < rg.far_hi && hi > rg.far_lo;
  const int nlo = max(rg.near_blks, rg.near_lo_valid), nhi = min(min(rg.swa_lo_blk, rg.kt_eff), rg.kt_cap);
  const bool has_near = rg.near_on && lo < nhi && hi > nlo && hi > lo;
  const bool far_mm = l1_far_uses_minmax<GENERIC>(g), near_mm = l1_near_uses_minmax<GENERIC>(g);
  *need_mm = (has_far && far_mm) || (has_near && near_mm);
  *need_sum = (has_far && !far_mm) || (has_near && !near_mm);
}

// Issue the copies of the tile [p0, p0 + TP) into `stage` and arm `bar` with their byte count.
// Called by all 32 lanes of one warp (lane i handles group i of the tile).  The groups of a row are
// contiguous in global memory and their slots contiguous in the stage, so the min/max rows of a run of
// neighbouring groups travel as ONE bulk copy (the usual tile lies inside the far pool: one copy of
// GROUPS * SLOT bytes instead of one per group, whose issue by the lanes of a warp is serialised);
// the sums (a handful of groups per row) and any second run go group by group.
template <int DSUB, int TP, bool GENERIC>
__device__ __forceinline__ void l1_issue_tile(const loda_geometry& g, const Regions& rg, int p0, int page_end,
                                              unsigned char* stage, uint64_t* bar, const unsigned char* mm_row,
                                              const unsigned char* sum_row) {
  using T = L1Tile<DSUB, TP>;
  const int lane = threadIdx.x & 31;
  bool nm = false, ns = false;
  if (lane < T::GROUPS) l1_group_needs<GENERIC>(g, rg, p0 + STAT_GROUP * lane, page_end, &nm, &ns);
  const uint32_t bytes = (nm ? T::SLOT : 0) + (ns ? T::SUMG : 0);
  const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
  const uint32_t mmask = __ballot_sync(0xffffffffu, nm);
  const int first = __ffs(mmask) - 1, count = __popc(mmask);
  const bool one_run = mmask != 0u && ((mmask >> first) + 1u & (mmask >> first)) == 0u;   // the set bits are neighbours
  if (lane == 0) mbar_arrive_expect_tx(bar, total);
  __syncwarp();
  const size_t gidx = (size_t)(p0 / STAT_GROUP) + lane;
  if (one_run) {
    if (lane == first) bulk_copy_g2s(stage + lane * T::SLOT, mm_row + gidx * T::SLOT, (uint32_t)count * T::SLOT, bar);
  } else if (nm) {
    bulk_copy_g2s(stage + lane * T::SLOT, mm_row + gidx * T::SLOT, T::SLOT, bar);
  }
  if (ns) bulk_copy_g2s(nm ? stage + T::GROUPS * T::SLOT : stage + lane * T::SLOT, sum_row + gidx * T::SUMG, T::SUMG, bar);
}

// Ordered 16-bit score of one logical page; 0 = the page is in neither pool or scores -inf.
// mm_src / sum_src: chunk 0 of the page's min/max rows / sum rows in the group layout (the chunks of a page
// lie STAT_GROUP * 16 bytes apart), in shared or global memory; only the one the page's pool is scored on
// is read.
// Per head the bound (min . min(q, 0) + max . max(q, 0)) or the mean score (mean . q) is rounded to
// bf16; the page score is the mean over the GQA group, rounded to bf16 — or, for the far method
// avg_top2, the mean of the two best per-head mean scores computed from the unrounded scaled query
// qraw (nfa_layer_batch_selector.py:290-354, 2412-2427).
template <int DSUB, bool GENERIC = false>
__device__ __forceinline__ uint32_t l1_page_score_src(const loda_geometry& g, const Regions& rg, int page,
                                                      const unsigned char* mm_src, const unsigned char* sum_src,
                                                      const float* qhat, const float* qmm, int G,
                                                      const float* qraw = nullptr) {
  constexpr int NC = DSUB / 8, CS = STAT_GROUP * 16;      // CS: bytes between two chunks of a page
  uint32_t ord = 0;
  const float gf = (float)G;
  const bool far = in_far_pool(rg, page);
  const bool near = !far && in_near_pool(rg, page);
  if (!far && !near) return 0u;
  const bool use_mm = far ? l1_far_uses_minmax<GENERIC>(g) : l1_near_uses_minmax<GENERIC>(g);
  if (use_mm) {
    const unsigned char* src = mm_src;
    unsigned long long kp[DSUB];                      // (min_d, max_d) as packed fp32
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const uint4 a = *(const uint4*)(src + c * CS), z = *(const uint4*)(src + (NC + c) * CS);
      kp[8 * c + 0] = pack_u32x2(a.x << 16, z.x << 16); kp[8 * c + 1] = pack_u32x2(a.x & 0xFFFF0000u, z.x & 0xFFFF0000u);
      kp[8 * c + 2] = pack_u32x2(a.y << 16, z.y << 16); kp[8 * c + 3] = pack_u32x2(a.y & 0xFFFF0000u, z.y & 0xFFFF0000u);
      kp[8 * c + 4] = pack_u32x2(a.z << 16, z.z << 16); kp[8 * c + 5] = pack_u32x2(a.z & 0xFFFF0000u, z.z & 0xFFFF0000u);
      kp[8 * c + 6] = pack_u32x2(a.w << 16, z.w << 16); kp[8 * c + 7] = pack_u32x2(a.w & 0xFFFF0000u, z.w & 0xFFFF0000u);
    }
    float acc = 0.0f;
#pragma unroll 1
    for (int j = 0; j < G; ++j) acc = __fadd_rn(acc, bf16r(bound_pair<DSUB>(kp, qmm + j * 2 * DSUB)));
    ord = ord16(bf16r(__fdiv_rn(acc, gf)));
  } else {
    const unsigned char* src = sum_src;
    float kavg[DSUB];
    // mean = sum / page: the page size is a power of two, so the division is an exact scaling and
    // the multiplication by 1 / page gives the same bits at a fraction of the instructions
    const float inv_bs = 1.0f / (float)g.page;
#pragma unroll
    for (int c = 0; c < NC; ++c) unpack8(*(const uint4*)(src + c * CS), *(float(*)[8])(kavg + 8 * c));
#pragma unroll
    for (int i = 0; i < DSUB; ++i) kavg[i] = bf16r(__fmul_rn(kavg[i], inv_bs));
    if (GENERIC && far && g.far_method == LODA_FAR_AVG_TOP2) {
      float t1 = -INFINITY, t2 = -INFINITY;
#pragma unroll 1
      for (int j = 0; j < G; ++j) {
        const float v = bf16r(dot_chunks<DSUB>(kavg, qraw + j * DSUB));
        const float second = v > t1 ? t1 : v;
        t1 = v > t1 ? v : t1;
        t2 = second > t2 ? second : t2;
      }
      ord = ord16(bf16r(__fdiv_rn(__fadd_rn(t1, t2), 2.0f)));
    } else {
      float acc = 0.0f;
#pragma unroll 1
      for (int j = 0; j < G; ++j) acc = __fadd_rn(acc, bf16r(dot_chunks<DSUB>(kavg, qhat + j * DSUB)));
      ord = ord16(bf16r(__fdiv_rn(acc, gf)));
    }
  }
  return ord == ORD16_NEG_INF ? 0u : ord;   // a -inf score never competes (it equals "not in the pool")
}

// The same for the logical page p0 + threadIdx.x of a tile staged by l1_issue_tile: the sums sit in the
// group's own slot, or in the spill slot when the group also staged min/max rows.
template <int DSUB, int TP, bool GENERIC = false>
__device__ __forceinline__ uint32_t l1_page_score(const loda_geometry& g, const Regions& rg, int p0, int page_end,
                                                  const unsigned char* stage, const float* qhat, const float* qmm,
                                                  int G, const float* qraw = nullptr) {
  using T = L1Tile<DSUB, TP>;
  const int grp = (int)threadIdx.x / STAT_GROUP, lane = (int)threadIdx.x % STAT_GROUP;
  bool nm, ns;
  l1_group_needs<GENERIC>(g, rg, p0 + grp * STAT_GROUP, page_end, &nm, &ns);
  const unsigned char* mm_src = stage + grp * T::SLOT + lane * 16;
  const unsigned char* sum_src = (nm ? stage + T::GROUPS * T::SLOT : stage + grp * T::SLOT) + lane * 16;
  return l1_page_score_src<DSUB, GENERIC>(g, rg, p0 + (int)threadIdx.x, mm_src, sum_src, qhat, qmm, G, qraw);
}

// the selecting CTA reuses the staging area: 40 KB for the far pool's scores (2 bytes per page)
// and 1 KB for the near pool's
constexpr size_t L1_TAIL_BYTES = 41 * 1024;
constexpr int L1_NEAR_CAP = 512;     // scores of the near row (1 KB behind the 40 KB far row)

// Rank the n kept pages of one pool best-first (score descending, lower id
// first) and append fillers (lowest page ids not kept): the page-id lists the
// reference selector exposes.  Optional output, used by parity checks.
template <int NT>
__device__ void emit_best_first(const int* kept, int n, int k, const uint16_t* sc, int32_t* out_ids,
                                int32_t* out_n, int max_blocks) {
  const int tid = threadIdx.x;
  for (int i = tid; i < n; i += NT) {
    const int id = kept[i];
    const uint32_t key = ((uint32_t)sc[id] << 16) | (uint32_t)(0xFFFF - id);
    int rank = 0;
    for (int j = 0; j < n; ++j) {
      const int idj = kept[j];
      rank += (((uint32_t)sc[idj] << 16) | (uint32_t)(0xFFFF - idj)) > key;
    }
    out_ids[rank] = id;
  }
  for (int j = tid; j < k - n; j += NT) {   // kept[] is ascending: j-th smallest id not kept
    int c = j;
    for (int i = 0; i < n; ++i) {
      if (kept[i] <= c) ++c; else break;
    }
    out_ids[n + j] = min(c, max_blocks - 1);
  }
  if (tid == 0) *out_n = n;
}

// The selecting CTA's work once the row's scores sit in shared memory, far pool in scf (pages
// [0, n_far), zero outside the pool) and near pool in scn (pages [near_lo8, near_lo8 + n_near)):
// exact top-k of each pool, the optional best-first lists, and the ascending page list
// kept[0, np) = [sink bypass] far... near... [window bypass].  Returns np.  All P threads call.
// keys: 2 P + 8 words; wtot: 256 ints; sh: 8 ints.
// trigger: release the dependent launch after the two selections.
// HIST (P == 512): hist holds the far pool's scores counted by their top 12 bits (block_hist_kth_bin).
template <int P, bool HIST = false>
__device__ __forceinline__ int l1_select_pages(const loda_geometry& g, const Regions& rg, const loda_selection& out,
                                               int row, uint16_t* scf, uint16_t* scn, int n_far, int far_lo, int n_near,
                                               int near_lo, int near_lo8, int near_hi, int* kept, uint32_t* keys,
                                               int* wtot, int* sh, bool trigger, const uint32_t* hist = nullptr) {
  static_assert(!HIST || P == 512, "the histogram serves the two-group selection");
  const int tid = threadIdx.x;
  int np = 0;
  const bool want_lists = out.i_far != nullptr;
  if (rg.quota > 0 || want_lists) {
    if (rg.quota > 0 && rg.sink_byp && rg.spl < rg.kt_eff) { if (tid == 0) kept[0] = rg.spl; np = 1; }
    int* kept_near = kept + np + g.k_far;                // compacted below
    int n_f = 0, n_n = 0;
    if constexpr (P == 512) {
      // the two pools are selected at the same time: far by the first 256 threads, near by the
      // other 256, each group on its own named barrier, key buffer and sum columns
      constexpr int H = 256;
      if (tid < H) {
        int r = 0;
        if (n_far > far_lo) {
          if (n_far <= H) {
            r = block_rank_topk_small<H, 1, 0>(scf, n_far, g.k_far, kept + np, keys, wtot);
          } else if (n_far <= 2 * H) {
            r = block_rank_topk_pair<H, 1, 0>(scf, n_far, g.k_far, kept + np, keys, wtot);
          } else {
            r = g.k_far <= 128 ? block_prefilter_topk<H, 1, 0, HIST>(scf, n_far, g.k_far, kept + np, keys, wtot, sh, hist)
                               : -1;
            if (r < 0) r = block_bisect_topk<H, 1, 0, 4, HIST>(scf, n_far, g.k_far, kept + np, wtot, hist);   // heavily tied scores
          }
        }
        if (tid == 0) sh[2] = r;
      } else {
        int r = 0;
        if (n_near > 0) {
          r = n_near <= H ? block_rank_topk_small<H, 2, H>(scn, n_near, g.k_near, kept_near, keys + 2 * H + 8, wtot + 192)
                          : block_rank_topk_pair<H, 2, H>(scn, n_near, g.k_near, kept_near, keys + 2 * H + 8, wtot + 192);
          for (int i = tid - H; i < r; i += H) kept_near[i] += near_lo8;
        }
        if (tid == H) sh[3] = r;
      }
      LODA_SUB(22);
      __syncthreads();
      LODA_SUB(23);
      n_f = sh[2];
      n_n = sh[3];
    } else {
      if (n_far > far_lo) {
        if (n_far <= P) {
          n_f = block_rank_topk_small<P>(scf, n_far, g.k_far, kept + np, keys, wtot);
        } else {
          n_f = g.k_far <= 128 ? block_prefilter_topk<P>(scf, n_far, g.k_far, kept + np, keys, wtot, sh) : -1;
          if (n_f < 0) n_f = block_bisect_topk<P>(scf, n_far, g.k_far, kept + np, wtot);   // heavily tied scores
        }
      }
      if (n_near > 0) {
        // the near row starts at a multiple of 8 pages; ranked from the pool's first page on, the usual
        // pool of P pages takes the one-score-per-thread routine (half the compares of the pair routine)
        const int lead = near_lo - near_lo8, nn = n_near - lead;
        if (nn > 0)
          n_n = nn <= P ? block_rank_topk_small<P>(scn + lead, nn, g.k_near, kept_near, keys, wtot)
                        : block_rank_topk_pair<P>(scn + lead, nn, g.k_near, kept_near, keys, wtot);
        for (int i = tid; i < n_n; i += P) kept_near[i] += near_lo;
        __syncthreads();
      }
    }
    if (trigger) pdl_launch_dependents();
    if (want_lists) {
      // best-first lists need the scores by page id: near scores go back beside the far ones
      for (int i = near_lo + tid; i < near_hi; i += P) scf[i] = scn[i - near_lo8];
      __syncthreads();
      emit_best_first<P>(kept + np, n_f, g.k_far, scf, out.i_far + (size_t)row * g.k_far, out.n_far + row, g.max_blocks);
      emit_best_first<P>(kept_near, n_n, g.k_near, scf, out.i_near + (size_t)row * g.k_near, out.n_near + row,
                         g.max_blocks);
      __syncthreads();
    }
    LODA_SUB(25);
    if (rg.quota > 0) {
      // ascending list: [sink bypass] far... near... [window bypass]
      const int v0 = tid < n_n ? kept_near[tid] : 0;     // k_near <= 2 P
      const int v1 = tid + P < n_n ? kept_near[tid + P] : 0;
      __syncthreads();
      LODA_SUB(26);
      if (tid < n_n) kept[np + n_f + tid] = v0;
      if (tid + P < n_n) kept[np + n_f + tid + P] = v1;
      np += n_f + n_n;
      if (rg.swa_byp) { if (tid == 0) kept[np] = rg.swa_byp_blk; ++np; }
    }
    LODA_SUB(27);
    __syncthreads();
    LODA_SUB(24);
  }
  return np;
}

// Logit of one token from its packed 4-bit codes (WORDS 32-bit words, dim 2i in the low nibble of byte i):
// de-quantised key bf16(bf16(code * scale) - zero), one left-to-right fp32 chain of separate multiplies
// and adds over the d' dims, rounded to bf16.
// The de-quantisation runs two dims at a time in packed bf16 arithmetic, which gives the same bits as
// the fp32 form with its two roundings to bf16 and keeps the conversion unit (a quarter of the fp32
// rate, and three conversions per dim in the fp32 form) out of the loop:
//   code -> bf16: 0x4300 | code is the bf16 number 128 + code; minus 128 is exact;
//   bf16(code * scale): the product of an integer below 16 and a bf16 number is exact in fp32, so the
//     fp32 form rounds once, as mul.rn.bf16x2 does;
//   bf16(t - zero): the difference of two bf16 numbers is exact in fp32 when their exponents differ by
//     15 or less; beyond that the smaller one is less than 2^-6 of half a bf16 unit of the larger, and
//     both forms return the larger: one rounding either way.
// sz: the token's (scale, zero) pair as stored, scale in the low half.
// ROLLED: one loop body per word of codes, for a caller that scores a single slot per thread (the
// straight-line form costs more in instruction fetch there than its arithmetic)
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// the eight de-quantised keys of one word of codes, as fp32
__device__ __forceinline__ void l2_dequant_word(uint32_t w, uint32_t scale2, uint32_t zero2, float (&x)[8]) {
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    // nibble n into the low half, nibble n + 4 into the high half, each as the bf16 number 128 + code
    const uint32_t c = bf16x2_sub(((w >> (4 * n)) & 0x000F000Fu) | 0x43004300u, 0x43004300u);
    const uint32_t k = bf16x2_sub(bf16x2_mul(c, scale2), zero2);
    x[n] = __uint_as_float(k << 16);
    x[n + 4] = __uint_as_float(k & 0xFFFF0000u);
  }
}

template <int DSUB, bool ROLLED = false>
__device__ __forceinline__ float l2_logit_words(uint32_t (&w)[DSUB / 8], uint32_t sz, const float* __restrict__ qf) {
  constexpr int WORDS = DSUB / 8;   // 32-bit words of packed codes
  const uint32_t scale2 = __byte_perm(sz, 0u, 0x1010), zero2 = __byte_perm(sz, 0u, 0x3232);
  float acc = 0.0f;
  if constexpr (ROLLED) {
#pragma unroll 1
    for (int i = 0; i < WORDS; ++i) {
      const uint32_t wi = w[0];
#pragma unroll
      for (int r = 0; r + 1 < WORDS; ++r) w[r] = w[r + 1];       // the registers rotate
      float x[8];
      l2_dequant_word(wi, scale2, zero2, x);
#pragma unroll
      for (int n = 0; n < 8; ++n) acc = __fadd_rn(acc, __fmul_rn(x[n], qf[8 * i + n]));
    }
  } else {
#pragma unroll
    for (int i = 0; i < WORDS; ++i) {
      float x[8];
      l2_dequant_word(w[i], scale2, zero2, x);
#pragma unroll
      for (int n = 0; n < 8; ++n) acc = __fadd_rn(acc, __fmul_rn(x[n], qf[8 * i + n]));
    }
  }
  return bf16r(acc);
}

template <int DSUB>
__device__ __forceinline__ void l2_load_codes(const uint8_t* __restrict__ codes, uint32_t (&w)[DSUB / 8]) {
  constexpr int WORDS = DSUB / 8;
  if constexpr (WORDS == 4) {
    const uint4 u = *(const uint4*)codes;
    w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w;
  } else if constexpr (WORDS == 2) {
    const uint2 u = *(const uint2*)codes;
    w[0] = u.x; w[1] = u.y;
  } else {
#pragma unroll
    for (int i = 0; i < WORDS; i += 4) {
      const uint4 u = *(const uint4*)(codes + 4 * i);
      w[i] = u.x; w[i + 1] = u.y; w[i + 2] = u.z; w[i + 3] = u.w;
    }
  }
}

template <int DSUB, bool ROLLED = false>
__device__ __forceinline__ float l2_logit(const uint8_t* __restrict__ codes, uint32_t sz, const float* __restrict__ qf) {
  uint32_t w[DSUB / 8];
  l2_load_codes<DSUB>(codes, w);
  return l2_logit_words<DSUB, ROLLED>(w, sz, qf);
}

// Ordered 16-bit logit of candidate slot (logical page pg, physical page ph, offset o); 0 = the
// token is not a candidate (outside the scored window, NaN or -inf logit, invalid page).
template <int DSUB, bool ROLLED = false>
__device__ __forceinline__ uint32_t l2_slot_score(const loda_geometry& g, const loda_layer& L, const Regions& rg,
                                                  int length, int kv, int pg, int ph, int o, const float* qf,
                                                  uint32_t* status) {
  const int tok = pg * g.page + o;
  uint32_t ord = 0;
  if (ph >= 0 && tok >= g.sink && tok < rg.swa_lo_tok && tok < length && tok >= rg.lower && tok < rg.upper) {
    const size_t trow = ((size_t)ph * g.num_kv_heads + kv) * g.page + o;
    const uint32_t sz = *(const uint32_t*)((const bf16*)L.tail_sz + trow * 2);
    const float lg = l2_logit<DSUB, ROLLED>((const uint8_t*)L.tail_code + trow * (DSUB / 2), sz, qf);
    if (lg == lg && lg != -INFINITY) ord = ord16(lg);
  } else if (ph < 0 && status && rg.shard_count <= 1) {     // under sequence sharding a missing page is another GPU's
    atomicOr(status, LODA_STATUS_BAD_PAGE);
  }
  return ord;
}

// The selecting CTA's work once the row's candidate scores sit in shared memory (sc, nitems
// slots; slot i * page + o is token pages[i] * page + o, physical page physs[i]): keep the
// quota best by bisection, fill holes, drop ids below the sink, and write
// sink ++ middle ++ window as physical slots.  Runs on the first NT threads of the CTA
// (BAR as in group_sync).  trigger: release the dependent launch after the selection.
// With a numeric near-token quota (rg.numeric) the far and the near region select separately on
// masked copies of the scores and their survivors are concatenated
// (nfa_layer_batch_selector.py:2274-2332); that needs sm.sc2 and sm.fin.
struct L2Shared {
  uint16_t* sc;
  int *pages, *physs, *mid_a, *mid_b, *wtot, *scan;
  uint8_t* win;
  const uint32_t* hist = nullptr;    // HIST: 12-bit histogram of the candidate scores (block_hist_kth_bin)
  int* list = nullptr;               // optional copy of the gather list in shared memory (max_visible ints) ...
  int* list_n = nullptr;             // ... and of its length
  uint16_t* sc2 = nullptr;           // numeric quota: nitems scores of one region
  int* fin = nullptr;                // numeric quota: level2_topk ints, the concatenated middle
};

#ifndef LODA_L2TAIL_INLINE
#define LODA_L2TAIL_INLINE __forceinline__
#endif
// NUMERIC: compile the numeric near-token quota path (a second selection and its hole fill); kernels that only
// serve the default quota leave it out — this code runs once per launch, cold, and its size is paid in
// instruction fetch
template <int NT, int BAR, bool HIST = false, bool NUMERIC = false>
__device__ LODA_L2TAIL_INLINE void l2_select_and_write(const loda_geometry& g, const Regions& rg, const loda_selection& S,
                                                    uint32_t* status, const int32_t* table, int b, int kv, int row,
                                                    int length, int nitems, const L2Shared& sm, int* ticket,
                                                    bool trigger) {
  const int tid = threadIdx.x;
  const int K2 = g.level2_topk;
  const int pl2 = 31 - __clz(g.page), pmask = g.page - 1;      // page is a power of two
  uint16_t* sc = sm.sc;
  int *pages = sm.pages, *physs = sm.physs, *mid_a = sm.mid_a, *mid_b = sm.mid_b, *wtot = sm.wtot, *scan = sm.scan;
  uint8_t* win = sm.win;
  int* slots_sel = mid_b;      // ascending candidate slots kept by the select

  // sink ++ mid[0, count_m) ++ window as physical slots through the block table
  auto write_union = [&](const int* mid, int count_m) {
    const int cap = g.max_blocks * g.page;
    const int sk_all = min(length, g.sink);
    const int count_s = min(length, g.sink + g.swa) - sk_all;
    const int s_lo = max(max(length - g.swa, 0), sk_all);
    const int s_hi = min(length - g.swa + count_s, cap);
    const int sk = S.middle_only ? 0 : sk_all;                       // middle only: no sink, no window
    const int n_s = S.middle_only ? 0 : max(s_hi - s_lo, 0);
    const int total = sk + count_m + n_s;
    const int n_out = min(total, g.max_visible);
    int32_t* gout = S.gather + ((size_t)b * g.num_kv_heads + kv) * g.max_visible;
    for (int i = tid; i < n_out; i += NT) {
      int id;
      if (i < sk) id = i;
      else if (i < sk + count_m) id = mid[i - sk];
      else id = s_lo + (i - sk - count_m);
      const int lp = (id >> pl2);
      int ph = lp < g.max_blocks ? table[lp] : -1;
      if (ph < 0 || ph >= g.num_pages) {
        if (rg.shard_count > 1) {
          ph = -1;              // another GPU's page: skipped by the attention
        } else {
          if (status) atomicOr(status, LODA_STATUS_BAD_PAGE);
          ph = g.num_pages - 1;   // PAD page: zeros, never out of bounds
        }
      }
      const int slot = ph >= 0 ? ph * g.page + (id & pmask) : -1;
      gout[i] = slot;
      if (sm.list) sm.list[i] = slot;
    }
    if (tid == 0) {
      if (sm.list_n) *sm.list_n = n_out;
      S.visible_lens[(size_t)b * g.num_kv_heads + kv] = n_out;
      if (total > g.max_visible && status) atomicOr(status, LODA_STATUS_TRUNCATED);
      if (ticket) *ticket = 0;
    }
  };

  // Survivors (slots_sel[0, take), ascending slots) of a selection with quota q over [lo, hi) as
  // ascending token ids: hole fill (nfa_layer_batch_selector.py:545-566), then ids below the sink
  // dropped (only holes can be there).  Returns the list and its length.
  auto finish_region = [&](int take, int lo, int q, int* count_out) -> const int* {
    for (int i = tid; i < take; i += NT) {
      const int sl = slots_sel[i];
      mid_a[i] = pages[(sl >> pl2)] * g.page + (sl & pmask);
    }
    group_sync<NT, BAR>();
    int count = take;
    int* mid = mid_a;
    if (take < q) {
      const int need = q - take;
      // the holes are among the first q ids of [lo, hi) (q <= hi - lo)
      for (int i = tid; i < q; i += NT) win[i] = 0;
      group_sync<NT, BAR>();
      int in_win = 0;
      for (int i = tid; i < take; i += NT) {
        const int w = mid_a[i] - lo;
        if (w < q) { win[w] = 1; ++in_win; }
      }
      int cw;
      block_exclusive_scan<NT, BAR>(in_win, scan, &cw);
      const int ipt = (q + NT - 1) / NT;
      const int wlo = min(tid * ipt, q), whi = min(wlo + ipt, q);
      int zeros = 0;
      for (int w = wlo; w < whi; ++w) zeros += win[w] == 0;
      int ztotal;
      int zrank = block_exclusive_scan<NT, BAR>(zeros, scan, &ztotal);
      int keep = 0;
      for (int w = wlo; w < whi; ++w) {
        if (win[w] == 0) { if (zrank < need) win[w] = 2; ++zrank; }
        keep += win[w] != 0;
      }
      int ktotal;
      int pos = block_exclusive_scan<NT, BAR>(keep, scan, &ktotal);
      for (int w = wlo; w < whi; ++w) {
        if (win[w] != 0) mid_b[pos++] = lo + w;
      }
      // chosen tokens beyond the window follow all holes
      for (int i = cw + tid; i < take; i += NT) mid_b[ktotal + (i - cw)] = mid_a[i];
      group_sync<NT, BAR>();
      count = ktotal + (take - cw);
      mid = mid_b;
    }
    int below = 0;
    for (int i = tid; i < min(count, g.sink); i += NT) below += mid[i] < g.sink;
    int d0;
    block_exclusive_scan<NT, BAR>(below, scan, &d0);
    *count_out = count - d0;
    return mid + d0;
  };

  if (NUMERIC && rg.numeric) {
    // ---- numeric near-token quota: far region, then near region, concatenated ----------------
    int total_m = 0;
    if (sm.sc2 != nullptr && sm.fin != nullptr) {
#pragma unroll 1
      for (int region = 0; region < 2; ++region) {
        const int lo = region == 0 ? rg.fq_lo : rg.nq_lo, hi = region == 0 ? rg.fq_hi : rg.nq_hi;
        const int q = region == 0 ? rg.fq : rg.nq;
        if (q <= 0) continue;
        for (int i = tid; i < nitems; i += NT) {
          const int tok = pages[i >> pl2] * g.page + (i & pmask);
          sm.sc2[i] = (tok >= lo && tok < hi) ? sc[i] : (uint16_t)0;
        }
        group_sync<NT, BAR>();
        const int take = block_bisect_topk<NT, BAR, 0, 4, false>(sm.sc2, nitems, min(q, K2), slots_sel, wtot);
        int count_m;
        const int* mid = finish_region(take, lo, q, &count_m);
        for (int i = tid; i < count_m; i += NT) sm.fin[total_m + i] = mid[i];
        total_m += count_m;
        group_sync<NT, BAR>();
      }
    }
    if (trigger) pdl_launch_dependents();
    if (S.middle != nullptr) {
      for (int i = tid; i < total_m; i += NT) S.middle[(size_t)row * K2 + i] = sm.fin[i];
      if (tid == 0) S.middle_counts[row] = total_m;
    }
    write_union(sm.fin, total_m);
    return;
  }

  const int quota = rg.quota;
  // two instantiations: rows of at most 9 NT slots (one chunk and one single score per thread: the
  // 2 080 slots of the default budgets) run a much shorter instruction stream, and executed once,
  // cold, a selection costs about as much in instruction fetch as in arithmetic
  const int take = nitems <= 9 * NT
                       ? block_bisect_topk<NT, BAR, 0, 1, HIST>(sc, nitems, min(quota, K2), slots_sel, wtot, sm.hist)
                       : block_bisect_topk<NT, BAR, 0, 4, HIST>(sc, nitems, min(quota, K2), slots_sel, wtot, sm.hist);
  if (trigger) pdl_launch_dependents();
  if (take == quota) {
    // Common case: the quota is filled by scored candidates (all of them >= sink, no holes).
    // The survivors' physical pages came with the page list, so only the sink and window ids
    // need a block-table lookup: sink ++ middle ++ window, one pass.
    const int cap = g.max_blocks * g.page;
    const int sk_all = min(length, g.sink);
    const int count_s = min(length, g.sink + g.swa) - sk_all;
    const int s_lo = max(max(length - g.swa, 0), sk_all);
    const int s_hi = min(length - g.swa + count_s, cap);
    const int sk = S.middle_only ? 0 : sk_all;                     // middle only: no sink, no window
    const int n_s = S.middle_only ? 0 : max(s_hi - s_lo, 0);
    const int total = sk + take + n_s;
    const int n_out = min(total, g.max_visible);
    int32_t* gout = S.gather + ((size_t)b * g.num_kv_heads + kv) * g.max_visible;
#pragma unroll 1
    for (int i = tid; i < n_out; i += NT) {
      int slot;
      if (i >= sk && i < sk + take) {
        const int sl = slots_sel[i - sk];
        const int ph = physs[(sl >> pl2)];                 // -1: the page lives on another GPU (sequence sharding)
        slot = ph >= 0 ? ph * g.page + (sl & pmask) : -1;
        if (S.middle != nullptr) S.middle[(size_t)row * K2 + (i - sk)] = pages[(sl >> pl2)] * g.page + (sl & pmask);
      } else {
        const int id = i < sk ? i : s_lo + (i - sk - take);
        const int lp = (id >> pl2);
        int ph = lp < g.max_blocks ? table[lp] : -1;
        if (ph < 0 || ph >= g.num_pages) {
          if (rg.shard_count > 1) {
            ph = -1;                                         // another GPU's page: skipped by the attention
          } else {
            if (status) atomicOr(status, LODA_STATUS_BAD_PAGE);
            ph = g.num_pages - 1;
          }
        }
        slot = ph >= 0 ? ph * g.page + (id & pmask) : -1;
      }
      gout[i] = slot;
      if (sm.list) sm.list[i] = slot;
    }
    if (tid == 0) {
      if (sm.list_n) *sm.list_n = n_out;
      if (S.middle != nullptr) S.middle_counts[row] = take;
      S.visible_lens[(size_t)b * g.num_kv_heads + kv] = n_out;
      if (total > g.max_visible && status) atomicOr(status, LODA_STATUS_TRUNCATED);
      if (ticket) *ticket = 0;
    }
    return;
  }
  int count_m;
  const int* mid = finish_region(take, rg.lower, quota, &count_m);
  if (S.middle != nullptr) {
    for (int i = tid; i < count_m; i += NT) S.middle[(size_t)row * K2 + i] = mid[i];
    if (tid == 0) S.middle_counts[row] = count_m;
  }
  // ---- union with sink and window ids (nfa_layer_batch_selector.py:1348-1437) --
  write_union(mid, count_m);
}

}  // namespace loda
