// Fused L1 kernel: stream page metadata, score every page of the far pool with
// the min/max upper bound and every page of the near pool with the page mean,
// and keep the exact top-k pages of each pool (ties toward the lower page id).
//
// Restates _nfa_l1_scores_kernel (nfa_layer_batch_selector.py:174-354) and the
// packed-key top-k (nfa_layer_batch_selector.py:1473-1532, 1765-1793).
//
// Work split: grid = (ceil(max_blocks / P) [+1], batch * Hkv).  CTA (s, row) owns
// the P consecutive logical pages [s P, s P + P) of one (request, kv head) row:
// it stages their metadata (one contiguous run in HBM) into shared memory with
// 16-byte cp.async copies, scores one page per thread and writes the 16-bit
// ordered score of every page to the row's score array.  The last CTA of a row
// to finish (atomic ticket, no spinning) reads the row's scores back (L2-cache
// resident, 2 bytes per page), selects each pool's top-k with two radix passes
// and a tie-resolving scan in page order, and hands the ascending page list
// (bypass pages included) with its physical page ids to the L2 launch.  An
// optional extra CTA per row carries the decode append.
//
// Canonical arithmetic (must match the CPU oracle bit for bit): a length-d' dot
// is split into chunks of 8 dims summed left to right from 0.0f, chunk sums are
// combined by a balanced pairwise tree; bound = tree(min chunks) + tree(max
// chunks); per-head scores are rounded to bf16, summed over the GQA group in
// head order, divided by G and rounded to bf16.  bf16 x bf16 products are exact
// in fp32, so fmaf equals a separate multiply and add here.
#include "loda_append.cuh"
#include "loda_select.cuh"

namespace loda {

LODA_PHASE_STORAGE(l1)
LODA_SUB_READER(l1)

constexpr int L1_TP = 256;                         // threads per CTA = pages per tile

template <int DSUB>
struct L1Shape {
  static constexpr int NSTAGE = DSUB >= 64 ? 2 : 3;          // tiles in flight per CTA
  static constexpr size_t STAGES_BYTES = (size_t)NSTAGE * L1Tile<DSUB, L1_TP>::STAGE;
  static constexpr size_t ROWS_BYTES = STAGES_BYTES > L1_TAIL_BYTES ? STAGES_BYTES : L1_TAIL_BYTES;
};

// The selecting CTA's work on one row once all its page scores are in the workspace: the scores are
// copied into two rows of shared memory, one per pool, each holding 0 outside its pool (`rows`: the
// consumed tile stages), the pages are selected, and the ascending page list with its physical
// pages is handed to the level-2 launch.  All P threads of the CTA.
template <int DSUB, int P, bool GENERIC>
__device__ __forceinline__ void l1_finish_row(const loda_geometry& g, const loda_layer& L, const Regions& rg,
                                              const loda_selection& out, const SelectWorkspace& ws, int row, int req,
                                              unsigned char* rows, int* kept, uint32_t* keys, int* wtot, int* sh,
                                              int cta_id, bool trigger) {
  const int tid = threadIdx.x;
  const uint16_t* row_scores = ws.l1_scores + (size_t)row * ws.score_stride;
  // the staging rows are consumed: the row's scores are copied into two rows of
  // shared memory, one per pool, each holding 0 outside its pool
  const int near_hi = min(min(rg.swa_lo_blk, rg.kt_eff), g.max_blocks);
  const int far_lo = rg.far_lo, far_hi = max(rg.far_hi, rg.far_lo);
  const int near_lo = rg.near_blks, near_lo8 = near_lo & ~7;
  const int n_far = far_hi;                                                   // far row: pages [0, far_hi)
  static_assert(2 * P >= L1_NEAR_CAP, "the near row is ranked with at most two scores per thread");
  const int n_near = near_hi > near_lo ? min(near_hi - near_lo8, L1_NEAR_CAP) : 0;   // near row: pages [near_lo8, ...)
  uint16_t* scf = (uint16_t*)rows;                       // up to 40 KB
  uint16_t* scn = (uint16_t*)(rows + 40 * 1024);         // L1_NEAR_CAP scores
  {
    // all the loads of a batch are issued before the first is used (one round trip, not one per load)
    const uint4* src = (const uint4*)row_scores;         // 8 scores per load; unscored pages hold 0
    // sequence sharding: the rows of all GPUs, ORed while loading
    auto ldrow = [&](int c) {
      if (ws.gathered == nullptr) return __ldcg(src + c);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      for (int s = 0; s < ws.n_gathered; ++s) {
        const uint4 u = __ldcg((const uint4*)(ws.gathered + s * ws.gathered_stride + (size_t)row * ws.score_stride) + c);
        v.x |= u.x; v.y |= u.y; v.z |= u.z; v.w |= u.w;
      }
      return v;
    };
    const int nc_far = (n_far + 7) / 8, nc_near = (n_near + 7) / 8;          // nc_near <= L1_NEAR_CAP / 8 <= P
    uint4 nreg = make_uint4(0u, 0u, 0u, 0u);
    if (tid < nc_near) nreg = ldrow(near_lo8 / 8 + tid);
    for (int c0 = 0; c0 < nc_far; c0 += 4 * P) {
      uint4 f[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = c0 + k * P + tid;
        f[k] = c < nc_far ? ldrow(c) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = c0 + k * P + tid;
        if (c < nc_far) {
          uint32_t v[8];
          unpack_u16x8(f[k], v);
#pragma unroll
          for (int j = 0; j < 8; ++j) { const int i = c * 8 + j; v[j] = (i >= far_lo && i < far_hi) ? v[j] : 0u; }
          ((uint4*)scf)[c] = make_uint4(v[0] | v[1] << 16, v[2] | v[3] << 16, v[4] | v[5] << 16, v[6] | v[7] << 16);
        }
      }
    }
    if (tid < nc_near) {
      uint32_t v[8];
      unpack_u16x8(nreg, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) { const int i = near_lo8 + tid * 8 + j; v[j] = (i >= near_lo && i < near_hi) ? v[j] : 0u; }
      ((uint4*)scn)[tid] = make_uint4(v[0] | v[1] << 16, v[2] | v[3] << 16, v[4] | v[5] << 16, v[6] | v[7] << 16);
    }
  }
  __syncthreads();
  LODA_PHASE(l1, cta_id, 6);
  const int np = l1_select_pages<P>(g, rg, out, row, scf, scn, n_far, far_lo, n_near, near_lo, near_lo8, near_hi, kept,
                                    keys, wtot, sh, trigger);
  LODA_PHASE(l1, cta_id, 8);
  // hand the ascending page list and its physical pages to the L2 launch
  const int np_max = g.k_far + g.k_near + 2;
  const int32_t* table = L.block_table + (size_t)req * g.max_blocks;
  for (int i = tid; i < np; i += P) {
    const int pg = kept[i];
    int ph = (pg >= 0 && pg < g.max_blocks) ? table[pg] : -1;
    if (ph < 0 || ph >= g.num_pages) ph = -1;
    ws.pages[(size_t)row * np_max + i] = pg;
    ws.phys[(size_t)row * np_max + i] = ph;
  }
  if (tid == 0) {
    ws.np[row] = np;
    ws.l1_ticket[row] = 0;
  }
}

template <int DSUB, int P, bool GENERIC>
__global__ void __launch_bounds__(P, 2) l1_kernel(loda_geometry g, loda_layer L, loda_batch B,
                                                   const bf16* __restrict__ q, float scale,
                                                   loda_selection out, SelectWorkspace ws, int nsplit,
                                                   int tiles_per_cta, AppendArgs ap, int phase) {
  static_assert(P == L1_TP, "one tile shape");
  using T = L1Tile<DSUB, P>;
  constexpr int NSTAGE = L1Shape<DSUB>::NSTAGE;
  constexpr size_t ROWS_BYTES = L1Shape<DSUB>::ROWS_BYTES;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* rows = smem;                                    // tile stages, later scores of the row
  uint64_t* bars = (uint64_t*)(smem + ROWS_BYTES);               // one mbarrier per stage
  float* qhat = (float*)(smem + ROWS_BYTES + 64);                // [G, DSUB] x3 (x4 GENERIC)
  const int G = g.num_q_heads / g.num_kv_heads;
  float* qmm = qhat + G * DSUB;                                  // [G, DSUB, 2]: (min(q, 0), max(q, 0)) interleaved
  float* qraw = qmm + 2 * G * DSUB;                              // GENERIC: the unrounded scaled query (avg_top2)
  constexpr int NQ = GENERIC ? 4 : 3;
  int* kept = (int*)(qhat + NQ * G * DSUB);                      // k_far + k_near + 2
  // (an offset, not pointer arithmetic through an integer: the compiler must keep seeing shared memory)
  const size_t keys_off = (ROWS_BYTES + 64 + (size_t)NQ * G * DSUB * 4 + (size_t)(g.k_far + g.k_near + 2) * 4 + 15) & ~(size_t)15;
  uint32_t* keys = (uint32_t*)(smem + keys_off);                 // 2 P + 8
  int* wtot = (int*)(keys + 2 * P + 8);                          // 8 x 32
  int* sh = wtot + 256;                                          // 8

  const int tid = threadIdx.x;
  const int split = blockIdx.x, row = blockIdx.y;
  const int b = row / g.num_kv_heads, kv = row % g.num_kv_heads;
  const int cta_id = blockIdx.y * gridDim.x + blockIdx.x;
  LODA_PHASE(l1, cta_id, 0);
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) mbar_init(bars + s, 1);
    mbar_init_fence();
  }
  pdl_wait();
#if LODA_PDL_TRIGGER == 0
  pdl_launch_dependents();
#endif
  LODA_PHASE(l1, cta_id, 1);
  if (split == nsplit) {
    // extra CTA of the row: the decode append.  It touches only the newest token
    // and its page, which lie in the sliding window and are read by neither L1
    // nor L2 of this step; the attention kernel runs after this launch completes.
    if (tid < 32) append_row<DSUB>(g, L, B, ap.k_new, ap.v_new, ap.slots, ap.status, b, kv, tid);
    return;
  }
  // this thread's first query element is requested before anything that depends on the
  // request's length, so that the two global round trips overlap
  const int nq = G * DSUB;
  float q_first = 0.0f;
  if (tid < nq)
    q_first = __bfloat162float(q[((size_t)b * g.num_q_heads + kv * G + tid / DSUB) * g.head_dim + sub_dim(g, tid % DSUB)]);
  int length = B.lengths[b];
  const int req = checked_request(g, B.active_req_ids[b], B.valid_req_ids[b], &length, ap.status);
  bool skip_far, skip_near;
  load_skip_flags(L, req, &skip_far, &skip_near);
  const Regions rg = make_regions(g, length, skip_far, skip_near);
  // this CTA's tiles of P pages: split, split + nsplit, ... (interleaved, so that the tiles a
  // short request really has are spread over the CTAs of its row); tiles past the request's
  // last page are neither read nor written, and a CTA without tiles only takes its ticket
  const size_t rowi = (size_t)req * g.num_kv_heads + kv;
  const unsigned char* mm_row = (const unsigned char*)L.page_mm + rowi * stat_row_bytes(g.max_blocks, T::CPR);
  const unsigned char* sum_row = (const unsigned char*)L.page_sum + rowi * stat_row_bytes(g.max_blocks, T::NC);
  uint16_t* row_scores = ws.l1_scores + (size_t)row * ws.score_stride;
  const int page_end = min(rg.kt_eff, g.max_blocks);
  const int tile_end = min(page_end, pools_end(rg));     // tiles behind the pools are skipped
  __syncthreads();                                       // the barriers are initialised
  // the first NSTAGE tiles are requested at once (issued first: the longest latency)
  if (tid < 32) {
#pragma unroll
    for (int it = 0; it < NSTAGE; ++it) {
      const int p0 = (split + it * nsplit) * P;
      if (it < tiles_per_cta && p0 < tile_end)
        l1_issue_tile<DSUB, P, GENERIC>(g, rg, p0, page_end, rows + (size_t)it * T::STAGE, bars + it, mm_row, sum_row);
    }
  }
  // scaled, bf16-rounded query on the subspace (nfa_layer_batch_selector.py:943-963)
  for (int i = tid; i < nq; i += P) {
    const int j = i / DSUB, d = i % DSUB;
    const float qv = i == tid ? q_first
                              : __bfloat162float(q[((size_t)b * g.num_q_heads + kv * G + j) * g.head_dim + sub_dim(g, d)]);
    const float qh = bf16r(__fmul_rn(qv, scale));
    qhat[i] = qh;
    *(float2*)(qmm + 2 * i) = make_float2(fminf(qh, 0.0f), fmaxf(qh, 0.0f));
    if (GENERIC) qraw[i] = __fmul_rn(qv, scale);
  }
  __syncthreads();
  LODA_PHASE(l1, cta_id, 2);
  bool timed_out = false;
#pragma unroll 1
  for (int it = 0; it < tiles_per_cta; ++it) {
    const int p0 = (split + it * nsplit) * P;
    if (p0 >= tile_end) break;
    const int st = it % NSTAGE;
    if (!mbar_wait(bars + st, (uint32_t)(it / NSTAGE) & 1u)) timed_out = true;
    if (it == 0) { LODA_PHASE(l1, cta_id, 3); }
    // one page per thread
    const uint32_t ord = l1_page_score<DSUB, P, GENERIC>(g, rg, p0, page_end, rows + (size_t)st * T::STAGE, qhat, qmm, G,
                                                          qraw);
    row_scores[p0 + tid] = (uint16_t)ord;     // the selecting CTA masks what lies outside the pools
    __syncthreads();                          // every thread has read the stage: refill it
    if (tid < 32) {
      const int nxt = it + NSTAGE, pn = (split + nxt * nsplit) * P;
      if (nxt < tiles_per_cta && pn < tile_end)
        l1_issue_tile<DSUB, P, GENERIC>(g, rg, pn, page_end, rows + (size_t)st * T::STAGE, bars + st, mm_row, sum_row);
    }
  }
  if (timed_out && tid == 0 && ap.status) atomicOr(ap.status, LODA_STATUS_TIMEOUT);
  LODA_PHASE(l1, cta_id, 4);

  // last CTA of the row selects.  phase 1 = scores only (the caller combines the score rows of
  // several GPUs before the selection), phase 2 = selection only (one CTA per row, no tiles)
  if (phase == 1) return;
  if (phase == 0) {
    __threadfence();
    __syncthreads();
    if (tid == 0) sh[0] = (atomicAdd(ws.l1_ticket + row, 1) == nsplit - 1);
    __syncthreads();
    LODA_PHASE(l1, cta_id, 5);
    if (!sh[0]) return;
    __threadfence();
  }
  l1_finish_row<DSUB, P, GENERIC>(g, L, rg, out, ws, row, req, rows, kept, keys, wtot, sh, cta_id, LODA_PDL_TRIGGER == 1);
  LODA_PHASE(l1, cta_id, 9);
}

// ---------------------------------------------------------------------------
// Level 1 for large batches: a grid that fills the GPU once (two CTAs per SM) and stays.  Every CTA
// first counts the tiles of P pages that each row of the batch really has (its pools' extent, from the
// row's length and skip flags) and forms their prefix sums, so all CTAs agree on one flat sequence of
// (row, tile) pairs, row by row; CTA c takes the c-th of gridDim.x equal slices of that sequence — the
// same number of tiles (one more or less) for every CTA, whatever the rows' lengths.  A slice touches a
// few consecutive rows: their metadata, region geometry and scaled queries are staged once (eight rows
// at a time).  Then every WARP runs a pipeline of its own over the slice: a warp scores the 32 pages of
// one group of each tile, and a group is one contiguous block of the statistics, so the warp fetches
// its group of the tiles ahead itself (one bulk copy of a group's min/max rows, or of its sum rows, on
// the warp's own mbarrier per stage) and never waits for another warp: no barrier of the CTA and no
// shared stage between two tiles, across rows as within them.  (The one group of a row that holds pages
// of both pools stages its min/max rows and reads its sums from global memory.)  A warp that has
// finished its tiles of a row publishes its scores and adds their number to the row's ticket.  When
// its warps are done the CTA turns to selection: it claims the next row from a queue (rows in order,
// the order in which they complete), waits — bounded — until the row's ticket shows all warps of all
// its tiles, and selects as the last CTA of a row does above.  Every CTA of the grid is resident (the
// host sizes the grid by the occupancy the runtime reports), so a CTA that waits for a row waits for
// CTAs that are running.
// ---------------------------------------------------------------------------
// (build-time knobs; measured on the 32-request batch with the earlier item scheme: 2 stages 48.7 us, 3 stages 48.8)
#ifndef LODA_L1S_STAGES
#define LODA_L1S_STAGES 2
#endif
constexpr int L1S_BATCH = 8;            // rows whose queries are staged at a time
constexpr int L1S_STAGES = LODA_L1S_STAGES;             // groups in flight per warp
constexpr int L1S_MAX_ROWS = 512;       // rows of a batch (the tile counts' prefix sums stay in shared memory)
constexpr int L1S_POLL_LIMIT = 1 << 18;

template <int DSUB>
struct L1Stream {
  using T = L1Tile<DSUB, L1_TP>;
  static constexpr size_t STAGES_BYTES = (size_t)L1S_STAGES * (L1_TP / 32) * T::SLOT;     // [stage][warp] slots
  static constexpr size_t ROWS_BYTES = STAGES_BYTES > L1_TAIL_BYTES ? STAGES_BYTES : L1_TAIL_BYTES;
  static constexpr size_t FIXED_BYTES = ROWS_BYTES + (L1_TP / 32) * L1S_STAGES * 8 + (L1S_MAX_ROWS + 4) * 4 +
                                        L1S_MAX_ROWS * 8 + L1S_BATCH * (16 + sizeof(Regions));
};

template <int DSUB, bool GENERIC>
__global__ void __launch_bounds__(L1_TP, 2) l1_stream_kernel(loda_geometry g, loda_layer L, loda_batch B,
                                                             const bf16* __restrict__ q, float scale,
                                                             loda_selection out, SelectWorkspace ws, AppendArgs ap,
                                                             int n_rows) {
  constexpr int P = L1_TP, NWARP = P / 32, NSTAGE = L1S_STAGES;
  using T = L1Tile<DSUB, P>;
  constexpr size_t ROWS_BYTES = L1Stream<DSUB>::ROWS_BYTES;
  constexpr int NQ = GENERIC ? 4 : 3;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* rows = smem;                                    // [NSTAGE][NWARP] group slots, later the row's scores
  uint64_t* full = (uint64_t*)(smem + ROWS_BYTES);               // [NWARP][NSTAGE]
  int* prefix = (int*)(full + NWARP * NSTAGE);                   // [n_rows + 1] tiles before each row
  int2* rowmeta = (int2*)(prefix + L1S_MAX_ROWS + 4);            // [n_rows] (length, request slot | skip bits << 28)
  int4* desc = (int4*)(rowmeta + L1S_MAX_ROWS);                  // [BATCH] (length, request slot, first tile, end tile)
  Regions* regs = (Regions*)(desc + L1S_BATCH);                  // [BATCH] the rows' region geometry
  const int G = g.num_q_heads / g.num_kv_heads;
  const int nq = G * DSUB;
  float* qall = (float*)(regs + L1S_BATCH);                      // [BATCH][NQ * G * DSUB]
  int* kept = (int*)(qall + (size_t)L1S_BATCH * NQ * nq);        // k_far + k_near + 2
  const size_t keys_off = (L1Stream<DSUB>::FIXED_BYTES + (size_t)L1S_BATCH * NQ * nq * 4 +
                           (size_t)(g.k_far + g.k_near + 2) * 4 + 15) & ~(size_t)15;
  uint32_t* keys = (uint32_t*)(smem + keys_off);                 // 2 P + 8
  int* wtot = (int*)(keys + 2 * P + 8);                          // 8 x 32
  int* sh = wtot + 256;                                          // 8

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cta = blockIdx.x, ncta = gridDim.x;
  const int cta_id = cta;
  LODA_PHASE(l1, cta_id, 0);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) mbar_init(full + warp * NSTAGE + s, 1);
    mbar_init_fence();
  }
  pdl_wait();
  LODA_PHASE(l1, cta_id, 1);
  // the decode append of the rows cta, cta + ncta, ...: the newest token and its page lie in the
  // sliding window and are read by neither level of this step
  if (ap.enabled && warp == NWARP - 1) {
    for (int r = cta; r < n_rows; r += ncta)
      append_row<DSUB>(g, L, B, ap.k_new, ap.v_new, ap.slots, ap.status, r / g.num_kv_heads, r % g.num_kv_heads, lane);
  }
  // metadata of one row, checked like checked_request (every CTA reads every row: only CTA 0 reports)
  auto row_meta = [&](int row, int* length, int* req, bool* skip_far, bool* skip_near) {
    const int b = row / g.num_kv_heads;
    *length = B.lengths[b];
    const long long act = B.active_req_ids[b], val = B.valid_req_ids[b];
    *req = 0;
    if (act < 0) { *length = 0; *req = (val >= 0 && val < g.max_requests) ? (int)val : 0; }
    else if (val < 0 || val >= g.max_requests) { *length = 0; if (ap.status && cta == 0) atomicOr(ap.status, LODA_STATUS_BAD_REQ); }
    else *req = (int)val;
    load_skip_flags(L, *req, skip_far, skip_near);
  };
  auto row_tiles = [&](const Regions& rg) {
    const int tile_end = min(min(rg.kt_eff, g.max_blocks), pools_end(rg));
    return (tile_end + P - 1) / P;
  };
  // tiles of every row, prefix sums (the same in every CTA)
  {
    int base = 0;
    for (int r0 = 0; r0 < n_rows; r0 += P) {
      const int row = r0 + tid;
      int nt = 0;
      if (row < n_rows) {
        int length, req;
        bool sf, sn;
        row_meta(row, &length, &req, &sf, &sn);
        nt = row_tiles(make_regions(g, length, sf, sn));
        rowmeta[row] = make_int2(length, req | (sf ? 1 << 28 : 0) | (sn ? 1 << 29 : 0));     // (max_requests < 2^28)
      }
      int total;
      const int before = block_exclusive_scan<P>(nt, wtot, &total);
      if (row < n_rows) prefix[row] = base + before;
      base += total;
      __syncthreads();                                   // the scan's scratch is reused by the next round
    }
    if (tid == 0) prefix[n_rows] = base;
  }
  __syncthreads();                                       // barriers and prefix sums are ready
  const int total_tiles = prefix[n_rows];
  const int lo = (int)((long long)cta * total_tiles / ncta), hi = (int)((long long)(cta + 1) * total_tiles / ncta);
  LODA_PHASE(l1, cta_id, 2);

  // ---- this CTA's slice [lo, hi) of the tile sequence, eight rows at a time ---------------------------
  if (lo < hi) {
    // the row that holds tile lo: the last row whose prefix is <= lo among rows that have tiles
    int rb = 0;
    {
      int a = 0, b2 = n_rows;                            // prefix[a] <= lo < prefix[b2]
      while (b2 - a > 1) {
        const int m = (a + b2) >> 1;
        if (prefix[m] <= lo) a = m; else b2 = m;
      }
      rb = a;
    }
    uint64_t* wfull = full + warp * NSTAGE;
    auto slot_of = [&](int st) { return rows + ((size_t)st * NWARP + warp) * T::SLOT; };
    int pseq = 0, cseq = 0;                              // places in the warp's stream (kept across the row batches)
    bool dead = false;                                   // a wait gave up: no further waiting
#pragma unroll 1
    while (rb < n_rows && prefix[rb] < hi) {
      int nr = 0;
      while (nr < L1S_BATCH && rb + nr < n_rows && prefix[rb + nr] < hi) ++nr;
      __syncthreads();                                   // the warps are done with the rows staged before
      if (tid < nr) {
        const int row = rb + tid;
        const int2 m = rowmeta[row];
        regs[tid] = make_regions(g, m.x, (m.y >> 28 & 1) != 0, (m.y >> 29 & 1) != 0);
        const int t0 = max(lo, prefix[row]) - prefix[row], t1 = min(hi, prefix[row + 1]) - prefix[row];
        desc[tid] = make_int4(m.x, m.y & 0x0FFFFFFF, t0, max(t1, t0));
      }
      // scaled, bf16-rounded queries of the rows on the subspace (nfa_layer_batch_selector.py:943-963)
      for (int i = tid; i < nr * nq; i += P) {
        const int k = i / nq, e = i % nq, j = e / DSUB, dd = e % DSUB;
        const int row = rb + k, b = row / g.num_kv_heads, kv = row % g.num_kv_heads;
        const float qv = __bfloat162float(q[((size_t)b * g.num_q_heads + kv * G + j) * g.head_dim + sub_dim(g, dd)]);
        const float qh = bf16r(__fmul_rn(qv, scale));
        float* qhat = qall + (size_t)k * NQ * nq;
        qhat[e] = qh;
        *(float2*)(qhat + nq + 2 * e) = make_float2(fminf(qh, 0.0f), fmaxf(qh, 0.0f));
        if (GENERIC) qhat[3 * nq + e] = __fmul_rn(qv, scale);
      }
      __syncthreads();
      // every warp: its group of every tile of the staged rows
      int pk = 0, pit = 0;                               // producer side: row of the batch, tile of its range
      auto issue_next = [&]() {
        while (pk < nr && desc[pk].z + pit >= desc[pk].w) { ++pk; pit = 0; }
        if (pk >= nr) return;
        const int4 d = desc[pk];
        const Regions& rg = regs[pk];
        const int row = rb + pk, kv = row % g.num_kv_heads;
        const int g0 = (d.z + pit) * P + warp * STAT_GROUP;          // first page of the warp's group
        bool nm, ns;
        l1_group_needs<GENERIC>(g, rg, g0, min(rg.kt_eff, g.max_blocks), &nm, &ns);
        if (lane == 0) {
          const int st = pseq % NSTAGE;
          const size_t rowi = (size_t)d.y * g.num_kv_heads + kv;
          const size_t gidx = (size_t)(g0 / STAT_GROUP);
          const uint32_t bytes = nm ? (uint32_t)T::SLOT : ns ? (uint32_t)T::SUMG : 0u;
          mbar_arrive_expect_tx(wfull + st, bytes);       // no bytes: the phase completes at once
          if (nm)
            bulk_copy_g2s(slot_of(st), (const unsigned char*)L.page_mm + rowi * stat_row_bytes(g.max_blocks, T::CPR) + gidx * T::SLOT,
                          T::SLOT, wfull + st);
          else if (ns)
            bulk_copy_g2s(slot_of(st), (const unsigned char*)L.page_sum + rowi * stat_row_bytes(g.max_blocks, T::NC) + gidx * T::SUMG,
                          T::SUMG, wfull + st);
        }
        ++pit;
        ++pseq;
      };
#pragma unroll 1
      for (int s = 0; s < NSTAGE; ++s) issue_next();
#pragma unroll 1
      for (int k = 0; k < nr; ++k) {
        const int4 d = desc[k];
        const int row = rb + k, kv = row % g.num_kv_heads;
        const int nt = d.w - d.z;
        if (nt <= 0) continue;
        const Regions rg = regs[k];
        const int page_end = min(rg.kt_eff, g.max_blocks);
        const float* qhat = qall + (size_t)k * NQ * nq;
        uint16_t* row_scores = ws.l1_scores + (size_t)row * ws.score_stride;
        const size_t rowi = (size_t)d.y * g.num_kv_heads + kv;
        const unsigned char* sum_row = (const unsigned char*)L.page_sum + rowi * stat_row_bytes(g.max_blocks, T::NC);
#pragma unroll 1
        for (int it = 0; it < nt; ++it) {
          const int st = cseq % NSTAGE;
          if (cseq < 10) { LODA_SUB0(32 + 3 * cseq); }
          if (!dead && !mbar_wait(wfull + st, (uint32_t)(cseq / NSTAGE) & 1u)) dead = true;
          if (cseq < 10) { LODA_SUB0(33 + 3 * cseq); }
          const int g0 = (d.z + it) * P + warp * STAT_GROUP;
          bool nm, ns;
          l1_group_needs<GENERIC>(g, rg, g0, page_end, &nm, &ns);
          const unsigned char* slot = slot_of(st) + lane * 16;
          // a group with pages of both pools staged its min/max rows: its sums come from global memory
          const unsigned char* sum_src = nm ? sum_row + (size_t)(g0 / STAT_GROUP) * T::SUMG + lane * 16 : slot;
          const uint32_t ord = l1_page_score_src<DSUB, GENERIC>(g, rg, g0 + lane, slot, sum_src, qhat, qhat + nq, G, qhat + 3 * nq);
          row_scores[g0 + lane] = (uint16_t)ord;         // the selecting CTA masks what lies outside the pools
          __syncwarp();                                  // every lane has read the slot
          if (cseq < 10) { LODA_SUB0(34 + 3 * cseq); }
          ++cseq;
          issue_next();
        }
        // this warp's tiles of the row are done: publish its scores, then count them on the row's ticket (a
        // row is complete at NWARP x its tiles; its selection may start while this CTA still scores)
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(ws.l1_ticket + row, nt);
      }
      rb += nr;
    }
    if (dead && lane == 0 && ap.status) atomicOr(ap.status, LODA_STATUS_TIMEOUT);
  }
  LODA_PHASE(l1, cta_id, 4);
  pdl_launch_dependents();

  // ---- selection: rows from the queue -------------------------------------------------------------
  int* queue = ws.l1_ticket + ws.ticket_rows;            // [0] next row to select, [1] CTAs that have left
#pragma unroll 1
  for (;;) {
    __syncthreads();                                     // sh and the selection buffers of the row before are consumed
    if (tid == 0) {
      const int r = atomicAdd(queue, 1);
      int ok = 1;
      if (r < n_rows) {
        const int want = (prefix[r + 1] - prefix[r]) * NWARP;
        int tries = 0;
        while (*(volatile int*)(ws.l1_ticket + r) < want) {
          if (++tries > L1S_POLL_LIMIT) { ok = 0; break; }
          __nanosleep(64);
        }
      }
      sh[4] = r;
      sh[5] = ok;
    }
    __syncthreads();
    const int r = sh[4];
    if (r >= n_rows) break;
    if (!sh[5]) {                                        // the row never completed: report, leave its outputs alone
      if (tid == 0 && ap.status) atomicOr(ap.status, LODA_STATUS_TIMEOUT);
      continue;
    }
    __threadfence();                                     // the scores of the row's tiles, published before their tickets
    const int2 m = rowmeta[r];
    const int req = m.y & 0x0FFFFFFF;
    const Regions rg = make_regions(g, m.x, (m.y >> 28 & 1) != 0, (m.y >> 29 & 1) != 0);
    LODA_PHASE(l1, cta_id, 5);
    l1_finish_row<DSUB, P, GENERIC>(g, L, rg, out, ws, r, req, rows, kept, keys, wtot, sh, cta_id, false);
    LODA_PHASE(l1, cta_id, 9);
  }
  if (tid == 0 && atomicAdd(queue + 1, 1) == ncta - 1) {   // the last CTA to leave rearms the queue
    queue[0] = 0;
    queue[1] = 0;
  }
}

static bool l1_generic(const loda_geometry& g) { return g.far_method != LODA_FAR_MINMAX || g.near_minmax != 0; }

template <int DS>
static size_t l1_smem_bytes_d(const loda_geometry& g) {
  const int G = g.num_q_heads / g.num_kv_heads;
  return L1Shape<DS>::ROWS_BYTES + 64 + (size_t)(l1_generic(g) ? 4 : 3) * G * DS * 4 +
         (size_t)(g.k_far + g.k_near + 2) * 4 + (size_t)(2 * L1_TP + 8) * 4 + (256 + 8) * 4 + 32;
}

size_t l1_smem_bytes(const loda_geometry& g) {
  return g.sub_dims == 16 ? l1_smem_bytes_d<16>(g) : g.sub_dims == 32 ? l1_smem_bytes_d<32>(g) : l1_smem_bytes_d<64>(g);
}

// scores per row in the workspace: whole tiles
int l1_score_stride(const loda_geometry& g) { return (g.max_blocks + 511) / 512 * 512; }

// CTAs per row: one tile each while the grid is small (batch 1: latency), several interleaved
// tiles per CTA (a pipeline of bulk copies inside the CTA) once rows x tiles exceeds about eight
// CTAs per SM (fewer, longer CTAs lengthen the tail: the last CTAs to start score and then select while
// the GPU drains)
static void l1_split(const loda_geometry& g, int rows, int P, int* ctas_per_row, int* tiles_per_cta) {
  const int ntiles = (g.max_blocks + P - 1) / P;
  const int sms = device_sm_count();
  int tpc = (rows * ntiles + 8 * sms - 1) / (8 * sms);
  tpc = tpc < 1 ? 1 : tpc > ntiles ? ntiles : tpc;
  *tiles_per_cta = tpc;
  *ctas_per_row = (ntiles + tpc - 1) / tpc;
}

template <int DS>
static size_t l1_stream_smem_bytes_d(const loda_geometry& g) {
  const int G = g.num_q_heads / g.num_kv_heads;
  return L1Stream<DS>::FIXED_BYTES + (size_t)L1S_BATCH * (l1_generic(g) ? 4 : 3) * G * DS * 4 +
         (size_t)(g.k_far + g.k_near + 2) * 4 + (size_t)(2 * L1_TP + 8) * 4 + (256 + 8) * 4 + 32;
}

// Grid of the streaming kernel: every CTA resident at once (what the runtime reports for this kernel
// and its shared memory, per device), or 0 when the kernel cannot be used.
template <int DS, bool GENERIC>
static int l1_stream_grid(size_t smem) {
  // per device ordinal, remembered for the shared-memory size it was asked for (the size follows the
  // geometry: another GQA group or page budget may change how many CTAs an SM holds)
  static int per_sm[64] = {};                    // -1 = refused
  static size_t asked[64] = {};
  const int dev = device_ordinal();
  if (dev < 0 || dev >= 64) return 0;
  if (per_sm[dev] == 0 || asked[dev] != smem) {
    int n = 0;
    if (set_kernel_smem(l1_stream_kernel<DS, GENERIC>, smem) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, l1_stream_kernel<DS, GENERIC>, L1_TP, smem) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      n = -1;
    }
    per_sm[dev] = n >= 2 ? 2 : -1;                // one CTA per SM would leave the warps' latencies uncovered
    asked[dev] = smem;
  }
  return per_sm[dev] > 0 ? per_sm[dev] * device_sm_count() : 0;
}

template <int DS, bool GENERIC>
static cudaError_t launch_l1_p(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                               float scale, const loda_selection& out, const SelectWorkspace& ws,
                               const AppendArgs& ap, int phase, cudaStream_t st) {
  constexpr int P = L1_TP;
  const int rows = B.batch * g.num_kv_heads;
  // large batches: the streaming kernel (LODA_B200_L1_PATH=grid keeps the grid of one CTA per item,
  // =stream takes the streaming kernel for small batches too)
  if (phase == 0 && ws.gathered == nullptr) {
    const char* e = getenv("LODA_B200_L1_PATH");
    const bool never = e && strcmp(e, "grid") == 0, always = e && strcmp(e, "stream") == 0;
    const size_t smem = l1_stream_smem_bytes_d<DS>(g);
    const int ntiles = (g.max_blocks + P - 1) / P;
    const int ncta = never ? 0 : l1_stream_grid<DS, GENERIC>(smem);
    // (measured on 131 072-token rows: 32 rows = 1 056 tiles 30.7 us against 33.4 us on the item grid, 16 rows =
    // 528 tiles 25.5 against 20.9: the resident grid pays once a CTA has about three tiles)
    if (ncta > 0 && rows <= L1S_MAX_ROWS && g.max_requests < (1 << 28) && (always || (long long)rows * ntiles >= 3LL * ncta))
      return launch_pdl(l1_stream_kernel<DS, GENERIC>, dim3(ncta), dim3(P), smem, st, g, L, B, (const bf16*)q, scale, out,
                        ws, ap, rows);
  }
  int nsplit, tpc;
  l1_split(g, rows, P, &nsplit, &tpc);
  dim3 grid(nsplit + (ap.enabled ? 1 : 0), rows);
  if (phase == 2) {                 // selection only: one CTA per row and no tiles
    grid = dim3(1, rows);
    tpc = 0;
  }
  const size_t smem = l1_smem_bytes_d<DS>(g);
  cudaError_t e = set_kernel_smem(l1_kernel<DS, P, GENERIC>, smem);
  if (e != cudaSuccess) return e;
  return launch_pdl(l1_kernel<DS, P, GENERIC>, grid, dim3(P), smem, st, g, L, B, (const bf16*)q, scale, out, ws, nsplit, tpc,
                    ap, phase);
}

template <int DS>
static cudaError_t launch_l1_d(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                               float scale, const loda_selection& out, const SelectWorkspace& ws,
                               const AppendArgs& ap, int phase, cudaStream_t st) {
  // other level-1 methods than the defaults read them at run time
  return l1_generic(g) ? launch_l1_p<DS, true>(g, L, B, q, scale, out, ws, ap, phase, st)
                       : launch_l1_p<DS, false>(g, L, B, q, scale, out, ws, ap, phase, st);
}

// phase 0: scores and selection; 1: scores only; 2: selection only (of the scores in the workspace)
cudaError_t launch_l1(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                      float scale, const loda_selection& out, const SelectWorkspace& ws, const AppendArgs& ap,
                      int phase, cudaStream_t st) {
  switch (g.sub_dims) {
    case 16: return launch_l1_d<16>(g, L, B, q, scale, out, ws, ap, phase, st);
    case 32: return launch_l1_d<32>(g, L, B, q, scale, out, ws, ap, phase, st);
    case 64: return launch_l1_d<64>(g, L, B, q, scale, out, ws, ap, phase, st);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace loda
