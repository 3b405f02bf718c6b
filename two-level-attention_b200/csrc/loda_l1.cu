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

constexpr int L1_TP = 256;                         // threads per CTA = pages per tile

template <int DSUB>
struct L1Shape {
  static constexpr int NSTAGE = DSUB >= 64 ? 2 : 3;          // tiles in flight per CTA
  static constexpr size_t STAGES_BYTES = (size_t)NSTAGE * L1Tile<DSUB, L1_TP>::STAGE;
  static constexpr size_t ROWS_BYTES = STAGES_BYTES > L1_TAIL_BYTES ? STAGES_BYTES : L1_TAIL_BYTES;
};

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
  __syncthreads();                                       // the barriers are initialised
  // the first NSTAGE tiles are requested at once (issued first: the longest latency)
  if (tid < 32) {
#pragma unroll
    for (int it = 0; it < NSTAGE; ++it) {
      const int p0 = (split + it * nsplit) * P;
      if (it < tiles_per_cta && p0 < page_end)
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
    if (p0 >= page_end) break;
    const int st = it % NSTAGE;
    if (!mbar_wait(bars + st, (uint32_t)(it / NSTAGE) & 1u)) timed_out = true;
    if (it == 0) { LODA_PHASE(l1, cta_id, 3); }
    // one page per thread
    const uint32_t ord = l1_page_score<DSUB, P, GENERIC>(g, rg, p0, page_end, rows + (size_t)st * T::STAGE, qhat, qmm, G,
                                                          qraw);
    row_scores[p0 + tid] = (uint16_t)ord;     // the selecting CTA reads pages below page_end (rounded up to 8)
    __syncthreads();                          // every thread has read the stage: refill it
    if (tid < 32) {
      const int nxt = it + NSTAGE, pn = (split + nxt * nsplit) * P;
      if (nxt < tiles_per_cta && pn < page_end)
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
#if LODA_PDL_TRIGGER == 3
  pdl_launch_dependents();
#endif
  LODA_PHASE(l1, cta_id, 6);
  const int np = l1_select_pages<P>(g, rg, out, row, scf, scn, n_far, far_lo, n_near, near_lo, near_lo8, near_hi, kept,
                                    keys, wtot, sh, LODA_PDL_TRIGGER == 1);
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
  LODA_PHASE(l1, cta_id, 9);
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

template <int DS, bool GENERIC>
static cudaError_t launch_l1_p(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                               float scale, const loda_selection& out, const SelectWorkspace& ws,
                               const AppendArgs& ap, int phase, cudaStream_t st) {
  constexpr int P = L1_TP;
  const int rows = B.batch * g.num_kv_heads;
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
