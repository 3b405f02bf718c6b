// The two selector levels of one decode step in ONE launch, for grids that fit the GPU in a
// single round (batch 1 at long context): a thread-block cluster of 16 CTAs per (request, kv
// head) row keeps everything the two levels exchange in shared memory.
//
//   1. every CTA stages and scores its tiles of 512 pages (as l1_kernel does) and stores the
//      16-bit page scores straight into the row leader's shared memory (DSMEM);
//   2. cluster barrier; the leader (rank 0) selects the far pages, rank 1 selects the near pages
//      (it copies their scores out of the leader's shared memory and stores its result back
//      there; run beside the far selection on the leader's SM it slowed the longer of the two
//      by a fifth), both look up the physical pages; rank 2 performs the decode append of the row;
//   3. cluster barrier; every CTA scores its share of the candidate slots on the packed 4-bit
//      tail keys, reading the page list from the leader's shared memory and storing the 16-bit
//      logits there;
//   4. cluster barrier; the peers exit, the leader's first 256 threads select the quota, fill
//      holes and write the gather list (the routines of l2_kernel on a named barrier).
//
// Against the two-launch chain this removes one launch boundary, the global round trip of the
// page scores and of the candidate logits with their fences and tickets, and the second
// kernel's prologue.  Same device routines, same arithmetic, same results.
// Restates the same reference code as loda_l1.cu and loda_l2.cu
// (nfa_layer_batch_selector.py:174-354, 422-605, 1194-1251, 1336-1437, 1473-1793).
//
// The cluster barriers are hardware barriers (no spinning in this code); every CTA of a
// cluster executes all of them on every path (four, six with the attention phase).
#include <cooperative_groups.h>

#include <cstdlib>
#include <cstring>

#include "loda_append.cuh"
#include "loda_attn.cuh"
#include "loda_select.cuh"

namespace loda {

namespace cg = cooperative_groups;

LODA_PHASE_STORAGE(sel)
LODA_SUB_READER(sel)

constexpr int SF_P = 512;          // threads per CTA = pages per tile
constexpr int SF_CLUSTER_MAX = 16; // CTAs per row: 16, or 8 when the GPU cannot hold a 16-CTA cluster for every row
// (clusters of 12 and 10 were measured too: where 16 do not fit, 10 did, and ran the step slower than 8 —
// 27.0 against 26.6 us per layer-step at 131 072 tokens: every extra CTA lengthens the cluster barriers)
constexpr int SF_NSIZES = 2;
constexpr int SF_CLUSTER_SIZES[SF_NSIZES] = {16, 8};
constexpr int SF_L2_NT = 256;      // threads of the leader that run the level-2 selection

struct FusedLayout {
  size_t rows_bytes, bars, qv, kept, physk, kept2, physk2, keys, wtot, scan, sh, hist2, list, pfm, pfo, scall, total;
};

__host__ __device__ inline FusedLayout fused_layout(const loda_geometry& g, int tiles_per_cta, int cluster_size) {
  const int G = g.num_q_heads / g.num_kv_heads;
  const int np_max = g.k_far + g.k_near + 2;
  FusedLayout f;
  // one tile stage: 16 groups of min/max rows and the spill slot of sums (L1Tile<d', 512>::STAGE)
  const size_t rows = (size_t)(SF_P / STAT_GROUP) * 128 * g.sub_dims + 64 * (size_t)g.sub_dims;
  f.rows_bytes = rows > L1_TAIL_BYTES ? rows : L1_TAIL_BYTES;
  // the attention phase lays a tile of up to 128 tokens (K rows, V rows, slots) and the warps' partial
  // outputs over the staging area: a single buffer must hold that much
  const size_t attend = ((size_t)128 * ((size_t)(g.head_dim + 8) * 2 + (size_t)(g.head_dim_v + 8) * 2 + 4) + 127) & ~(size_t)127;
  if (tiles_per_cta <= 1 && f.rows_bytes < attend && g.head_dim == 128 && g.head_dim_v == 128) f.rows_bytes = attend;
  size_t off = f.rows_bytes * (tiles_per_cta > 1 ? 2 : 1);      // two staging buffers when a CTA has several tiles
  f.bars = off; off += 16;                                             // one mbarrier per staging buffer
  f.qv = off; off += (size_t)(3 * G + 1) * g.sub_dims * 4;             // qhat, qlow, qhigh [G][d'], qf [d']
  f.kept = off; off += (size_t)np_max * 4;
  f.physk = off; off += (size_t)np_max * 4;
  f.kept2 = off; off += (size_t)np_max * 4;                            // the list without its gaps (leader)
  f.physk2 = off; off += (size_t)np_max * 4;
  off = (off + 15) & ~(size_t)15;
  f.keys = off; off += (size_t)(2 * SF_P + 8) * 4;
  f.wtot = off; off += 256 * 4;
  f.scan = off; off += 40 * 4;
  f.sh = off; off += 8 * 4;
  off = (off + 15) & ~(size_t)15;
  f.hist2 = off; off += 2048 * 4;                                      // candidate scores by their top 12 bits
  f.list = off; off += ((size_t)g.max_visible * 4 + 15) & ~(size_t)15;     // the row's gather list, for the attention phase
  // the CTAs' attention partials, collected by the leader: max and sum [cs][2][16], output [cs][G][Dv] (fp32)
  f.pfm = off; off += (size_t)cluster_size * 32 * 4;
  f.pfo = off; off += (size_t)cluster_size * G * g.head_dim_v * 4;
  f.scall = off; off += (size_t)tiles_per_cta * cluster_size * SF_P * 2 + 16;   // every page score of the row
  f.total = off;
  return f;
}

// bytes of the level-2 arrays the leader lays over the staging rows
__host__ __device__ inline size_t fused_l2_bytes(const loda_geometry& g) {
  const size_t np_max = g.k_far + g.k_near + 2;
  return ((np_max * g.page * 2 + 15) & ~(size_t)15) + 2 * (size_t)g.level2_topk * 4 + g.level2_topk + 32;
}

// the attention phase of the launch: query_to_req [batch] (the identity, or < 0 for a row of zeros),
// out [batch, Hq, head_dim_v]
struct FusedAttend {
  const int32_t* query_to_req;
  bf16* out;
  float scale_log2;
};

// tokens of the attention tile a CTA stages at a time: what fits the staging rows, 256 at most
__host__ __device__ inline int fused_attend_tile(const loda_geometry& g, size_t rows_total) {
  const size_t per_token = (size_t)(g.head_dim + 8) * 2 + (size_t)(g.head_dim_v + 8) * 2 + 4;
  const size_t cap = rows_total / per_token;
  return (int)(cap > 256 ? 256 : cap) & ~15;
}

// D: head dimension of the attention phase (keys and values alike), 0 = selection only
template <int DSUB, int D>
__global__ void __launch_bounds__(SF_P) select_fused_kernel(loda_geometry g, loda_layer L, loda_batch B,
                                                            const bf16* __restrict__ q, float scale, loda_selection S,
                                                            uint32_t* status, AppendArgs ap, int tiles_per_cta,
                                                            FusedAttend at) {
  constexpr int P = SF_P;
  using T = L1Tile<DSUB, P>;
  extern __shared__ __align__(128) unsigned char smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int CS = (int)cluster.num_blocks();
  const FusedLayout lay = fused_layout(g, tiles_per_cta, CS);
  const int G = g.num_q_heads / g.num_kv_heads;
  unsigned char* rows = smem;
  uint64_t* bars = (uint64_t*)(smem + lay.bars);
  float* qhat = (float*)(smem + lay.qv);
  float* qmm = qhat + G * DSUB;                      // [G, DSUB, 2]: (min(q, 0), max(q, 0)) interleaved
  float* qf = qmm + 2 * G * DSUB;
  int* kept = (int*)(smem + lay.kept);
  int* physk = (int*)(smem + lay.physk);
  int* kept2 = (int*)(smem + lay.kept2);
  int* physk2 = (int*)(smem + lay.physk2);
  uint32_t* keys = (uint32_t*)(smem + lay.keys);
  int* wtot = (int*)(smem + lay.wtot);
  int* scan = (int*)(smem + lay.scan);
  int* sh = (int*)(smem + lay.sh);
  uint16_t* scall = (uint16_t*)(smem + lay.scall);
  uint32_t* hist2 = (uint32_t*)(smem + lay.hist2);
  int* list = (int*)(smem + lay.list);

  const int tid = threadIdx.x;
  const int rank = (int)cluster.block_rank();        // = blockIdx.x: the cluster spans the grid's x
  const int row = blockIdx.y;
  const int b = row / g.num_kv_heads, kv = row % g.num_kv_heads;
#ifdef LODA_PHASES
  // debug timeline: launches that carry the chained flag record behind the others
  const int cta_id = blockIdx.y * gridDim.x + blockIdx.x + ((S.flags & LODA_SEL_CHAINED) ? gridDim.x * gridDim.y : 0);
#else
  const int cta_id = blockIdx.y * gridDim.x + blockIdx.x;
#endif
  // The leader's copies of what the cluster shares.  The leader itself uses its plain shared
  // addresses: a store through the cluster window into the CTA's own shared memory is a remote
  // store that the CTA's next barrier has to wait for (measured: the leader reached the first
  // cluster barrier 2 000 cycles after its peers).
  const bool own = rank == 0;
  uint16_t* l_scall = own ? scall : cluster.map_shared_rank(scall, 0);
  int* l_kept = own ? kept : cluster.map_shared_rank(kept, 0);
  int* l_physk = own ? physk : cluster.map_shared_rank(physk, 0);
  int* l_sh = own ? sh : cluster.map_shared_rank(sh, 0);
  uint16_t* l_sc2 = (uint16_t*)(own ? rows : cluster.map_shared_rank(rows, 0));     // level-2 scores, over the leader's rows
  uint32_t* l_hist2 = own ? hist2 : cluster.map_shared_rank(hist2, 0);

  LODA_PHASE(sel, cta_id, 0);
  if (tid == 0) {
    mbar_init(bars, 1);
    mbar_init(bars + 1, 1);
    mbar_init_fence();
  }
  if (rank == 0) *(uint4*)(hist2 + 4 * tid) = make_uint4(0, 0, 0, 0);      // 2048 words; counted into after barrier (2)
  // rank 1 collects the near pool's scores in the same place of its own shared memory (it has no
  // histogram): zero outside the pool, so cleared before any peer may store
  if (rank == 1 && tid < (L1_NEAR_CAP + 8) / 2) hist2[tid] = 0;
  cluster.barrier_arrive();   // (0) "this CTA runs": waited for just before the first store into a peer
  // With LODA_SEL_CHAINED the caller guarantees that the launch before this one is a decode step of
  // this library on the same batch metadata, complete before that launch began: the metadata and
  // the page statistics of the two pools are then fetched before the dependency wait, while the
  // previous launch drains (it writes neither: the only statistics a step writes are those of the
  // newest token's page, which lies in the sliding window, outside both pools).  Without the flag
  // nothing is read before the wait.  The query and everything else are always read after it.
  const bool early = (S.flags & LODA_SEL_CHAINED) != 0;
  LODA_SUB0(48);
  if (!early) pdl_wait();
  LODA_SUB0(49);
  const int nq = G * DSUB;
  int length = B.lengths[b];
  const int req = checked_request(g, B.active_req_ids[b], B.valid_req_ids[b], &length, status);
  bool skip_far, skip_near;
  load_skip_flags(L, req, &skip_far, &skip_near);
  Regions rg = make_regions(g, length, skip_far, skip_near);
  rg.shard_rank = 0;          // this launch never serves a sequence-sharded geometry: the ownership
  rg.shard_count = 0;         // tests fold away
  const size_t rowi = (size_t)req * g.num_kv_heads + kv;
  const unsigned char* mm_row = (const unsigned char*)L.page_mm + rowi * stat_row_bytes(g.max_blocks, T::CPR);
  const unsigned char* sum_row = (const unsigned char*)L.page_sum + rowi * stat_row_bytes(g.max_blocks, T::NC);
  const int page_end = min(rg.kt_eff, g.max_blocks);
  const int tile_end = min(page_end, pools_end(rg));     // tiles behind the pools are skipped
  const int near_hi = min(min(rg.swa_lo_blk, rg.kt_eff), g.max_blocks);
  const int near_lo = rg.near_blks, near_lo8 = near_lo & ~7;
  const int n_near = near_hi > near_lo ? min(near_hi - near_lo8, L1_NEAR_CAP) : 0;
  uint16_t* r1_scn = (uint16_t*)(rank == 1 ? hist2 : cluster.map_shared_rank(hist2, 1));   // near row of rank 1

  // ---- level 1: score this CTA's tiles (rank, rank + CS, ...), two staging buffers ------------
  // one bulk copy per group of 32 pages, issued by the lanes of warp 0, counted on the buffer's mbarrier
  auto stage = [&](int it) {
    const int p0 = (rank + it * CS) * P;
    if (it < tiles_per_cta && p0 < tile_end)
      l1_issue_tile<DSUB, P, false>(g, rg, p0, page_end, rows + (size_t)(it & 1) * lay.rows_bytes, bars + (it & 1), mm_row,
                                    sum_row);
  };
  LODA_SUB0(50);
  __syncthreads();                                       // the barriers are initialised
  if (tid < 32) {
    stage(0);
    stage(1);
  }
  LODA_SUB0(51);
  if (early) pdl_wait();
  // scaled, bf16-rounded query on the subspace (nfa_layer_batch_selector.py:943-963)
  for (int i = tid; i < nq; i += P) {
    const int j = i / DSUB, d = i % DSUB;
    const float qv = __bfloat162float(q[((size_t)b * g.num_q_heads + kv * G + j) * g.head_dim + sub_dim(g, d)]);
    const float qh = bf16r(__fmul_rn(qv, scale));
    qhat[i] = qh;
    *(float2*)(qmm + 2 * i) = make_float2(fminf(qh, 0.0f), fmaxf(qh, 0.0f));
  }
  LODA_SUB0(52);
  cluster.barrier_wait();     // (0) every CTA of the cluster runs: its shared memory may be addressed from now on
  __syncthreads();            // (and qhat is complete)
  LODA_SUB0(53);
  // grouped query of level 2: the fp32 sum over the group, in head order, of the bf16-rounded scaled
  // query elements — exactly the values just stored in qhat (the barrier above orders them)
  if (tid < DSUB) {
    float acc = 0.0f;
    for (int j = 0; j < G; ++j) acc = __fadd_rn(acc, qhat[j * DSUB + tid]);
    qf[tid] = acc;
  }
  bool timed_out = false;
#pragma unroll 1
  for (int it = 0; it < tiles_per_cta; ++it) {
    const int p0 = (rank + it * CS) * P;
    if (p0 >= tile_end) break;
    if (!mbar_wait(bars + (it & 1), (uint32_t)(it >> 1) & 1u)) timed_out = true;      // tile it has landed
    LODA_SUB0(54 + 2 * it);
    const int page = p0 + tid;
    const uint32_t ord = l1_page_score<DSUB, P, false>(g, rg, p0, page_end, rows + (size_t)(it & 1) * lay.rows_bytes, qhat,
                                                       qmm, G);
    l_scall[page] = (uint16_t)ord;                       // into the leader's shared memory
    if (page >= near_lo && page < near_hi && page - near_lo8 < n_near) r1_scn[page - near_lo8] = (uint16_t)ord;
    __syncthreads();                                     // the buffer is free
    LODA_SUB0(55 + 2 * it);
    if (tid < 32) stage(it + 2);
  }
  if (timed_out && tid == 0 && status) atomicOr(status, LODA_STATUS_TIMEOUT);
  LODA_PHASE(sel, cta_id, 1);
  cluster.sync();                                        // (1) all page scores are in the leader
  LODA_PHASE(sel, cta_id, 2);

  if (rank == 2 && ap.enabled && tid < 32) {
    // The decode append of the row.  It touches only the newest token and its page, which lie
    // in the sliding window and are read by neither level of this step.  The attention phase of
    // this launch (and an attention launch after it) reads the token's K/V from global memory:
    // the cluster barriers between here and there order these stores before those reads.
    append_row<DSUB>(g, L, B, ap.k_new, ap.v_new, ap.slots, ap.status, b, kv, tid);
  }
  const int32_t* table = L.block_table + (size_t)req * g.max_blocks;
  // The page list lives in the leader in four parts at fixed places, so that the two selecting
  // CTAs need not know each other's counts:
  //   [0, np0) sink bypass | [np0, np0 + n_f) far | [np0 + k_far, .. + n_n) near | [np0 + k_far + k_near] window bypass
  const bool listed = rg.quota > 0;
  const bool want_lists = S.i_far != nullptr;
  const int np0 = (listed && rg.sink_byp && rg.spl < rg.kt_eff) ? 1 : 0;
  const int near_at = np0 + g.k_far, swa_at = np0 + g.k_far + g.k_near;
  auto phys_of = [&](int pg) {
    int ph = (pg >= 0 && pg < g.max_blocks) ? table[pg] : -1;
    return (ph < 0 || ph >= g.num_pages) ? -1 : ph;
  };
  if (rank == 0) {
    // far row = the row's scores in place, zero outside the far pool
    const int far_lo = rg.far_lo, far_hi = max(rg.far_hi, rg.far_lo);
    const int n_far = far_hi;
    uint16_t* scf = scall;
#pragma unroll 1
    for (int i = tid; i < far_lo; i += P) scf[i] = 0;
#pragma unroll 1
    for (int i = far_hi + tid; i < ((n_far + 7) & ~7); i += P) scf[i] = 0;
    __syncthreads();
    LODA_PHASE(sel, cta_id, 3);
    constexpr int H = P, HB = 0;       // the selection runs on all threads of the CTA (barrier 0)
    if (tid < H) {
      int r = 0;
      if ((listed || want_lists) && n_far > far_lo) {
        if (n_far <= H) {
          r = block_rank_topk_small<H, HB, 0>(scf, n_far, g.k_far, kept + np0, keys, wtot);
        } else if (n_far <= 2 * H) {
          r = block_rank_topk_pair<H, HB, 0>(scf, n_far, g.k_far, kept + np0, keys, wtot);
        } else {
          r = g.k_far <= 128 ? block_prefilter_topk<H, HB, 0>(scf, n_far, g.k_far, kept + np0, keys, wtot, sh) : -1;
          if (r < 0) r = block_bisect_topk<H, HB, 0>(scf, n_far, g.k_far, kept + np0, wtot);   // heavily tied scores
        }
      }
      if (tid == 0) sh[2] = r;
    }
    __syncthreads();
    const int n_f = sh[2];
    LODA_PHASE(sel, cta_id, 8);
    if (want_lists)
      emit_best_first<P>(kept + np0, n_f, g.k_far, scf, S.i_far + (size_t)row * g.k_far, S.n_far + row, g.max_blocks);
    if (listed) {
      if (tid == 0 && np0) { kept[0] = rg.spl; physk[0] = phys_of(rg.spl); }
      if (tid == 32 && rg.swa_byp) { kept[swa_at] = rg.swa_byp_blk; physk[swa_at] = phys_of(rg.swa_byp_blk); }
#pragma unroll 1
      for (int i = tid; i < n_f; i += P) physk[np0 + i] = phys_of(kept[np0 + i]);
    }
    LODA_PHASE(sel, cta_id, 4);
  } else if (rank == 1) {
    // near row: the pool's scores as the scoring CTAs stored them, zero outside the pool
    uint16_t* scn = (uint16_t*)hist2;
    int n_n = 0;
    if ((listed || want_lists) && n_near > 0) {      // n_near <= 512 = P
      n_n = block_rank_topk_small<P>(scn, n_near, g.k_near, kept, keys, wtot);
    }
    if (want_lists) {
      for (int i = tid; i < n_n; i += P) kept[i] += near_lo8;
      __syncthreads();
      // scores by page id: the row starts at page near_lo8
      emit_best_first<P>(kept, n_n, g.k_near, scn - near_lo8, S.i_near + (size_t)row * g.k_near, S.n_near + row,
                         g.max_blocks);
      __syncthreads();
      for (int i = tid; i < n_n; i += P) kept[i] -= near_lo8;
      __syncthreads();
    }
    if (listed) {
#pragma unroll 1
      for (int i = tid; i < n_n; i += P) {
        const int pg = kept[i] + near_lo8;
        l_kept[near_at + i] = pg;
        l_physk[near_at + i] = phys_of(pg);
      }
    }
    if (tid == 0) l_sh[3] = listed ? n_n : 0;
  }
  cluster.sync();                                        // (2) page list and physical pages are in the leader
  LODA_PHASE(sel, cta_id, 5);

  // ---- level 2: score this CTA's share of the candidate slots ---------------------------------
  const int np_max = g.k_far + g.k_near + 2;
  const int n_f = listed ? l_sh[2] : 0, n_n = l_sh[3];
  const int np = listed ? np0 + n_f + n_n + (rg.swa_byp ? 1 : 0) : 0;
  // place of list entry i in the leader's arrays
  auto place_of = [&](int i) { return i < np0 + n_f ? i : i < np0 + n_f + n_n ? i - n_f + g.k_far : swa_at; };
  const int nitems = np * g.page;
  {
    const int per = ((nitems + CS - 1) / CS + 7) & ~7;
    const int lo = min(rank * per, nitems), hi = min(lo + per, nitems);
#pragma unroll 1
    for (int idx = lo + tid; idx < hi; idx += P) {
      const int i = idx >> (31 - __clz(g.page)), o = idx & (g.page - 1);      // page is a power of two
      const int at = place_of(i);
      const int pg = l_kept[at], ph = l_physk[at];
      const uint32_t ord = l2_slot_score<DSUB, true>(g, L, rg, length, kv, pg, ph, o, qf, status);
      l_sc2[idx] = (uint16_t)ord;
      // the leader's histogram of the scores by their top 12 bits (two 16-bit counters per word)
      if (ord != 0u) atomicAdd(l_hist2 + (ord >> 5), 1u << ((ord >> 4 & 1u) * 16));
    }
    // the leader closes the gaps of its list for the last phase; its highest threads have no slot to score
    if (rank == 0) {
#pragma unroll 1
      for (int i = P - 1 - tid; i < np; i += P) {
        const int at = place_of(i);
        kept2[i] = kept[at];
        physk2[i] = physk[at];
      }
    }
  }
  LODA_PHASE(sel, cta_id, 6);
  cluster.sync();                                        // (3) all candidate scores are in the leader
  if (D == 0 && (rank != 0 || tid >= SF_L2_NT)) return;
  LODA_PHASE(sel, cta_id, 7);

  // ---- leader, first 256 threads: quota selection, hole fill, union, gather list --------------
  if (rank == 0 && tid < SF_L2_NT) {
    const int K2 = g.level2_topk;
    size_t off = ((size_t)np_max * g.page * 2 + 15) & ~(size_t)15;     // behind the scores
    L2Shared shm;
    shm.sc = (uint16_t*)rows;
    shm.pages = kept2;
    shm.physs = physk2;
    shm.mid_a = (int*)(rows + off); off += (size_t)K2 * 4;
    shm.mid_b = (int*)(rows + off); off += (size_t)K2 * 4;
    shm.win = (uint8_t*)(rows + off);
    shm.wtot = wtot;
    shm.scan = scan;
    shm.hist = hist2;
    if (D > 0) { shm.list = list; shm.list_n = sh + 5; }
    // with an attention phase the dependent launch is released after its tiles instead
    l2_select_and_write<SF_L2_NT, 1, true>(g, rg, S, status, table, b, kv, row, length, nitems, shm, nullptr, D == 0);
  }
  LODA_PHASE(sel, cta_id, 9);
  if constexpr (D > 0) {
    // ---- attention over the row's gather list, split over the CTAs of the cluster ------------
    // Every CTA takes a balanced chunk of the list (read from the leader's shared memory),
    // stages its K and V rows at once, each warp handles 16 tokens (attn_warp_step); warps,
    // then CTAs, merge by log-sum-exp in a fixed order; the CTAs' partials go to the leader,
    // which merges them and writes the output.
    constexpr int DV = D, KSTR = D + 8, VSTR = DV + 8, NTV = DV / 8, KCH = D / 8, NW = SF_P / 32;
    const int lane = tid & 31, warp = tid >> 5;
    const int q2r = at.query_to_req[b];
    uint32_t qa[D / 16][4];
    attn_load_q<D>(qa, q + ((size_t)b * g.num_q_heads + kv * G) * D, G, lane);
    const int* l_list = own ? list : cluster.map_shared_rank(list, 0);
    const int tcap = fused_attend_tile(g, lay.rows_bytes * (tiles_per_cta > 1 ? 2 : 1));
    bf16* Ks = (bf16*)rows;                              // [tcap][KSTR]
    bf16* Vs = Ks + (size_t)tcap * KSTR;                 // [tcap][VSTR]
    int* slot_t = (int*)(Vs + (size_t)tcap * VSTR);      // [tcap]
    float* wm = (float*)keys;                            // [NW][16]
    float* wz = wm + NW * 16;                            // [NW][16]
    float* wo = (float*)Ks;                              // [NW][G][DV], over the consumed K tile
    float* pfm = (float*)(smem + lay.pfm);               // leader: [CS][2][16]
    float* pfo = (float*)(smem + lay.pfo);               // leader: [CS][G][DV]
    float* l_pfm = own ? pfm : cluster.map_shared_rank(pfm, 0);
    float* l_pfo = own ? pfo : cluster.map_shared_rank(pfo, 0);
    const int page_log2 = 31 - __clz(g.page);
    const int slot_end = g.num_pages * g.page;
    float oacc[NTV][4];
#pragma unroll
    for (int i = 0; i < NTV; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, z_run[2] = {0.0f, 0.0f};
    cluster.sync();                                      // (4) the gather list is in the leader
    const int n = q2r == b ? min(max(l_sh[5], 0), g.max_visible) : 0;
    const int c0 = (int)(((long long)rank * n) / CS), c1 = (int)(((long long)(rank + 1) * n) / CS);
#pragma unroll 1
    for (int p0 = c0; p0 < c1; p0 += tcap) {
      const int ntok = min(tcap, c1 - p0);
      __syncthreads();                                 // the tile (or the partials) of the pass before is consumed
      // 16-byte chunk kc of rows kr, kr + 32, ...: all their list entries in one round of remote loads,
      // then the copies; masked rows, and rows beyond ntok up to the next multiple of 16, are zero-filled
      constexpr int RPI = SF_P / KCH, NIT = 256 / RPI;
      const int kr = tid / KCH, kc = tid % KCH;
      const int nrow = (ntok + 15) & ~15;
      int sl[NIT];
#pragma unroll
      for (int k = 0; k < NIT; ++k) {
        const int r = kr + k * RPI;
        const int s = r < ntok ? l_list[p0 + r] : -1;
        sl[k] = s >= slot_end ? -1 : s;
      }
#pragma unroll
      for (int k = 0; k < NIT; ++k) {
        const int r = kr + k * RPI, s = sl[k];
        if (r < nrow) {
          const long long off = s >= 0 ? ((long long)(s >> page_log2) * g.num_kv_heads + kv) * g.page + (s & (g.page - 1)) : 0;
          cp_async16(Ks + (size_t)r * KSTR + kc * 8, (const bf16*)L.pool_k + off * D + kc * 8, s >= 0);
          cp_async16(Vs + (size_t)r * VSTR + kc * 8, (const bf16*)L.pool_v + off * DV + kc * 8, s >= 0);
          if (kc == 0) slot_t[r] = s;
        }
      }
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
      if (warp * 16 < ntok) attn_warp_step<D, DV>(Ks, Vs, slot_t, warp * 16, ntok, qa, at.scale_log2, oacc, m_run, z_run);
    }
    // The dependent launch is released here: the next layer's launch then runs its prologue (metadata,
    // first statistics tiles) while this one merges.  Releasing earlier gains nothing (measured at the
    // kernel's start, after level 1 and before the attention: the same step time): the prologue is
    // already hidden, and the dependent's wait ends when this grid has completed, wherever it was released.
    pdl_launch_dependents();
    LODA_PHASE(sel, cta_id, 10);
    // merge the warps of this CTA (fixed order) and hand the CTA's partial to the leader
    __syncthreads();                                   // every warp is done with the tile
    {
      const int r0 = lane >> 2;
      if ((lane & 3) == 0) {
        wm[warp * 16 + r0] = m_run[0]; wz[warp * 16 + r0] = z_run[0];
        wm[warp * 16 + r0 + 8] = m_run[1]; wz[warp * 16 + r0 + 8] = z_run[1];
      }
#pragma unroll
      for (int i = 0; i < NTV; ++i) {
        const int col = i * 8 + (lane & 3) * 2;
        if (r0 < G) { wo[(warp * G + r0) * DV + col] = oacc[i][0]; wo[(warp * G + r0) * DV + col + 1] = oacc[i][1]; }
        if (r0 + 8 < G) { wo[(warp * G + r0 + 8) * DV + col] = oacc[i][2]; wo[(warp * G + r0 + 8) * DV + col + 1] = oacc[i][3]; }
      }
    }
    __syncthreads();
#pragma unroll 1
    for (int e = tid; e < G * DV; e += SF_P) {
      const int gi = e / DV, dv = e % DV;
      float pm[NW];
#pragma unroll
      for (int w = 0; w < NW; ++w) pm[w] = wm[w * 16 + gi];
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) M = fmaxf(M, pm[w]);
      float z = 0.0f, o = 0.0f;
      if (M != -INFINITY) {
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          const float a = exp2f(pm[w] - M);
          z += wz[w * 16 + gi] * a;
          o += wo[(w * G + gi) * DV + dv] * a;
        }
      }
      l_pfo[(size_t)rank * G * DV + e] = o;
      if (dv == 0) { l_pfm[rank * 32 + gi] = M; l_pfm[rank * 32 + 16 + gi] = z; }
    }
    if (rank != 0) {
      cluster.sync();                                    // (5) every CTA's partial is in the leader
      return;
    }
    // the leader merges the CTAs' partials in rank order and writes the row's output
    {
      cluster.sync();                                    // (5)
      LODA_PHASE(sel, cta_id, 11);
#pragma unroll 1
      for (int e = tid; e < G * DV; e += SF_P) {
        const int gi = e / DV, dv = e % DV;
        float pm[SF_CLUSTER_MAX];
#pragma unroll
        for (int s2 = 0; s2 < SF_CLUSTER_MAX; ++s2) pm[s2] = s2 < CS ? pfm[s2 * 32 + gi] : -INFINITY;
        float M = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < SF_CLUSTER_MAX; ++s2) M = fmaxf(M, pm[s2]);
        float z = 0.0f, o = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
          for (int s2 = 0; s2 < SF_CLUSTER_MAX; ++s2) {
            if (s2 < CS) {
              const float a = exp2f(pm[s2] - M);
              z += pfm[s2 * 32 + 16 + gi] * a;
              o += pfo[(size_t)s2 * G * DV + e] * a;
            }
          }
        }
        at.out[((size_t)b * g.num_q_heads + kv * G + gi) * DV + dv] = __float2bfloat16_rn(z == 0.0f ? 0.0f : o / z);
      }
    }
    LODA_PHASE(sel, cta_id, 12);
  }
}

// Host state of the launch decision, kept per device ordinal: a refusal on one GPU or an occupancy
// answer from one GPU says nothing about another.  (Host calls are single-threaded per device.)
constexpr int kMaxDevices = 64;
static bool g_fused_refused[kMaxDevices][3] = {};    // per sub-space width: a launch failed, stay on the chain

static thread_local int g_last_cluster_size = 0;      // CTAs per row of the calling thread's latest one-launch call
int select_fused_last_cluster() { return g_last_cluster_size; }

static int fused_slot(int sub_dims) { return sub_dims == 16 ? 0 : sub_dims == 32 ? 1 : 2; }

static int fused_tiles_per_cta(const loda_geometry& g, int cs) {
  const int ntiles = (g.max_blocks + SF_P - 1) / SF_P;
  return (ntiles + cs - 1) / cs;
}

static bool fused_shape_ok(const loda_geometry& g, int cs) {
  const FusedLayout lay = fused_layout(g, fused_tiles_per_cta(g, cs), cs);
  return lay.total <= 220 * 1024 && fused_l2_bytes(g) <= lay.rows_bytes;     // the level-2 arrays overlay the rows
}

// whether the fused launch may serve this geometry and batch (the launch itself still asks the
// GPU how many clusters of the shape it can hold)
bool select_fused_applicable(const loda_geometry& g, int rows) {
  // LODA_B200_SELECT_PATH=split forces the two-launch chain (A/B measurements, tests of both paths)
  const char* path = getenv("LODA_B200_SELECT_PATH");
  if (path && strcmp(path, "split") == 0) return false;
  if (g.sub_dims != 16 && g.sub_dims != 32 && g.sub_dims != 64) return false;
  const int dev = device_ordinal();
  if (dev < 0 || dev >= kMaxDevices || g_fused_refused[dev][fused_slot(g.sub_dims)]) return false;
  if (rows < 1 || rows * 8 > device_sm_count()) return false;                // one round of clusters of 8 at least
  // other level-1 methods and the numeric near-token quota run on the two-launch chain
  if (g.far_method != LODA_FAR_MINMAX || g.near_minmax != 0 || g.near_tokens_p1 > 0) return false;
  if ((size_t)g.max_blocks * 2 + 16 > 40 * 1024) return false;
  for (int i = 0; i < SF_NSIZES; ++i)
    if (fused_shape_ok(g, SF_CLUSTER_SIZES[i])) return true;
  return false;
}

// whether the launch may also run the attention of the step on a cluster of cs CTAs
static bool fused_attend_ok(const loda_geometry& g, int cs) {
  // LODA_B200_DECODE_PATH=split keeps the attention in its own launch (A/B measurements, tests of both paths)
  const char* path = getenv("LODA_B200_DECODE_PATH");
  if (path && strcmp(path, "split") == 0) return false;
  if (g.head_dim != 128 || g.head_dim_v != 128) return false;
  const int G = g.num_q_heads / g.num_kv_heads;
  const FusedLayout lay = fused_layout(g, fused_tiles_per_cta(g, cs), cs);
  const int tcap = fused_attend_tile(g, lay.rows_bytes * (fused_tiles_per_cta(g, cs) > 1 ? 2 : 1));
  // the warps' partial outputs and the CTA's merged one lie over the K tile
  return tcap >= 16 && (size_t)(SF_P / 32 + 1) * G * g.head_dim_v * 4 <= (size_t)tcap * (g.head_dim + 8) * 2 && G <= 16;
}

template <int DS, int D>
static cudaError_t launch_fused_d(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                                  float scale, const loda_selection& S, uint32_t* status, const AppendArgs& ap,
                                  const FusedAttend& at, cudaStream_t st) {
  const int rows = B.batch * g.num_kv_heads;
  auto kernel = select_fused_kernel<DS, D>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) return e;
  // clusters of 16 CTAs when the GPU holds one for every row at once (a cluster lives inside one GPC, so the
  // count that fits depends on the GPCs' sizes), else clusters of 8; the answers are remembered per shape
  struct Memo { size_t smem; int rows_ok; };
  static Memo memo[kMaxDevices][3][SF_NSIZES] = {};      // (per instantiation of this template)
  const int dev = device_ordinal();
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorNotSupported;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cfg.blockDim = dim3(SF_P);
  cfg.stream = st;
  const char* force = getenv("LODA_B200_CLUSTER");       // A/B measurements: one cluster size only
  const int forced = force ? atoi(force) : 0;
  for (int which = 0; which < SF_NSIZES; ++which) {
    int cs = SF_CLUSTER_SIZES[which];
    if (forced >= 3 && forced <= SF_CLUSTER_MAX) {         // a forced size need not be one of the defaults
      if (which > 0) break;
      cs = forced;
    }
    if (!fused_shape_ok(g, cs) || rows * cs > device_sm_count()) continue;
    if (D > 0 && !fused_attend_ok(g, cs)) continue;
    const int tpc = fused_tiles_per_cta(g, cs);
    const size_t smem = fused_layout(g, tpc, cs).total;
    e = set_kernel_smem(kernel, smem);
    if (e != cudaSuccess) return e;
    cfg.gridDim = dim3(cs, rows);
    cfg.dynamicSmemBytes = smem;
    attr[1].val.clusterDim.x = cs;
    Memo& m = memo[dev][fused_slot(DS)][which];
    if (m.smem != smem) {
      int nclusters = 0;
      if (cudaOccupancyMaxActiveClusters(&nclusters, kernel, &cfg) != cudaSuccess) { (void)cudaGetLastError(); nclusters = 0; }
      m.smem = smem;
      m.rows_ok = nclusters;
    }
    if (rows > m.rows_ok) continue;                      // the clusters of all rows must run at once
    g_last_cluster_size = cs;
    return cudaLaunchKernelEx(&cfg, kernel, g, L, B, (const bf16*)q, scale, S, status, ap, tpc, at);
  }
  return cudaErrorNotSupported;
}

void select_fused_refuse(int sub_dims) {
  const int dev = device_ordinal();
  if (dev >= 0 && dev < kMaxDevices) g_fused_refused[dev][fused_slot(sub_dims)] = true;
}

// cudaErrorNotSupported = the caller launches the two-kernel chain instead
cudaError_t launch_select_fused(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                                float scale, const loda_selection& S, uint32_t* status, const AppendArgs& ap,
                                cudaStream_t st) {
  const FusedAttend none{nullptr, nullptr, 0.0f};
  switch (g.sub_dims) {
    case 16: return launch_fused_d<16, 0>(g, L, B, q, scale, S, status, ap, none, st);
    case 32: return launch_fused_d<32, 0>(g, L, B, q, scale, S, status, ap, none, st);
    case 64: return launch_fused_d<64, 0>(g, L, B, q, scale, S, status, ap, none, st);
    default: return cudaErrorNotSupported;
  }
}

// The same launch followed, inside it, by the attention of the step (out [batch, Hq, head_dim_v],
// query_to_req the identity or < 0).  cudaErrorNotSupported = nothing was launched: the caller runs
// the selection and the attention as separate launches.
cudaError_t launch_decode_fused(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                                float scale, const loda_selection& S, uint32_t* status, const AppendArgs& ap,
                                const int32_t* query_to_req, void* out, cudaStream_t st) {
  const FusedAttend at{query_to_req, (bf16*)out, scale * 1.4426950408889634f};
  switch (g.sub_dims) {
    case 16: return launch_fused_d<16, 128>(g, L, B, q, scale, S, status, ap, at, st);
    case 32: return launch_fused_d<32, 128>(g, L, B, q, scale, S, status, ap, at, st);
    case 64: return launch_fused_d<64, 128>(g, L, B, q, scale, S, status, ap, at, st);
    default: return cudaErrorNotSupported;
  }
}

}  // namespace loda
