// Fused L2 kernel: the tokens of the pages that survived L1 are scored on the
// packed 4-bit tail keys (unpacked in registers) by L2_SPLIT CTAs per
// (request, kv head) row; the last CTA of the row to finish (atomic ticket, no
// spinning) keeps the exact top-quota tokens (ties toward the lower token id),
// fills holes, merges the sink and sliding-window tokens and writes physical
// slots.
//
// Restates candidate expansion (nfa_layer_batch_selector.py:1194-1251), the
// grouped-query logits (:422-516, :978-1002), the filtered top-k with quota and
// hole fill (:518-605) and the final union (:1336-1437).  Candidates are
// implicit: L1 hands over the selected pages in ascending page order, so the
// local slot (rank * page + offset) is monotone in the token id; selecting on
// the 16-bit ordered logit with ties toward the lower slot, compacted in slot
// order, yields the survivors as ascending tokens without a sort.
//
// Canonical arithmetic: the de-quantised key is bf16(bf16(code * scale) - zero);
// q_fine[d] is the fp32 sum over the GQA group (head order) of the bf16-rounded
// scaled query; the logit is one left-to-right fp32 chain of separate multiplies
// and adds over the d' dims, rounded to bf16.
#include "loda_select.cuh"

namespace loda {

#ifndef LODA_L2_MINB
#define LODA_L2_MINB 1     // resident CTAs per SM the register budget must allow (4 costs spills)
#endif
#ifndef LODA_L2_CTAS_PER_SM
#define LODA_L2_CTAS_PER_SM 1
#endif

LODA_PHASE_STORAGE(l2)
LODA_SUB_READER(l2)

constexpr int L2_SPLIT = 8;
constexpr int L2_NT = 256;

template <int DSUB, int NT, bool NUMERIC>
__global__ void __launch_bounds__(NT, LODA_L2_MINB) l2_kernel(loda_geometry g, loda_layer L, loda_batch B,
                                                 const bf16* __restrict__ q, float scale,
                                                 loda_selection S, SelectWorkspace ws, uint32_t* status,
                                                 int nsplit, int chained, int phase) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int np_max = g.k_far + g.k_near + 2;
  const int K2 = g.level2_topk;
  // shared memory: scores (u16) | qf | pages | mid | mid2 | hist | scan | sh | win
  // (offsets, not pointer arithmetic through integers: the compiler must keep seeing shared memory)
  uint16_t* sc = (uint16_t*)smem;
  size_t off = ((size_t)np_max * g.page * 2 + 15) & ~(size_t)15;
  float* qf = (float*)(smem + off); off += DSUB * 4;
  int* pages = (int*)(smem + off); off += (size_t)np_max * 4;
  int* physs = (int*)(smem + off); off += (size_t)np_max * 4;
  int* mid_a = (int*)(smem + off); off += (size_t)K2 * 4;
  int* mid_b = (int*)(smem + off); off += (size_t)K2 * 4;
  off = (off + 15) & ~(size_t)15;
  int* wtot = (int*)(smem + off); off += 192 * 4;
  int* scan = (int*)(smem + off); off += 40 * 4;
  int* sh = (int*)(smem + off); off += 16 * 4;
  uint8_t* win = (uint8_t*)(smem + off); off += ((size_t)K2 + 15) & ~(size_t)15;
  uint32_t* hist = (uint32_t*)(smem + off); off += 2048 * 4;      // the row's scores by their top 12 bits (selecting CTA)
  // numeric near-token quota only: one region's scores and the concatenated middle
  uint16_t* sc2 = (uint16_t*)(smem + off); off += ((size_t)np_max * g.page * 2 + 15) & ~(size_t)15;
  int* fin = (int*)(smem + off);

  const int tid = threadIdx.x;
  const int split = blockIdx.x, row = blockIdx.y;
  const int cta_id = row * gridDim.x + split;
  LODA_PHASE(l2, cta_id, 0);
  const int b = row / g.num_kv_heads, kv = row % g.num_kv_heads;
  const int G = g.num_q_heads / g.num_kv_heads;
  // A launch chained behind the level-1 launch of the same call (which writes neither) reads the batch
  // metadata and the query before its dependency wait; a launch that stands alone may follow any
  // kernel (one that advances the lengths, for instance) and reads nothing before the wait.
  if (!chained) pdl_wait();
  int length = B.lengths[b];
  const int req = checked_request(g, B.active_req_ids[b], B.valid_req_ids[b], &length, status);
  bool skip_far, skip_near;
  load_skip_flags(L, req, &skip_far, &skip_near);
  const Regions rg = make_regions(g, length, skip_far, skip_near);
  const int32_t* table = L.block_table + (size_t)req * g.max_blocks;

  // ---- grouped query on the subspace ---------------------------------------
  // It depends only on inputs of the step.  Chained behind the L1 launch of the same call
  // (which reads the query after its own wait) it is computed before this launch's wait;
  // a launch that stands alone computes it after.
  auto group_query = [&]() {
    if (tid < DSUB) {
      float acc = 0.0f;
      for (int j = 0; j < G; ++j) {
        const float qv = __bfloat162float(q[((size_t)b * g.num_q_heads + kv * G + j) * g.head_dim + sub_dim(g, tid)]);
        acc = __fadd_rn(acc, bf16r(__fmul_rn(qv, scale)));
      }
      qf[tid] = acc;
    }
  };
  group_query();
  LODA_PHASE(l2, cta_id, 1);
  if (chained) pdl_wait();
#if LODA_PDL_TRIGGER == 0
  pdl_launch_dependents();
#endif
  __syncthreads();
  LODA_PHASE(l2, cta_id, 2);

  const int np = min(__ldcg(ws.np + row), np_max);
  const int nitems = np * g.page;
  uint16_t* row_scores = ws.l2_scores + (size_t)row * np_max * g.page;
  // the row's page list (at most k_far + k_near + 2 entries) in shared memory: the scoring loop and the
  // selection both index it
  for (int i = tid; i < np; i += NT) {
    pages[i] = __ldcg(ws.pages + (size_t)row * np_max + i);
    physs[i] = __ldcg(ws.phys + (size_t)row * np_max + i);
  }
  __syncthreads();
  // ---- score this CTA's share of the candidate slots ---------------------------
  // U slots per thread and round: first every slot's codes and (scale, zero) are requested, then the
  // logits are formed — one round trip to memory per round instead of one per slot
  {
    constexpr int U = 4, WORDS = DSUB / 8;
    const int pl2 = 31 - __clz(g.page), pmask = g.page - 1;         // page is a power of two
    const int per = ((nitems + nsplit - 1) / nsplit + 7) & ~7;         // multiple of 8 slots
    const int lo = min(split * per, nitems), hi = phase == 2 ? lo : min(lo + per, nitems);
#pragma unroll 1
    for (int base = lo + tid; base < hi; base += U * NT) {
      uint32_t w[U][WORDS];
      uint32_t sz[U];
      bool ok[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = base + u * NT;
        ok[u] = false;
        if (idx < hi) {
          const int i = idx >> pl2, o = idx & pmask;
          const int pg = pages[i], ph = physs[i];
          const int tok = pg * g.page + o;
          if (ph >= 0 && tok >= g.sink && tok < rg.swa_lo_tok && tok < length && tok >= rg.lower && tok < rg.upper) {
            const size_t trow = ((size_t)ph * g.num_kv_heads + kv) * g.page + o;
            sz[u] = *(const uint32_t*)((const bf16*)L.tail_sz + trow * 2);
            l2_load_codes<DSUB>((const uint8_t*)L.tail_code + trow * (DSUB / 2), w[u]);
            ok[u] = true;
          } else if (ph < 0 && status && rg.shard_count <= 1) {      // under sequence sharding a missing page is another GPU's
            atomicOr(status, LODA_STATUS_BAD_PAGE);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = base + u * NT;
        if (idx < hi) {
          uint32_t ord = 0;
          if (ok[u]) {
            const float lg = l2_logit_words<DSUB>(w[u], sz[u], qf);
            if (lg == lg && lg != -INFINITY) ord = ord16(lg);
          }
          row_scores[idx] = (uint16_t)ord;
        }
      }
    }
  }
  LODA_PHASE(l2, cta_id, 3);

  // ---- last CTA of the row selects ----------------------------------------------
  // phase 1 = scores only (the caller combines the score rows of several GPUs before the
  // selection), phase 2 = selection only (one CTA per row, which scored nothing above)
  if (phase == 1) return;
  if (phase == 0) {
    __threadfence();
    __syncthreads();
    if (tid == 0) sh[0] = (atomicAdd(ws.l2_ticket + row, 1) == nsplit - 1);
    __syncthreads();
    LODA_PHASE(l2, cta_id, 4);
    if (!sh[0]) return;
    __threadfence();
  }
  // the row's scores into shared memory, counted on the way into a histogram by their top 12 bits (two
  // 16-bit counters per word): the selection starts from the bin of the quota-th best score
  for (int i = tid; i < 2048 / 4; i += NT) ((uint4*)hist)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  for (int i = tid; i < (nitems + 7) / 8; i += NT) {
    uint4 v;
    if (ws.gathered == nullptr) {
      v = __ldcg((const uint4*)row_scores + i);
    } else {                                               // sequence sharding: the rows of all GPUs, ORed while loading
      v = make_uint4(0u, 0u, 0u, 0u);
      for (int s = 0; s < ws.n_gathered; ++s) {
        const uint4 u = __ldcg((const uint4*)(ws.gathered + s * ws.gathered_stride + (size_t)row * np_max * g.page) + i);
        v.x |= u.x; v.y |= u.y; v.z |= u.z; v.w |= u.w;
      }
    }
    ((uint4*)sc)[i] = v;
    uint32_t o[8];
    unpack_u16x8(v, o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (o[j] != 0u && i * 8 + j < nitems) atomicAdd(hist + (o[j] >> 5), 1u << ((o[j] >> 4 & 1u) * 16));
    }
  }
  __syncthreads();
#if LODA_PDL_TRIGGER == 3
  pdl_launch_dependents();
#endif
  LODA_PHASE(l2, cta_id, 5);
  L2Shared shm{sc, pages, physs, mid_a, mid_b, wtot, scan, win};
  shm.sc2 = sc2;
  shm.fin = fin;
  shm.hist = hist;
  l2_select_and_write<NT, 0, true, NUMERIC>(g, rg, S, status, table, b, kv, row, length, nitems, shm, ws.l2_ticket + row,
                                             LODA_PDL_TRIGGER == 1);
  LODA_PHASE(l2, cta_id, 9);
}

// sink ++ window of every (batch row, kv head) as physical slots: the union of l2_select_and_write
// with an empty middle (the reference builds its protected list the same way,
// paged_region_kernels_nfa.py:84-119)
__global__ void __launch_bounds__(128) protected_gather_kernel(loda_geometry g, loda_layer L, loda_batch B,
                                                               int32_t* __restrict__ gather,
                                                               int32_t* __restrict__ visible_lens, uint32_t* status) {
  const int row = blockIdx.x, b = row / g.num_kv_heads, kv = row % g.num_kv_heads;
  pdl_wait();
  int length = B.lengths[b];
  const int req = checked_request(g, B.active_req_ids[b], B.valid_req_ids[b], &length, status);
  const int32_t* table = L.block_table + (size_t)req * g.max_blocks;
  const int pl2 = 31 - __clz(g.page), pmask = g.page - 1;
  const int cap = g.max_blocks * g.page;
  const int sk = min(length, g.sink);
  const int count_s = min(length, g.sink + g.swa) - sk;
  const int s_lo = max(max(length - g.swa, 0), sk);
  const int s_hi = min(length - g.swa + count_s, cap);
  const int n_s = max(s_hi - s_lo, 0);
  const int total = sk + n_s;
  const int n_out = min(total, g.max_visible);
  int32_t* gout = gather + ((size_t)b * g.num_kv_heads + kv) * g.max_visible;
  for (int i = threadIdx.x; i < n_out; i += blockDim.x) {
    const int id = i < sk ? i : s_lo + (i - sk);
    const int lp = id >> pl2;
    int ph = lp < g.max_blocks ? table[lp] : -1;
    if (ph < 0 || ph >= g.num_pages) {
      if (g.shard_count > 1) {
        ph = -1;
      } else {
        if (status) atomicOr(status, LODA_STATUS_BAD_PAGE);
        ph = g.num_pages - 1;
      }
    }
    gout[i] = ph >= 0 ? ph * g.page + (id & pmask) : -1;
  }
  if (threadIdx.x == 0) {
    visible_lens[(size_t)b * g.num_kv_heads + kv] = n_out;
    if (total > g.max_visible && status) atomicOr(status, LODA_STATUS_TRUNCATED);
  }
}

cudaError_t launch_protected_gather(const loda_geometry& g, const loda_layer& L, const loda_batch& B, int32_t* gather,
                                    int32_t* visible_lens, uint32_t* status, cudaStream_t st) {
  const int rows = B.batch * g.num_kv_heads;
  if (rows <= 0) return cudaSuccess;
  return launch_pdl(protected_gather_kernel, dim3(rows), dim3(128), 0, st, g, L, B, gather, visible_lens, status);
}

size_t l2_smem_bytes(const loda_geometry& g) {
  const size_t np_max = g.k_far + g.k_near + 2;
  const bool numeric = g.near_tokens_p1 > 0;      // a masked copy of the scores and the concatenated middle
  return ((np_max * g.page * 2 + 15) & ~(size_t)15) * (numeric ? 2 : 1) + g.sub_dims * 4 + 2 * np_max * 4 +
         (numeric ? 3 : 2) * (size_t)g.level2_topk * 4 + 192 * 4 + (40 + 16) * 4 + g.level2_topk + 64 + 2048 * 4;
}

template <int DS>
static cudaError_t launch_l2_d(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                               float scale, const loda_selection& S, const SelectWorkspace& ws, uint32_t* status,
                               bool chained, int phase, cudaStream_t st) {
  // scoring CTAs per row: 8 at batch 1 (latency), one once the rows alone give every SM a CTA
  // (every CTA of a row pays the ticket; the row's selection runs in one CTA either way)
  const int rows = B.batch * g.num_kv_heads;
  int nsplit = (LODA_L2_CTAS_PER_SM * device_sm_count() + rows - 1) / rows;
  nsplit = nsplit < 1 ? 1 : nsplit > L2_SPLIT ? L2_SPLIT : nsplit;
  const dim3 grid(phase == 2 ? 1 : nsplit, rows);      // selection only: one CTA per row
  const size_t smem = l2_smem_bytes(g);
  if (g.near_tokens_p1 > 0) {      // numeric near-token quota: the instantiation with the two-region selection
    cudaError_t e = set_kernel_smem(l2_kernel<DS, L2_NT, true>, smem);
    if (e != cudaSuccess) return e;
    return launch_pdl(l2_kernel<DS, L2_NT, true>, grid, dim3(L2_NT), smem, st, g, L, B, (const bf16*)q, scale, S, ws,
                      status, nsplit, (int)chained, phase);
  }
  cudaError_t e = set_kernel_smem(l2_kernel<DS, L2_NT, false>, smem);
  if (e != cudaSuccess) return e;
  return launch_pdl(l2_kernel<DS, L2_NT, false>, grid, dim3(L2_NT), smem, st, g, L, B, (const bf16*)q, scale, S, ws, status,
                    nsplit, (int)chained, phase);
}

cudaError_t launch_l2(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                      float scale, const loda_selection& S, const SelectWorkspace& ws, uint32_t* status,
                      bool chained, int phase, cudaStream_t st) {
  switch (g.sub_dims) {
    case 16: return launch_l2_d<16>(g, L, B, q, scale, S, ws, status, chained, phase, st);
    case 32: return launch_l2_d<32>(g, L, B, q, scale, S, ws, status, chained, phase, st);
    case 64: return launch_l2_d<64>(g, L, B, q, scale, S, ws, status, chained, phase, st);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace loda
