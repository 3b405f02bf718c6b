// Fused L2 kernel: one CTA per (request, kv head) row scores every token of the
// pages that survived L1 on the packed 4-bit tail keys, keeps the exact
// top-quota tokens (ties toward the lower token id), fills holes, merges the
// sink and sliding-window tokens and writes physical slots — all in shared
// memory and registers.
//
// Restates candidate expansion (nfa_layer_batch_selector.py:1194-1251), the
// grouped-query logits (:422-516, :978-1002), the filtered top-k with quota and
// hole fill (:518-605) and the final union (:1336-1437).  Candidates are
// implicit: the selected pages are sorted by page id, so the local slot
// (sorted rank * page + offset) is monotone in the token id; the key
// (ordered bf16 logit << 16) | (0xFFFF - slot) then orders by logit descending
// and token ascending, and a compaction in slot order yields ascending tokens
// without a sort.
//
// Canonical arithmetic: the de-quantised key is bf16(bf16(code * scale) - zero);
// q_fine[d] is the fp32 sum over the GQA group (head order) of the bf16-rounded
// scaled query; the logit is one left-to-right fp32 chain of separate multiplies
// and adds over the d' dims, rounded to bf16.
#include "loda_common.cuh"

namespace loda {

using bf16 = __nv_bfloat16;

template <int DSUB>
__device__ __forceinline__ float l2_logit(const uint8_t* __restrict__ codes, float scale, float zero,
                                          const float* __restrict__ qf) {
  constexpr int WORDS = DSUB / 8;   // 32-bit words of packed codes
  uint32_t w[WORDS];
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
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < WORDS; ++i) {
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float c = (float)((w[i] >> (4 * n)) & 15u);
      const float x = bf16r(__fsub_rn(bf16r(__fmul_rn(c, scale)), zero));
      acc = __fadd_rn(acc, __fmul_rn(x, qf[8 * i + n]));
    }
  }
  return bf16r(acc);
}

struct L2Smem {
  int* pages;      // [np_max] selected pages (unsorted)
  int* sorted;     // [np_max] ascending page ids
  int* phys;       // [np_max]
  float* qf;       // [DSUB]
  uint32_t* keys;  // [np_max * page]
  int* mid;        // [K2]
  int* mid2;       // [K2]
  uint8_t* win;    // [K2]
  int* hist;       // 258
  int* scan;       // 40
  int* sh;         // 16
};

template <int DSUB, int NT>
__global__ void __launch_bounds__(NT) l2_kernel(loda_geometry g, loda_layer L, loda_batch B,
                                                 const bf16* __restrict__ q, float scale,
                                                 loda_selection S, uint32_t* status) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int np_max = g.k_far + g.k_near + 2;
  const int K2 = g.level2_topk;
  L2Smem m;
  {
    unsigned char* p = smem;
    m.keys = (uint32_t*)p; p += (size_t)np_max * g.page * 4;
    m.qf = (float*)p; p += DSUB * 4;
    m.pages = (int*)p; p += np_max * 4;
    m.sorted = (int*)p; p += np_max * 4;
    m.phys = (int*)p; p += np_max * 4;
    m.mid = (int*)p; p += K2 * 4;
    m.mid2 = (int*)p; p += K2 * 4;
    m.hist = (int*)p; p += 258 * 4;
    m.scan = (int*)p; p += 40 * 4;
    m.sh = (int*)p; p += 16 * 4;
    m.win = (uint8_t*)p;
  }
  const int tid = threadIdx.x;
  const int row = blockIdx.x;
  const int b = row / g.num_kv_heads, kv = row % g.num_kv_heads;
  const int G = g.num_q_heads / g.num_kv_heads;
  const bool active = B.active_req_ids[b] >= 0;
  const int length = active ? B.lengths[b] : 0;
  const int req = (int)B.valid_req_ids[b];
  const Regions rg = make_regions(g, length);
  const int32_t* table = L.block_table + (size_t)req * g.max_blocks;

  // ---- grouped query on the subspace ---------------------------------------
  if (tid < DSUB) {
    float acc = 0.0f;
    for (int j = 0; j < G; ++j) {
      const float qv = __bfloat162float(q[((size_t)b * g.num_q_heads + kv * G + j) * g.head_dim + sub_dim(g, tid)]);
      acc = __fadd_rn(acc, bf16r(__fmul_rn(qv, scale)));
    }
    m.qf[tid] = acc;
  }

  // everything above depends only on inputs of the step; the L1 results below
  // are produced by the preceding launch
  pdl_wait();
  pdl_launch_dependents();

  // ---- page list -------------------------------------------------------------
  int np = 0;
  const int n_f = rg.quota > 0 ? min(S.n_far[row], g.k_far) : 0;
  const int n_n = rg.quota > 0 ? min(S.n_near[row], g.k_near) : 0;
  if (rg.quota > 0) {
    for (int i = tid; i < n_f; i += NT) m.pages[i] = S.i_far[(size_t)row * g.k_far + i];
    for (int i = tid; i < n_n; i += NT) m.pages[n_f + i] = S.i_near[(size_t)row * g.k_near + i];
    np = n_f + n_n;
    if (rg.sink_byp) { if (tid == 0) m.pages[np] = rg.spl; ++np; }
    if (rg.swa_byp) { if (tid == 0) m.pages[np] = rg.swa_byp_blk; ++np; }
  }
  __syncthreads();
  // ascending rank by counting (page ids are distinct)
  for (int i = tid; i < np; i += NT) {
    const int pg = m.pages[i];
    int rank = 0;
    for (int j = 0; j < np; ++j) rank += m.pages[j] < pg;
    m.sorted[rank] = pg;
    int ph = (pg >= 0 && pg < g.max_blocks) ? table[pg] : -1;
    if (ph < 0 || ph >= g.num_pages) {
      ph = -1;
      if (status) atomicOr(status, LODA_STATUS_BAD_PAGE);
    }
    m.phys[rank] = ph;
  }
  __syncthreads();

  // ---- logits and keys -------------------------------------------------------
  const int nitems = np * g.page;
  int my_valid = 0;
  for (int idx = tid; idx < nitems; idx += NT) {
    const int i = idx / g.page, o = idx % g.page;
    const int tok = m.sorted[i] * g.page + o;
    const int ph = m.phys[i];
    uint32_t key = 0;
    if (ph >= 0 && tok >= g.sink && tok < rg.swa_lo_tok && tok < length && tok >= rg.lower && tok < rg.upper) {
      const size_t trow = ((size_t)ph * g.num_kv_heads + kv) * g.page + o;
      const __nv_bfloat162 sz = *(const __nv_bfloat162*)((const bf16*)L.tail_sz + trow * 2);
      const float lg = l2_logit<DSUB>(L.tail_code + trow * (DSUB / 2), __low2float(sz), __high2float(sz), m.qf);
      if (lg == lg && lg != -INFINITY) {
        key = (ord16(lg) << 16) | (uint32_t)(0xFFFF - idx);
        ++my_valid;
      }
    }
    m.keys[idx] = key;
  }
  const int quota = rg.quota;
  int nvalid = 0;
  block_exclusive_scan<NT>(my_valid, m.scan, &nvalid);   // also a barrier for keys[]
  const int take = min(quota, nvalid);
  uint32_t thr = 1u;
  if (nvalid > quota) thr = block_kth_largest<NT>(m.keys, nitems, quota, m.hist);

  // ---- compaction in slot order = ascending token order -----------------------
  {
    const int ipt = (nitems + NT - 1) / NT;
    const int lo = min(tid * ipt, nitems), hi = min(lo + ipt, nitems);
    int cnt = 0;
    for (int idx = lo; idx < hi; ++idx) cnt += (m.keys[idx] >= thr && m.keys[idx] != 0);
    int total;
    int pos = block_exclusive_scan<NT>(cnt, m.scan, &total);
    for (int idx = lo; idx < hi; ++idx) {
      if (m.keys[idx] >= thr && m.keys[idx] != 0) {
        if (pos < K2) m.mid[pos] = m.sorted[idx / g.page] * g.page + idx % g.page;
        ++pos;
      }
    }
  }
  __syncthreads();
  int count = take;
  int* mid = m.mid;

  // ---- hole fill (nfa_layer_batch_selector.py:545-566) -------------------------
  if (take < quota) {
    const int need = quota - take;
    // the holes are among the first `quota` ids of [lower, upper)
    for (int p = tid; p < quota; p += NT) m.win[p] = 0;
    __syncthreads();
    int in_win = 0;
    for (int i = tid; i < take; i += NT) {
      const int p = m.mid[i] - rg.lower;
      if (p < quota) { m.win[p] = 1; ++in_win; }
    }
    int cw;
    block_exclusive_scan<NT>(in_win, m.scan, &cw);
    const int ipt = (quota + NT - 1) / NT;
    const int lo = min(tid * ipt, quota), hi = min(lo + ipt, quota);
    int zeros = 0;
    for (int p = lo; p < hi; ++p) zeros += m.win[p] == 0;
    int ztotal;
    int zrank = block_exclusive_scan<NT>(zeros, m.scan, &ztotal);
    int keep = 0;
    for (int p = lo; p < hi; ++p) {
      if (m.win[p] == 0) { if (zrank < need) m.win[p] = 2; ++zrank; }
      keep += m.win[p] != 0;
    }
    int ktotal;
    int pos = block_exclusive_scan<NT>(keep, m.scan, &ktotal);
    for (int p = lo; p < hi; ++p) {
      if (m.win[p] != 0) m.mid2[pos++] = rg.lower + p;
    }
    // chosen tokens beyond the window follow all holes
    for (int i = cw + tid; i < take; i += NT) m.mid2[ktotal + (i - cw)] = m.mid[i];
    __syncthreads();
    count = ktotal + (take - cw);
    mid = m.mid2;
  }

  // ---- drop ids below the sink (only holes can be there), ascending already ----
  int below = 0;
  for (int i = tid; i < min(count, g.sink); i += NT) below += mid[i] < g.sink;
  int d0;
  block_exclusive_scan<NT>(below, m.scan, &d0);
  const int count_m = count - d0;
  if (S.middle != nullptr) {
    for (int i = tid; i < count_m; i += NT) S.middle[(size_t)row * K2 + i] = mid[d0 + i];
    if (tid == 0) S.middle_counts[row] = count_m;
  }

  // ---- union with sink and window ids (nfa_layer_batch_selector.py:1348-1437) --
  const int cap = g.max_blocks * g.page;
  const int sc = min(length, g.sink);
  const int count_s = min(length, g.sink + g.swa) - sc;
  const int s_lo = max(max(length - g.swa, 0), sc);
  const int s_hi = min(length - g.swa + count_s, cap);
  const int n_s = max(s_hi - s_lo, 0);
  const int total = sc + count_m + n_s;
  const int n_out = min(total, g.max_visible);
  int32_t* gout = S.gather + ((size_t)b * g.num_kv_heads + kv) * g.max_visible;
  for (int p = tid; p < n_out; p += NT) {
    int id;
    if (p < sc) id = p;
    else if (p < sc + count_m) id = mid[d0 + p - sc];
    else id = s_lo + (p - sc - count_m);
    const int lp = id / g.page;
    int ph = lp < g.max_blocks ? table[lp] : -1;
    if (ph < 0 || ph >= g.num_pages) {
      if (status) atomicOr(status, LODA_STATUS_BAD_PAGE);
      ph = g.num_pages - 1;   // PAD page: zeros, never out of bounds
    }
    gout[p] = ph * g.page + id % g.page;
  }
  if (tid == 0) {
    S.visible_lens[(size_t)b * g.num_kv_heads + kv] = n_out;
    if (total > g.max_visible && status) atomicOr(status, LODA_STATUS_TRUNCATED);
  }
}

constexpr int L2_NT = 512;

size_t l2_smem_bytes(const loda_geometry& g) {
  const size_t np_max = g.k_far + g.k_near + 2;
  return np_max * g.page * 4 + g.sub_dims * 4 + 3 * np_max * 4 + 2 * (size_t)g.level2_topk * 4 +
         (258 + 40 + 16) * 4 + g.level2_topk + 16;
}

cudaError_t launch_l2(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                      float scale, const loda_selection& S, uint32_t* status, cudaStream_t st) {
  const dim3 grid(B.batch * g.num_kv_heads);
  const size_t smem = l2_smem_bytes(g);
  cudaError_t e;
#define LODA_L2_CASE(DS)                                                                                 \
  case DS:                                                                                               \
    e = cudaFuncSetAttribute(l2_kernel<DS, L2_NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return e;                                                                      \
    e = launch_pdl(l2_kernel<DS, L2_NT>, grid, dim3(L2_NT), smem, st, g, L, B, (const bf16*)q, scale, S, \
                   status);                                                                              \
    if (e != cudaSuccess) return e;                                                                      \
    break;
  switch (g.sub_dims) {
    LODA_L2_CASE(16)
    LODA_L2_CASE(32)
    LODA_L2_CASE(64)
    default: return cudaErrorInvalidValue;
  }
#undef LODA_L2_CASE
  return cudaGetLastError();
}

}  // namespace loda
