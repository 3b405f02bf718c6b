// Fused L1 kernel: stream page metadata, score every page of the far pool with
// the min/max upper bound and every page of the near pool with the page mean,
// and keep the exact top-k pages of each pool (ties toward the lower page id).
//
// Restates _nfa_l1_scores_kernel (nfa_layer_batch_selector.py:174-354) and the
// packed-key top-k (nfa_layer_batch_selector.py:1473-1532, 1765-1793).
//
// Work split: grid = (ceil(max_blocks / P), batch * Hkv).  CTA (s, row) owns the
// P consecutive logical pages [s P, s P + P) of one (request, kv head) row: it
// stages their metadata (one contiguous run in HBM) into shared memory with
// 16-byte cp.async copies, scores one page per thread, keeps its best k_far /
// k_near keys with a radix select and appends them to the row's partial list.
// The last CTA of a row to finish (atomic ticket, no spinning) merges the
// partial lists, sorts the survivors and writes the page ids.
//
// Canonical arithmetic (must match the CPU oracle bit for bit): a length-d' dot
// is split into chunks of 8 dims summed left to right from 0.0f, chunk sums are
// combined by a balanced pairwise tree; bound = tree(min chunks) + tree(max
// chunks); per-head scores are rounded to bf16, summed over the GQA group in
// head order, divided by G and rounded to bf16.  bf16 x bf16 products are exact
// in fp32, so fmaf equals a separate multiply and add here.
#include "loda_append.cuh"

namespace loda {

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

// Merge the partial key lists of one row, keep the best k, write ids sorted by
// key descending followed by fillers (lowest page ids not selected).
template <int NT>
__device__ void merge_partials(const uint32_t* part, const int* cnt, int nsplit, int k, int kcap,
                               uint32_t* buf, uint32_t* sel, int* ids_sorted, int* hist, int* sh,
                               int32_t* out_ids, int32_t* out_n, int max_blocks) {
  const int tid = threadIdx.x;
  // counts of all splits in one round of loads, offsets by a short serial scan
  int* cnts = hist;            // [nsplit] (hist is free until the select below)
  int* offs = hist + 129;      // [nsplit]
  for (int s = tid; s < nsplit; s += NT) cnts[s] = min(__ldcg(cnt + s), kcap);
  __syncthreads();
  if (tid == 0) {
    int total = 0;
    for (int s = 0; s < nsplit; ++s) { offs[s] = total; total += cnts[s]; }
    sh[0] = total;
    sh[1] = 0;
  }
  __syncthreads();
  const int total = sh[0];
  // gather every partial key with independent loads
#pragma unroll 4
  for (int idx = tid; idx < nsplit * kcap; idx += NT) {
    const int s = idx / kcap, i = idx - s * kcap;
    if (i < cnts[s]) buf[offs[s] + i] = __ldcg(part + idx);
  }
  __syncthreads();
  int n = total;
  if (total > k) {
    const uint32_t thr = block_kth_largest<NT>(buf, total, k, hist);
    for (int i = tid; i < total; i += NT) {
      const uint32_t key = buf[i];
      if (key >= thr) sel[atomicAdd(&sh[1], 1)] = key;
    }
    n = k;
  } else {
    for (int i = tid; i < total; i += NT) sel[i] = buf[i];
  }
  __syncthreads();
  // rank by key (descending) and by page id (ascending); keys are unique
  for (int i = tid; i < n; i += NT) {
    const uint32_t key = sel[i];
    int rank = 0;
    for (int j = 0; j < n; ++j) rank += sel[j] > key;
    const int id = 0xFFFF - (int)(key & 0xFFFFu);
    out_ids[rank] = id;
  }
  __syncthreads();
  for (int i = tid; i < n; i += NT) {
    const int id = 0xFFFF - (int)(sel[i] & 0xFFFFu);
    int rank = 0;
    for (int j = 0; j < n; ++j) rank += (0xFFFF - (int)(sel[j] & 0xFFFFu)) < id;
    ids_sorted[rank] = id;
  }
  __syncthreads();
  // fillers: the j-th smallest page id that was not selected
  for (int j = tid; j < k - n; j += NT) {
    int c = j;
    for (int i = 0; i < n; ++i) {
      if (ids_sorted[i] <= c) ++c; else break;
    }
    out_ids[n + j] = min(c, max_blocks - 1);
  }
  if (tid == 0) *out_n = n;
  __syncthreads();
}

template <int DSUB, int P>
__global__ void __launch_bounds__(P) l1_kernel(loda_geometry g, loda_layer L, loda_batch B,
                                                const bf16* __restrict__ q, float scale,
                                                loda_selection out, L1Workspace ws, int nsplit,
                                                AppendArgs ap) {
  constexpr int NC = DSUB / 8;            // 8-dim chunks per statistic
  constexpr int CPR = 2 * NC;             // 16-byte chunks per min/max row
  constexpr int ROWB = 4 * DSUB + 16;     // padded row: conflict-free 16-byte reads
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* rows = smem;                                    // P * ROWB
  float* qhat = (float*)(smem + (size_t)P * ROWB);               // [G, DSUB] x3
  const int G = g.num_q_heads / g.num_kv_heads;
  float* qlow = qhat + G * DSUB;
  float* qhigh = qlow + G * DSUB;
  uint32_t* keys_f = (uint32_t*)(qhigh + G * DSUB);              // P
  uint32_t* keys_n = keys_f + P;                                 // P
  int* hist = (int*)(keys_n + P);                                // 258
  int* sh = hist + 258;                                          // 40

  const int tid = threadIdx.x;
  const int split = blockIdx.x, row = blockIdx.y;
  const int b = row / g.num_kv_heads, kv = row % g.num_kv_heads;
  pdl_wait();
  pdl_launch_dependents();
  if (split == nsplit) {
    // extra CTA of the row: the decode append.  It touches only the newest token
    // and its page, which lie in the sliding window and are read by neither L1
    // nor L2 of this step; the attention kernel runs after this launch completes.
    if (tid < 32) append_row<DSUB>(g, L, B, ap.k_new, ap.v_new, ap.slots, ap.status, b, kv, tid);
    return;
  }
  const bool active = B.active_req_ids[b] >= 0;
  const int length = active ? B.lengths[b] : 0;
  const int req = (int)B.valid_req_ids[b];
  const Regions rg = make_regions(g, length);
  const int p0 = split * P;

  // scaled, bf16-rounded query on the subspace (nfa_layer_batch_selector.py:943-963)
  for (int i = tid; i < G * DSUB; i += P) {
    const int j = i / DSUB, d = i % DSUB;
    const float qv = __bfloat162float(q[((size_t)b * g.num_q_heads + kv * G + j) * g.head_dim + sub_dim(g, d)]);
    const float qh = bf16r(__fmul_rn(qv, scale));
    qhat[i] = qh;
    qlow[i] = fminf(qh, 0.0f);
    qhigh[i] = fmaxf(qh, 0.0f);
  }

  // stage metadata rows of this CTA's pages
  const size_t pg0 = ((size_t)req * g.num_kv_heads + kv) * g.max_blocks;
  const unsigned char* mm_base = (const unsigned char*)L.page_mm + pg0 * (4 * DSUB);
  const unsigned char* sum_base = (const unsigned char*)L.page_sum + pg0 * (2 * DSUB);
  for (int c = tid; c < P * CPR; c += P) {
    const int pl = c / CPR, cc = c % CPR;
    const int page = p0 + pl;
    if (in_far_pool(rg, page)) {
      cp_async16(rows + (size_t)pl * ROWB + cc * 16, mm_base + (size_t)page * (4 * DSUB) + cc * 16, true);
    } else if (cc < NC && in_near_pool(rg, page)) {
      cp_async16(rows + (size_t)pl * ROWB + cc * 16, sum_base + (size_t)page * (2 * DSUB) + cc * 16, true);
    }
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  // one page per thread
  const int page = p0 + tid;
  uint32_t key_f = 0, key_n = 0;
  const unsigned char* myrow = rows + (size_t)tid * ROWB;
  const float gf = (float)G;
  if (in_far_pool(rg, page)) {
    float kmin[DSUB], kmax[DSUB];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      unpack8(*(const uint4*)(myrow + c * 16), *(float(*)[8])(kmin + 8 * c));
      unpack8(*(const uint4*)(myrow + (NC + c) * 16), *(float(*)[8])(kmax + 8 * c));
    }
    float acc = 0.0f;
#pragma unroll 1
    for (int j = 0; j < G; ++j) {
      const float mm = __fadd_rn(dot_chunks<DSUB>(kmin, qlow + j * DSUB), dot_chunks<DSUB>(kmax, qhigh + j * DSUB));
      acc = __fadd_rn(acc, bf16r(mm));
    }
    const float score = bf16r(__fdiv_rn(acc, gf));
    const uint32_t o = ord16(score);
    if (o != ORD16_NEG_INF) key_f = (o << 16) | (uint32_t)(0xFFFF - page);
  } else if (in_near_pool(rg, page)) {
    float kavg[DSUB];
    const float bsf = (float)g.page;
#pragma unroll
    for (int c = 0; c < NC; ++c) unpack8(*(const uint4*)(myrow + c * 16), *(float(*)[8])(kavg + 8 * c));
#pragma unroll
    for (int i = 0; i < DSUB; ++i) kavg[i] = bf16r(__fdiv_rn(kavg[i], bsf));
    float acc = 0.0f;
#pragma unroll 1
    for (int j = 0; j < G; ++j) acc = __fadd_rn(acc, bf16r(dot_chunks<DSUB>(kavg, qhat + j * DSUB)));
    const float score = bf16r(__fdiv_rn(acc, gf));
    const uint32_t o = ord16(score);
    if (o != ORD16_NEG_INF) key_n = (o << 16) | (uint32_t)(0xFFFF - page);
  }
  keys_f[tid] = key_f;
  keys_n[tid] = key_n;
  if (tid == 0) { sh[2] = 0; sh[3] = 0; }
  const int nf = __syncthreads_count(key_f != 0);
  const int nn = __syncthreads_count(key_n != 0);

  const size_t pslot = (size_t)row * nsplit + split;
  if (nf > 0) {
    const uint32_t thr = nf > g.k_far ? block_kth_largest<P>(keys_f, P, g.k_far, hist) : 1u;
    if (key_f >= thr && key_f != 0) ws.part_far[pslot * g.k_far + atomicAdd(&sh[2], 1)] = key_f;
  }
  if (nn > 0) {
    const uint32_t thr = nn > g.k_near ? block_kth_largest<P>(keys_n, P, g.k_near, hist) : 1u;
    if (key_n >= thr && key_n != 0) ws.part_near[pslot * g.k_near + atomicAdd(&sh[3], 1)] = key_n;
  }
  if (tid == 0) {
    ws.cnt_far[pslot] = min(nf, g.k_far);
    ws.cnt_near[pslot] = min(nn, g.k_near);
  }

  // last CTA of the row merges
  __threadfence();
  __syncthreads();
  if (tid == 0) sh[4] = (atomicAdd(ws.ticket + row, 1) == nsplit - 1);
  __syncthreads();
  if (!sh[4]) return;
  __threadfence();
  uint32_t* buf = (uint32_t*)rows;                    // nsplit * k entries fit in the staging area
  uint32_t* selk = keys_f;                            // k <= P
  int* ids_sorted = (int*)keys_n;
  merge_partials<P>(ws.part_far + (size_t)row * nsplit * g.k_far, ws.cnt_far + (size_t)row * nsplit,
                    nsplit, g.k_far, g.k_far, buf, selk, ids_sorted, hist, sh,
                    out.i_far + (size_t)row * g.k_far, out.n_far + row, g.max_blocks);
  merge_partials<P>(ws.part_near + (size_t)row * nsplit * g.k_near, ws.cnt_near + (size_t)row * nsplit,
                    nsplit, g.k_near, g.k_near, buf, selk, ids_sorted, hist, sh,
                    out.i_near + (size_t)row * g.k_near, out.n_near + row, g.max_blocks);
  if (tid == 0) ws.ticket[row] = 0;
}

constexpr int L1_P = 512;

size_t l1_smem_bytes(const loda_geometry& g) {
  const int G = g.num_q_heads / g.num_kv_heads;
  return (size_t)L1_P * (4 * g.sub_dims + 16) + (size_t)3 * G * g.sub_dims * 4 + (size_t)2 * L1_P * 4 +
         (258 + 40) * 4;
}

int l1_nsplit(const loda_geometry& g) { return (g.max_blocks + L1_P - 1) / L1_P; }

cudaError_t launch_l1(const loda_geometry& g, const loda_layer& L, const loda_batch& B, const void* q,
                      float scale, const loda_selection& out, const L1Workspace& ws, const AppendArgs& ap,
                      cudaStream_t st) {
  const int nsplit = l1_nsplit(g);
  const dim3 grid(nsplit + (ap.enabled ? 1 : 0), B.batch * g.num_kv_heads);
  const size_t smem = l1_smem_bytes(g);
  cudaError_t e = cudaSuccess;
#define LODA_L1_CASE(DS)                                                                            \
  case DS: {                                                                                        \
    static bool attr_set = false;                                                                   \
    if (!attr_set) {                                                                                \
      e = cudaFuncSetAttribute(l1_kernel<DS, L1_P>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); \
      if (e != cudaSuccess) return e;                                                               \
      attr_set = true;                                                                              \
    }                                                                                               \
    e = launch_pdl(l1_kernel<DS, L1_P>, grid, dim3(L1_P), smem, st, g, L, B, (const bf16*)q, scale, out, ws, \
                   nsplit, ap);                                                                     \
    if (e != cudaSuccess) return e;                                                                 \
  } break;
  switch (g.sub_dims) {
    LODA_L1_CASE(16)
    LODA_L1_CASE(32)
    LODA_L1_CASE(64)
    default: return cudaErrorInvalidValue;
  }
#undef LODA_L1_CASE
  return cudaGetLastError();
}

}  // namespace loda
