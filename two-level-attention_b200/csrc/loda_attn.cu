// Split-K gather attention over the selected tokens of the paged KV cache.
//
// Restates sparse_paged_attention_gather (sparse_attn/ops/paged_region_kernels.py:
// 800-1041; grouped kernel :251-363, split kernel :367-529, combine :578-607):
// for query row t, kv head h and its GQA group, exact softmax attention over
// the physical slots gather[req, h, 0:visible_lens[req, h]]; slots < 0 are
// skipped; an empty list gives zeros; rows with query_to_req < 0 give zeros.
//
// Grid = (nsplit, Hkv, n_query).  CTA (s, h, t) owns the balanced chunk
// [floor(s n / nsplit), floor((s + 1) n / nsplit)) of the list.  K and V rows
// are staged by physical slot with 16-byte cp.async copies (one 256-byte row per
// 16 lanes) into padded shared-memory tiles of 64 tokens; each of the 4 warps
// owns 16 tokens of a tile: S = Q K^T with mma.sync m16n8k16 (M = the GQA group
// padded to 16 rows, operands bf16, fp32 accumulate), fp32 online softmax in the
// exp2 domain, O += P V with P rounded to bf16.  Warps, then splits, are merged
// by log-sum-exp in a fixed order.  The splits of a (t, h) pair form one thread
// block cluster: after a cluster barrier each CTA reduces its slice of the
// output columns straight out of its peers' shared memory (DSMEM), so the
// partials never touch global memory.  Where a cluster of that size cannot be
// launched, and for the static-scratch entry point, the partials go through
// global scratch and the last CTA of the pair to finish (atomic ticket, no
// spinning) performs the merge.
#include <cooperative_groups.h>

#include <cstdio>
#include <cstdlib>

#include "loda_attn.cuh"
#include "loda_common.cuh"

namespace loda {

using bf16 = __nv_bfloat16;
namespace cg = cooperative_groups;

constexpr int ATT_TILE = 64;
constexpr int ATT_WARPS = 4;
constexpr int ATT_NT = 32 * ATT_WARPS;
constexpr int ATT_MAX_SPLIT = 16;
constexpr int ATT_STAGES = 3;
#ifndef LODA_ATTN_CTAS_PER_SM
#define LODA_ATTN_CTAS_PER_SM 1
#endif

LODA_PHASE_STORAGE(attn)

template <int D, int DV, bool CLUSTER>
__global__ void __launch_bounds__(ATT_NT) attn_kernel(
    loda_geometry g, loda_layer L, const bf16* __restrict__ q, const int32_t* gather,
    const int32_t* visible_lens, const int32_t* query_to_req,
    int n_req_rows, float scale_log2, bf16* __restrict__ out, float* __restrict__ lse, AttnWorkspace ws,
    int nsplit, int chained, int identity) {
  constexpr int KSTR = D + 8, VSTR = DV + 8;   // padded rows: conflict-free ldmatrix
  constexpr int KSTEPS = D / 16, NTV = DV / 8;
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* Ks = (bf16*)smem;                                   // [STAGES][TILE][KSTR]
  bf16* Vs = Ks + ATT_STAGES * ATT_TILE * KSTR;             // [STAGES][TILE][VSTR]
  int* slot_s = (int*)(Vs + ATT_STAGES * ATT_TILE * VSTR);  // [STAGES][TILE] physical slot of each staged token
  float* wm = (float*)(slot_s + ATT_STAGES * ATT_TILE);     // [WARPS][16]
  float* wz = wm + ATT_WARPS * 16;                 // [WARPS][16]
  int* sh = (int*)(wz + ATT_WARPS * 16);           // 4
  float* fm = (float*)(sh + 4);                    // [16] merged max of this CTA
  float* fz = fm + 16;                             // [16] merged sum of this CTA
  float* wo = (float*)Vs;                          // [WARPS][G][DV], after the last tile (V stages consumed)

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, kv = blockIdx.y, t = blockIdx.z;
  const int G = g.num_q_heads / g.num_kv_heads;
  const int page_log2 = 31 - __clz(g.page);
  const int cta_id = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  LODA_PHASE(attn, cta_id, 0);
  // Q fragments: A operand, rows = heads of the group (zero beyond G).  When this launch is
  // chained behind the selector launches of the same step (which read the query too, after
  // their own wait), the query was complete before they could release this launch, and it is
  // read before the wait; a launch that stands alone reads it after.
  uint32_t qa[KSTEPS][4];
  auto load_q = [&]() { attn_load_q<D>(qa, q + ((size_t)t * g.num_q_heads + kv * G) * D, G, lane); };
  if (chained) load_q();
  pdl_wait();
#if LODA_PDL_TRIGGER == 0
  pdl_launch_dependents();
#endif
  if (!chained) load_q();
  LODA_PHASE(attn, cta_id, 1);
  // The lists and their lengths are written by the launch this one may be chained behind: they
  // are read with L2-coherent loads placed after the wait above, through pointers the compiler
  // may not treat as read-only (declared const __restrict__, their loads were hoisted above
  // the wait and saw the lists of the step before).
  int req = __ldcg(query_to_req + t);
  // identity: the caller's contract is one query per batch row (query_to_req[t] == t, or < 0 for a row of zeros);
  // any other value gives a row of zeros here as in the one-launch decode step
  if (identity && req != t) req = -1;
  int n = 0;
  if (req >= 0 && req < n_req_rows) n = min(max(__ldcg(visible_lens + (size_t)req * g.num_kv_heads + kv), 0), g.max_visible);
  const int c0 = (int)(((long long)split * n) / nsplit);
  const int c1 = (int)(((long long)(split + 1) * n) / nsplit);
  const int32_t* list = gather + ((size_t)max(req, 0) * g.num_kv_heads + kv) * g.max_visible;

  LODA_PHASE(attn, cta_id, 2);
  float oacc[NTV][4];
#pragma unroll
  for (int i = 0; i < NTV; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0f; }
  float m_run[2] = {-INFINITY, -INFINITY}, z_run[2] = {0.0f, 0.0f};   // rows lane/4 and lane/4 + 8

  // Staging: 16-byte chunk (row kr + k * RPI, column kc) of every tile belongs to this
  // thread, so it reads the gather-list entries of its own rows into registers and needs
  // no shared slot table to issue the copies.  ATT_STAGES tiles are in flight: all the
  // lists of the first tiles are fetched in one round of loads, then all their copies are
  // issued; after the math of tile i its stage is refilled with tile i + ATT_STAGES, whose
  // list entries were fetched one iteration earlier.
  constexpr int KCH = D / 8, VCH = DV / 8;
  static_assert(KCH == VCH, "K and V rows are staged by the same threads");
  constexpr int RPI = ATT_NT / KCH, NIT = ATT_TILE / RPI;
  static_assert(ATT_NT % KCH == 0 && ATT_TILE % RPI == 0, "tile shape");
  const int kr = tid / KCH, kc = tid % KCH;
  const int slot_end = g.num_pages * g.page;
  const int ntiles = (c1 - c0 + ATT_TILE - 1) / ATT_TILE;
  auto fetch_slots = [&](int (&sl)[NIT], int tile) {
    const int base = c0 + tile * ATT_TILE;
#pragma unroll
    for (int k = 0; k < NIT; ++k) {
      const int idx = base + kr + k * RPI;
      const int s = (tile < ntiles && idx < c1) ? __ldcg(list + idx) : -1;
      sl[k] = s >= slot_end ? -1 : s;
    }
  };
  auto issue = [&](int stage, const int (&sl)[NIT], int tile) {
    if (tile < ntiles) {
      bf16* Kb = Ks + stage * ATT_TILE * KSTR;
      bf16* Vb = Vs + stage * ATT_TILE * VSTR;
      int* sb = slot_s + stage * ATT_TILE;
#pragma unroll
      for (int k = 0; k < NIT; ++k) {
        const int r = kr + k * RPI, s = sl[k];
        // page is a power of two: slot -> pool row without a division
        const long long off = s >= 0 ? ((long long)(s >> page_log2) * g.num_kv_heads + kv) * g.page + (s & (g.page - 1)) : 0;
        cp_async16(Kb + r * KSTR + kc * 8, (const bf16*)L.pool_k + off * D + kc * 8, s >= 0);
        cp_async16(Vb + r * VSTR + kc * 8, (const bf16*)L.pool_v + off * DV + kc * 8, s >= 0);
        if (kc == 0) sb[r] = s;
      }
    }
    cp_async_commit();     // one group per tile index, empty past the last tile
  };
  int nxt[NIT];
  {
    int sl[ATT_STAGES][NIT];
#pragma unroll
    for (int s = 0; s < ATT_STAGES; ++s) fetch_slots(sl[s], s);
#pragma unroll
    for (int s = 0; s < ATT_STAGES; ++s) issue(s, sl[s], s);
  }
  fetch_slots(nxt, ATT_STAGES);
  LODA_PHASE(attn, cta_id, 3);
  int stage = 0;
  for (int it = 0; it < ntiles; ++it) {
    const int ntok = min(ATT_TILE, c1 - c0 - it * ATT_TILE);
    cp_async_wait<ATT_STAGES - 1>();
    __syncthreads();
    if (it == 0) { LODA_PHASE(attn, cta_id, 4); }
    const bf16* Kt = Ks + stage * ATT_TILE * KSTR;
    const bf16* Vt = Vs + stage * ATT_TILE * VSTR;
    const int* slot_t = slot_s + stage * ATT_TILE;

    const int tok0 = warp * 16;
    if (tok0 < ntok) {
      attn_warp_step<D, DV>(Kt, Vt, slot_t, tok0, ntok, qa, scale_log2, oacc, m_run, z_run);
    }
    __syncthreads();   // the stage is free: refill it
    issue(stage, nxt, it + ATT_STAGES);
    fetch_slots(nxt, it + ATT_STAGES + 1);
    stage = stage + 1 == ATT_STAGES ? 0 : stage + 1;
  }
  cp_async_wait<0>();

  // ---- merge the warps of this CTA (fixed order) -------------------------------
#if LODA_PDL_TRIGGER == 1 || LODA_PDL_TRIGGER == 3
  pdl_launch_dependents();
#endif
  LODA_PHASE(attn, cta_id, 5);
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
  const size_t pair = (size_t)t * g.num_kv_heads + kv;
  float* fo = (float*)Ks;   // [G][DV] merged output of this CTA (the K tile has been consumed)
  for (int e = tid; e < G * DV; e += ATT_NT) {
    const int gi = e / DV, dv = e % DV;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, wm[w * 16 + gi]);
    float z = 0.0f, o = 0.0f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < ATT_WARPS; ++w) {
        const float a = exp2f(wm[w * 16 + gi] - M);
        z += wz[w * 16 + gi] * a;
        o += wo[(w * G + gi) * DV + dv] * a;
      }
    }
    if (nsplit == 1) {
      out[((size_t)t * g.num_q_heads + kv * G + gi) * DV + dv] = __float2bfloat16_rn(z == 0.0f ? 0.0f : o / z);
      if (lse != nullptr && dv == 0) {
        lse[((size_t)t * g.num_q_heads + kv * G + gi) * 2 + 0] = M;
        lse[((size_t)t * g.num_q_heads + kv * G + gi) * 2 + 1] = z;
      }
    } else if (CLUSTER) {
      fo[e] = o;
      if (dv == 0) { fm[gi] = M; fz[gi] = z; }
    } else {
      const size_t ps = pair * nsplit + split;
      ws.part_o[(ps * G + gi) * DV + dv] = o;
      if (dv == 0) { ws.part_m[ps * G + gi] = M; ws.part_z[ps * G + gi] = z; }
    }
  }
  LODA_PHASE(attn, cta_id, 6);
  if (nsplit == 1) return;
  if constexpr (CLUSTER) {
    // the nsplit CTAs of this (t, kv) pair are one cluster (rank == split): each
    // reduces its slice of the G * DV outputs from every peer's shared memory
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    LODA_PHASE(attn, cta_id, 7);
    const int per = (G * DV + nsplit - 1) / nsplit;
    const int e_end = min((split + 1) * per, G * DV);
#pragma unroll 1
    for (int e = split * per + tid; e < e_end; e += ATT_NT) {      // a slice may hold more elements than the CTA has threads
      const int gi = e / DV, dv = e % DV;
      float pm[ATT_MAX_SPLIT], pz[ATT_MAX_SPLIT], po[ATT_MAX_SPLIT];
#pragma unroll
      for (int s = 0; s < ATT_MAX_SPLIT; ++s) {
        if (s < nsplit) {
          pm[s] = cluster.map_shared_rank(fm, s)[gi];
          pz[s] = cluster.map_shared_rank(fz, s)[gi];
          po[s] = cluster.map_shared_rank(fo, s)[e];
        } else {
          pm[s] = -INFINITY; pz[s] = 0.0f; po[s] = 0.0f;
        }
      }
      float M = -INFINITY;
#pragma unroll
      for (int s = 0; s < ATT_MAX_SPLIT; ++s) M = fmaxf(M, pm[s]);
      float z = 0.0f, o = 0.0f;
      if (M != -INFINITY) {
#pragma unroll
        for (int s = 0; s < ATT_MAX_SPLIT; ++s) {
          const float a = exp2f(pm[s] - M);
          z += pz[s] * a;
          o += po[s] * a;
        }
      }
      out[((size_t)t * g.num_q_heads + kv * G + gi) * DV + dv] = __float2bfloat16_rn(z == 0.0f ? 0.0f : o / z);
      if (lse != nullptr && dv == 0) {
        lse[((size_t)t * g.num_q_heads + kv * G + gi) * 2 + 0] = M;
        lse[((size_t)t * g.num_q_heads + kv * G + gi) * 2 + 1] = z;
      }
    }
    cluster.sync();   // nobody leaves while a peer may still read its shared memory
    LODA_PHASE(attn, cta_id, 8);
    return;
  }

  // ---- last CTA of the (t, kv) pair merges the splits in split order -------------
  __threadfence();
  __syncthreads();
  if (tid == 0) sh[0] = (atomicAdd(ws.ticket + pair, 1) == nsplit - 1);
  __syncthreads();
  LODA_PHASE(attn, cta_id, 7);
  if (!sh[0]) return;
  __threadfence();
  // all (m, z) pairs in one round of loads, weights once per (split, head), then
  // every output element sums its splits in split order from independent loads
  float* sm_m = wo;                          // [nsplit * G]
  float* sm_z = wo + ATT_MAX_SPLIT * 16;     // [nsplit * G]
  float* sm_w = wo + 2 * ATT_MAX_SPLIT * 16; // [nsplit * G] weight of each split
  float* sm_zt = wo + 3 * ATT_MAX_SPLIT * 16;  // [G]
  for (int i = tid; i < nsplit * G; i += ATT_NT) {
    sm_m[i] = __ldcg(ws.part_m + pair * nsplit * G + i);
    sm_z[i] = __ldcg(ws.part_z + pair * nsplit * G + i);
  }
  __syncthreads();
  if (tid < G) {
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, sm_m[s * G + tid]);
    float z = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
      const float a = M == -INFINITY ? 0.0f : exp2f(sm_m[s * G + tid] - M);
      sm_w[s * G + tid] = a;
      z += sm_z[s * G + tid] * a;
    }
    sm_zt[tid] = z;
    if (lse != nullptr) {
      lse[((size_t)t * g.num_q_heads + kv * G + tid) * 2 + 0] = M;
      lse[((size_t)t * g.num_q_heads + kv * G + tid) * 2 + 1] = z;
    }
  }
  __syncthreads();
  const float* po = ws.part_o + pair * nsplit * G * DV;
  for (int e = tid; e < G * DV / 4; e += ATT_NT) {
    const int gi = e / (DV / 4), dv = (e % (DV / 4)) * 4;
    float4 v[ATT_MAX_SPLIT];
#pragma unroll
    for (int s = 0; s < ATT_MAX_SPLIT; ++s)
      v[s] = s < nsplit ? __ldcg((const float4*)(po + ((size_t)s * G + gi) * DV + dv)) : make_float4(0, 0, 0, 0);
    float4 o = make_float4(0, 0, 0, 0);
#pragma unroll
    for (int s = 0; s < ATT_MAX_SPLIT; ++s) {
      if (s < nsplit) {
        const float a = sm_w[s * G + gi];
        o.x += v[s].x * a; o.y += v[s].y * a; o.z += v[s].z * a; o.w += v[s].w * a;
      }
    }
    const float z = sm_zt[gi];
    const float inv = z == 0.0f ? 0.0f : 1.0f / z;
    __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * inv, o.y * inv);
    __nv_bfloat162 hi = __floats2bfloat162_rn(o.z * inv, o.w * inv);
    uint2 packed;
    packed.x = *(uint32_t*)&lo;
    packed.y = *(uint32_t*)&hi;
    *(uint2*)(out + ((size_t)t * g.num_q_heads + kv * G + gi) * DV + dv) = packed;
  }
  LODA_PHASE(attn, cta_id, 8);
  if (tid == 0) ws.ticket[pair] = 0;
}

size_t attn_smem_bytes(const loda_geometry& g) {
  // the per-warp partial outputs [WARPS][G][DV] fp32 reuse the V stages (G <= 16 fits)
  return ATT_STAGES * ((size_t)ATT_TILE * (g.head_dim + 8) * 2 + (size_t)ATT_TILE * (g.head_dim_v + 8) * 2 + ATT_TILE * 4) +
         2 * ATT_WARPS * 16 * 4 + 16 + 2 * 16 * 4;
}

// power-of-two split count: no more splits than it takes to give every SM a CTA (a split
// costs a prologue and a merge, about as much as streaming 300 tokens), at least one
// 64-token tile per split, at most ATT_MAX_SPLIT (the largest cluster)
int attn_nsplit(const loda_geometry& g, int n_query) {
  const int pairs = n_query * g.num_kv_heads;
  const int want = (LODA_ATTN_CTAS_PER_SM * device_sm_count() + pairs - 1) / pairs;
  const int by_len = (g.max_visible + ATT_TILE - 1) / ATT_TILE;
  int ns = 1;
  while (ns < want && ns * 2 <= by_len && ns * 2 <= ATT_MAX_SPLIT) ns *= 2;
  return ns;
}

template <int D, int DV>
static cudaError_t launch_attn_dims(const loda_geometry& g, const loda_layer& L, const void* q,
                                    const int32_t* gather, const int32_t* visible_lens,
                                    const int32_t* query_to_req, int n_query, int n_req_rows, float scale_log2,
                                    void* out, float* lse, const AttnWorkspace& ws, bool allow_cluster,
                                    bool chained, bool identity, cudaStream_t st) {
  const int nsplit = attn_nsplit(g, n_query);
  const dim3 grid(nsplit, g.num_kv_heads, n_query);
  const size_t smem = attn_smem_bytes(g);
  static bool cluster_refused[64] = {};     // per device: set if this GPU / driver refuses the cluster launch
  const int dev = device_ordinal();
  const bool cluster_ok = dev >= 0 && dev < 64 && !cluster_refused[dev];
  cudaError_t e;
  if (allow_cluster && cluster_ok && nsplit > 1) {
    auto kernel = attn_kernel<D, DV, true>;
    e = set_kernel_smem(kernel, smem);
    if (e == cudaSuccess && nsplit > 8)
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(ATT_NT);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = st;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      attr[1].id = cudaLaunchAttributeClusterDimension;
      attr[1].val.clusterDim.x = nsplit;
      attr[1].val.clusterDim.y = 1;
      attr[1].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 2;
      e = cudaLaunchKernelEx(&cfg, kernel, g, L, (const bf16*)q, gather, visible_lens, query_to_req, n_req_rows,
                             scale_log2, (bf16*)out, lse, ws, nsplit, (int)chained, (int)identity);
    }
    if (e == cudaSuccess) return cudaSuccess;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(st, &cap);
    if (cap != cudaStreamCaptureStatusNone) return e;   // cannot retry inside a capture
    (void)cudaGetLastError();
    cluster_refused[dev] = true;
  }
  auto kernel = attn_kernel<D, DV, false>;
  e = set_kernel_smem(kernel, smem);
  if (e != cudaSuccess) return e;
  return launch_pdl(kernel, grid, dim3(ATT_NT), smem, st, g, L, (const bf16*)q, gather, visible_lens, query_to_req,
                    n_req_rows, scale_log2, (bf16*)out, lse, ws, nsplit, (int)chained, (int)identity);
}

cudaError_t launch_attn(const loda_geometry& g, const loda_layer& L, const void* q, const int32_t* gather,
                        const int32_t* visible_lens, const int32_t* query_to_req, int n_query,
                        int n_req_rows, float scale, void* out, float* lse, const AttnWorkspace& ws,
                        bool allow_cluster, bool chained, bool identity, cudaStream_t st) {
  if (n_query <= 0) return cudaSuccess;
  const float scale_log2 = scale * 1.4426950408889634f;
  if (g.head_dim == 128 && g.head_dim_v == 128)
    return launch_attn_dims<128, 128>(g, L, q, gather, visible_lens, query_to_req, n_query, n_req_rows, scale_log2,
                                      out, lse, ws, allow_cluster, chained, identity, st);
  if (g.head_dim == 64 && g.head_dim_v == 64)
    return launch_attn_dims<64, 64>(g, L, q, gather, visible_lens, query_to_req, n_query, n_req_rows, scale_log2,
                                    out, lse, ws, allow_cluster, chained, identity, st);
  return cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// Gather attention for callers that cannot hand the library any scratch memory
// ---------------------------------------------------------------------------
// Some hosts of this library cannot call cudaMalloc (or any allocating routine)
// at the point where they need attention: a plugin running inside another
// framework's memory plan, a process whose device memory was carved up at start,
// code running under a "no allocation" guard.  For them the split-K partials and
// the tickets live in the fixed array below, which every GPU that loads the
// library carries until the process exits (about 4.1 MiB).
constexpr int ATT_STATIC_MAX_PAIRS = 64;   // n_query * num_kv_heads
constexpr int ATT_STATIC_MAX_G = 8;        // query heads per kv head
constexpr int ATT_STATIC_MAX_DV = 128;
constexpr size_t ATT_STATIC_TICKET_BYTES = 256;                                     // 64 ints
constexpr size_t ATT_STATIC_MZ_BYTES = (size_t)ATT_STATIC_MAX_PAIRS * ATT_MAX_SPLIT * ATT_STATIC_MAX_G * 4;
constexpr size_t ATT_STATIC_O_BYTES = ATT_STATIC_MZ_BYTES * ATT_STATIC_MAX_DV;
constexpr size_t ATT_STATIC_BYTES = ATT_STATIC_TICKET_BYTES + 2 * ATT_STATIC_MZ_BYTES + ATT_STATIC_O_BYTES;

static __device__ __align__(256) unsigned char g_attn_static_scratch[ATT_STATIC_BYTES];

int report_error(int code, const char* message);
int check_gather_attend_args(const loda_geometry*, const loda_layer*, const void*, const int32_t*,
                             const int32_t*, const int32_t*, int32_t, int32_t, const void*);

// Device address of the static scratch on the current device.  The array's name
// is only a host-side handle; the address a kernel can use comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
static int static_scratch_address(unsigned char** out) {
  constexpr int kMaxDevices = 64;
  static unsigned char* address[kMaxDevices] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return report_error(LODA_ERR_LAUNCH, "cudaGetDevice failed or device ordinal >= 64");
  if (address[dev] == nullptr) {
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_attn_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      char msg[160];
      snprintf(msg, sizeof(msg), "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
      return report_error(LODA_ERR_LAUNCH, msg);
    }
    address[dev] = p;
  }
  *out = address[dev];
  return LODA_OK;
}

}  // namespace loda

extern "C" int loda_gather_attend_static(const loda_geometry* g, const loda_layer* layer, const void* q,
                                         const int32_t* gather, const int32_t* visible_lens,
                                         const int32_t* query_to_req, int32_t n_query, int32_t n_req_rows,
                                         float scale, void* out, void* stream) {
  using namespace loda;
  const int rc = check_gather_attend_args(g, layer, q, gather, visible_lens, query_to_req, n_query, n_req_rows, out);
  if (rc != LODA_OK) return rc;
  if (n_query == 0) return LODA_OK;
  const int G = g->num_q_heads / g->num_kv_heads;
  if (n_query * g->num_kv_heads > ATT_STATIC_MAX_PAIRS || G > ATT_STATIC_MAX_G || g->head_dim_v > ATT_STATIC_MAX_DV) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "static-scratch gather attention is limited to n_query * num_kv_heads <= %d, group <= %d, "
             "head_dim_v <= %d (got %d, %d, %d); use loda_gather_attend with a workspace",
             ATT_STATIC_MAX_PAIRS, ATT_STATIC_MAX_G, ATT_STATIC_MAX_DV, n_query * g->num_kv_heads, G, g->head_dim_v);
    return report_error(LODA_ERR_UNSUPPORTED, msg);
  }
  unsigned char* base = nullptr;
  const int rc2 = static_scratch_address(&base);
  if (rc2 != LODA_OK) return rc2;
  AttnWorkspace ws;
  ws.ticket = (int*)base;
  ws.part_m = (float*)(base + ATT_STATIC_TICKET_BYTES);
  ws.part_z = (float*)(base + ATT_STATIC_TICKET_BYTES + ATT_STATIC_MZ_BYTES);
  ws.part_o = (float*)(base + ATT_STATIC_TICKET_BYTES + 2 * ATT_STATIC_MZ_BYTES);
  // the array keeps whatever the previous call left: the tickets must start at zero
  cudaError_t e = cudaMemsetAsync(ws.ticket, 0, ATT_STATIC_TICKET_BYTES, (cudaStream_t)stream);
  if (e == cudaSuccess)
    e = launch_attn(*g, *layer, q, gather, visible_lens, query_to_req, n_query, n_req_rows, scale, out, nullptr, ws,
                    /*allow_cluster=*/false, /*chained=*/false, /*identity=*/false, (cudaStream_t)stream);   // this entry point exists for the scratch path
  if (e != cudaSuccess) {
    char msg[160];
    snprintf(msg, sizeof(msg), "gather_attend_static: %s", cudaGetErrorString(e));
    return report_error(LODA_ERR_LAUNCH, msg);
  }
  return LODA_OK;
}
